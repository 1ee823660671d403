// Test infrastructure, not product code.
//
// Stand-in for cutensor.h (cuTENSOR is not installed here): src/engine/gpu/utility.h:5 includes it for
// the one error-reporting helper below; the drop-in kernel manager uses no cuTENSOR at all.
#pragma once
typedef int cutensorStatus_t;
#define CUTENSOR_STATUS_SUCCESS 0
inline char const* cutensorGetErrorString(cutensorStatus_t)
{
    return "cuTENSOR is not part of this build";
}
