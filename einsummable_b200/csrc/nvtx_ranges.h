// Opt-in NVTX ranges around the library's launches (ES_B200_NVTX=1): one range per launch of the
// C ABI and per op of a program, named by the kernel kind and the einsummable string, so that a
// timeline tool shows memgraph nodes instead of anonymous kernels.  nvtx3 is header-only and does
// nothing unless a tool is attached.  The reference has no counterpart (its timetracker hooks,
// src/engine/cpu/kernel_executor.cc:459-591, are host-side and commented out).
#pragma once
#include <nvtx3/nvToolsExt.h>

#include <cstdlib>
#include <string>

namespace es {

inline bool nvtx_on()
{
    static bool const on = [] {
        char const* v = std::getenv("ES_B200_NVTX");
        return v && std::string(v) != "0";
    }();
    return on;
}

struct nvtx_range_t {
    bool on;
    explicit nvtx_range_t(char const* name) : on(nvtx_on())
    {
        if (on) nvtxRangePushA(name);
    }
    explicit nvtx_range_t(std::string const& name) : nvtx_range_t(name.c_str()) {}
    ~nvtx_range_t()
    {
        if (on) nvtxRangePop();
    }
    nvtx_range_t(nvtx_range_t const&) = delete;
    nvtx_range_t& operator=(nvtx_range_t const&) = delete;
};

} // namespace es
