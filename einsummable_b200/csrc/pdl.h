// Programmatic dependent launch between consecutive kernels of one lane of a program.
//
// A kernel launched with the attribute may be scheduled while the kernel before it in the stream is
// still running; its blocks stop at `griddepcontrol.wait` until that kernel has completed and its
// writes are visible.  Every kernel of this library therefore starts with ES_PDL_PROLOGUE() before it
// touches global memory (a no-op for ordinary launches), which lets the program executor hide the
// launch latency of the small ops that make up the dependency chains of a partitioned graph.  Short
// kernels also release their dependents at once (`griddepcontrol.launch_dependents`): those are then
// resident and waiting when the kernel ends.  The long persistent contraction kernel only waits.
#pragma once
#include <cuda_runtime.h>

#include <utility>

#include "common.h"

#define ES_PDL_WAIT() asm volatile("griddepcontrol.wait;" ::: "memory")
#define ES_PDL_PROLOGUE()                                                                          \
    do {                                                                                           \
        asm volatile("griddepcontrol.launch_dependents;");                                         \
        asm volatile("griddepcontrol.wait;" ::: "memory");                                         \
    } while (0)

namespace es {

// Set by the program executor around the launches of an op that may overlap the end of the op before it
// on its lane; the launch helpers below then ask for programmatic stream serialization.
bool& pdl_launch_flag();

struct pdl_scope_t {
    bool saved;
    explicit pdl_scope_t(bool on) : saved(pdl_launch_flag()) { pdl_launch_flag() = on; }
    ~pdl_scope_t() { pdl_launch_flag() = saved; }
};

template <typename... KArgs, typename... Args>
inline void launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (pdl_launch_flag()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    ES_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...));
}

} // namespace es
