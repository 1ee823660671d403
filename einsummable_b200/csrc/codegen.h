// Kernel planner + CUDA source generator for elementwise and reduction
// einsummables.  One fused kernel is generated per (join tree, index pattern,
// shape, dtypes); it replaces the reference's chain of one cuTENSOR call per
// simple op with temporaries in workspace
// (src/engine/gpu/gpu_kernel_manager.cc:1951-2079) and its one-thread-per-row
// reduction kernels (src/engine/gpu/cuda_kernels.cu:728-877).
#pragma once
#include <string>
#include <vector>

#include "einsum.h"

namespace es {

struct launch_t {
    std::string entry;      // extern "C" kernel name in the generated module
    uint32_t    grid = 1;
    uint32_t    block = 256;
    uint32_t    smem = 0;
};

struct plan_t {
    std::string           kind;     // ew_vec, ew_gather, red_row, red_split, red_generic, ...
    std::string           source;   // generated CUDA C++ (JIT kinds)
    std::vector<launch_t> launches; // run in order on the stream
    uint64_t              workspace_bytes = 0;
    int                   vec = 1;  // elements per 128-bit (or narrower) access
    // minimum alignment (bytes) every tensor pointer must have for this plan;
    // launches with less aligned pointers use the scalar twin (`fallback`).
    int                   align = 1;
};

// Plans the merged einsummable `e` as an elementwise or reduction kernel.
// force_scalar: generate the V=1 twin used for unaligned pointers.
plan_t plan_pointwise(einsum_t const& e, bool force_scalar = false);

// Every generated kernel has the signature
//   (void* out, const void* x0, ..., const void* x{n-1}, void* workspace).

} // namespace es
