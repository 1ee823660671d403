// Tensor-core (tcgen05 / TMEM / TMA) contraction kernels.
#pragma once
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "einsum.h"

namespace es {

struct contraction_plan_t {
    std::string       kind;            // "contraction_tc_f16", "contraction_tc_3xtf32", ...
    std::string       info;            // tile sizes etc. for introspection
    uint64_t          workspace_bytes = 0;
    int               n_launches = 1;
    std::vector<char> blob;            // kernel parameters prepared at build time
};

// Returns false when the einsummable cannot be mapped onto the tensor-core
// kernel (dtype, alignment or mode structure); the caller then uses the
// generated SIMT kernel.
bool plan_contraction(einsum_t const& e, int f32_policy, contraction_plan_t& plan);

void launch_contraction(contraction_plan_t const& plan,
                        cudaStream_t              stream,
                        void*                     out,
                        void const*               lhs,
                        void const*               rhs,
                        void*                     workspace);

} // namespace es
