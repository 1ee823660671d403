// Tensor-core (tcgen05 / TMEM / TMA) contraction kernels.
#pragma once
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "codegen.h"
#include "einsum.h"
#include "jit.h"

namespace es {

struct contraction_plan_t {
    std::string       kind;            // "contraction_tc_f16", "contraction_tc_3xtf32", ...
    std::string       info;            // tile sizes etc. for introspection
    uint64_t          workspace_bytes = 0;
    int               n_launches = 1;
    std::vector<char> blob;            // kernel parameters prepared at build time
    // Pre-pass permutation kernels (generated): an f32 operand whose innermost
    // mode is an output mode is first copied into the workspace with its
    // contracted mode innermost, so that the TF32 MMAs only ever see K-major tiles.
    std::vector<plan_t>                    pre_plans;   // one per permuted operand, in A, B order
    std::vector<std::shared_ptr<module_t>> pre_modules; // loaded by the owner of the plan at build
    std::vector<std::vector<void*>>        pre_functions;
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

// True when both operand pointers satisfy the TMA base alignment (16 bytes).
inline bool contraction_pointers_ok(void const* lhs, void const* rhs)
{
    return ((reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs)) & 15) == 0;
}

// Reads and clears the device-side error word of the tensor-core kernels
// (nonzero = a bounded wait inside a kernel expired).  Synchronises the device.
unsigned int read_and_clear_tc_error();

// Trace builds (-DES_B200_TRACE): copies the first `n` clock samples of CTA 0 (see contraction.cu);
// returns the number copied, -1 when the library was built without the trace.
int read_trace(unsigned long long* out, int n);

} // namespace es
