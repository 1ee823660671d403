// The library handle (one per device) and its kernel cache.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "codegen.h"
#include "common.h"
#include "contraction.h"
#include "einsum.h"
#include "jit.h"

namespace es {

struct built_kernel_t {
    einsum_t                     e; // merged form
    std::string                  kind;
    // generated (JIT) kernels
    plan_t                       plan;
    std::shared_ptr<module_t>    module;
    std::vector<void*>           functions;
    // scalar twin for pointers that are not 16-byte aligned, built on first use
    std::unique_ptr<plan_t>      scalar_plan;
    std::shared_ptr<module_t>    scalar_module;
    std::vector<void*>           scalar_functions;
    // tensor-core contraction
    std::unique_ptr<contraction_plan_t> contraction;
    uint64_t                     workspace_bytes = 0;
    uint64_t                     algorithmic_bytes = 0;
    uint64_t                     algorithmic_flops = 0; // contractions only
};

} // namespace es

struct es_b200 {
    int                                              device = 0;
    int                                              f32_policy = ES_F32_3XTF32;
    std::mutex                                       build_mutex;
    std::map<std::string, uint64_t>                  by_key;
    std::vector<std::unique_ptr<es::built_kernel_t>> kernels;
    std::atomic<uint64_t>                            counters[4];   // launches per class
    std::atomic<uint64_t>                            work_bytes[4]; // algorithmic bytes per class
    std::atomic<uint64_t>                            work_flops;    // contraction flops
};

namespace es {

// The body of es_b200_launch_einsummable; throws es_error.
void launch_built(es_b200*           h,
                  uint64_t           kernel_id,
                  cudaStream_t       stream,
                  void*              out,
                  void const* const* inns,
                  int                n_inn,
                  void*              workspace,
                  uint64_t           workspace_bytes);

} // namespace es
