// Cross-GPU exchange kernels of the program executor: epoch-valued flags, batched pulls.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace es {

// One move of a batched pull, as the device reads it.
struct pull_item_t {
    char const* src;    // peer-mapped source (16-byte aligned)
    char*       dst;    // local destination (16-byte aligned)
    uint64_t    bytes;
    uint32_t*   ready;  // local flag the source rank raises when the bytes may be read
    uint32_t*   done;   // flag in the source rank's memory, raised when they have been read
    uint32_t    n_ctas; // CTAs that work on this move (<= gridDim.x)
    uint32_t    pad;
};

uint32_t pull_ctas_for(uint64_t bytes);

// Stores the GPU's nanosecond timer into *slot_dev (profiling runs of a program).
void launch_stamp(unsigned long long* slot_dev, cudaStream_t s);
void launch_epoch_bump(uint32_t* epoch_dev, cudaStream_t s);
void launch_signal_many(uint32_t* const* flags_dev, int n, uint32_t const* epoch_dev, cudaStream_t s);
void launch_wait_many(uint32_t* const* flags_dev, int n, uint32_t const* epoch_dev, uint32_t limit_ms, cudaStream_t s);
void launch_pull_batch(pull_item_t const* items_dev,
                       uint32_t*          counters_dev,
                       int                n,
                       uint32_t           max_ctas,
                       uint32_t const*    epoch_dev,
                       uint32_t           limit_ms,
                       cudaStream_t       s);

// 0 = fine, 3 = a pull's wait for its ready flag gave up, 4 = a wait for done flags gave up
unsigned int read_and_clear_exchange_error();

} // namespace es
