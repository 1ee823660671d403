// Cross-GPU exchange kernels of the program executor (program.cc): the move_t hand-shake between
// processes that each drive one GPU, with run counters ("epochs") instead of flags that are
// flipped back and forth, so that one launch can serve many moves.
//
// Every program owns a 32-bit epoch word in its own device memory; the first kernel of every
// run increments it.  A flag is a 32-bit word both GPUs can address, zero-initialised, and only
// ever holds the epoch of the last run in which it was raised:
//   signal : stores this rank's epoch into the peers' flags (system-scope release; no waiting)
//   wait   : waits (bounded) until every listed local flag has reached this rank's epoch
//   pull   : per move, copies the bytes from the peer-mapped source into local memory with 128-bit
//            loads, and the last CTA of the move stores the epoch into the "done" flag in the source
//            rank's memory; with a "ready" flag given it first waits (bounded) for that flag itself
//   (a touch whose input is peer-mapped acknowledges through the same "done" flag: kernels.cu)
// All ranks run the same number of runs, so their epochs agree.  A wait that exceeds its limit
// records an error code and carries on; nothing traps and no wait is unbounded.
#include <cuda_runtime.h>

#include <algorithm>

#include "common.h"
#include "exchange.h"
#include "pdl.h"

namespace es {

namespace {

__device__ unsigned int g_exchange_error; // 3 = a pull's wait gave up, 4 = a done-wait gave up

__device__ __forceinline__ uint32_t ld_acquire_sys(uint32_t const* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// true when the flag reached `epoch` (wrap-safe), false when the limit ran out
__device__ __forceinline__ bool spin_until(uint32_t const* flag, uint32_t epoch, unsigned long long limit_cycles)
{
    long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys(flag) - epoch) < 0) {
        if ((unsigned long long)(clock64() - t0) > limit_cycles) return false;
        __nanosleep(32);
    }
    return true;
}

__global__ void stamp_kernel(unsigned long long* slot)
{
    ES_PDL_PROLOGUE();
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        *slot = t;
    }
}

__global__ void epoch_bump_kernel(uint32_t* epoch)
{
    ES_PDL_PROLOGUE();
    if (blockIdx.x == 0 && threadIdx.x == 0) *epoch = *epoch + 1;
}

__global__ void signal_many_kernel(uint32_t* const* __restrict__ flags, int n, uint32_t const* __restrict__ epoch)
{
    ES_PDL_PROLOGUE();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t e = *epoch;
    __threadfence_system(); // the producers' writes (earlier kernels of this GPU) before the flag
    st_release_sys(flags[i], e);
}

__global__ void wait_many_kernel(uint32_t* const* __restrict__ flags,
                                 int                           n,
                                 uint32_t const* __restrict__  epoch,
                                 unsigned long long            limit_cycles)
{
    ES_PDL_PROLOGUE();
    uint32_t e = *epoch;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        if (!spin_until(flags[i], e, limit_cycles)) atomicCAS(&g_exchange_error, 0u, 4u);
    }
}

__global__ void __launch_bounds__(256) pull_batch_kernel(pull_item_t const* __restrict__ items,
                                                         uint32_t* __restrict__          counters,
                                                         uint32_t const* __restrict__    epoch,
                                                         unsigned long long              limit_cycles)
{
    ES_PDL_PROLOGUE();
    pull_item_t const it = items[blockIdx.y];
    if (blockIdx.x >= it.n_ctas) return;
    __shared__ int ok;
    uint32_t const e = *epoch;
    if (threadIdx.x == 0) {
        // ready == null: a wait op in front of this pull has already seen the flag
        bool got = it.ready == nullptr || spin_until(it.ready, e, limit_cycles);
        if (!got) atomicCAS(&g_exchange_error, 0u, 3u);
        ok = got ? 1 : 0;
    }
    __syncthreads();
    if (ok) {
        uint64_t const n16 = it.bytes >> 4;
        uint4 const*   src = reinterpret_cast<uint4 const*>(it.src);
        uint4*         dst = reinterpret_cast<uint4*>(it.dst);
        uint64_t const nth = (uint64_t)it.n_ctas * blockDim.x;
        uint64_t       i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
        // 8 loads in flight per thread, also in the last, partial round: the round trip over NVLink is
        // a few microseconds and most moves are a single round
        for (; i < n16; i += 8 * nth) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u != 8; ++u)
                if (i + u * nth < n16) v[u] = src[i + u * nth];
#pragma unroll
            for (int u = 0; u != 8; ++u)
                if (i + u * nth < n16) dst[i + u * nth] = v[u];
        }
        if (blockIdx.x == 0) {
            uint32_t tail = (uint32_t)(it.bytes & 15);
            if (threadIdx.x < tail) it.dst[(n16 << 4) + threadIdx.x] = it.src[(n16 << 4) + threadIdx.x];
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence(); // this CTA's loads have returned (their values were stored) before it counts
        uint32_t old = atomicAdd(&counters[blockIdx.y], 1u);
        if (old == it.n_ctas - 1) {
            counters[blockIdx.y] = 0; // ready for the next run
            st_release_sys(it.done, e);
        }
    }
}

unsigned long long limit_cycles_of(uint32_t limit_ms)
{
    // clock64 ticks at the SM clock (<= ~2 GHz here): an upper bound, not a timer
    return (unsigned long long)(limit_ms ? limit_ms : 2000) * 2000000ull;
}

} // namespace

uint32_t pull_ctas_for(uint64_t bytes)
{
    // one CTA per 32 KiB (one round of 8 x 16-byte loads per thread), at most one per SM: 48 CTAs
    // left a direction of NVLink 15 % short (652 of 770 GB/s) and made a 2 MB move -- the common size
    // on the dependency chain of a partitioned layer -- a third slower than a touch reading the same bytes
    uint64_t c = (bytes + 32767) / 32768;
    return (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>(c, 148));
}

void launch_stamp(unsigned long long* slot_dev, cudaStream_t s)
{
    launch_k(stamp_kernel, dim3(1), dim3(32), 0, s, slot_dev);
    ES_CUDA_CHECK(cudaGetLastError());
}

void launch_epoch_bump(uint32_t* epoch_dev, cudaStream_t s)
{
    launch_k(epoch_bump_kernel, dim3(1), dim3(32), 0, s, epoch_dev);
    ES_CUDA_CHECK(cudaGetLastError());
}

void launch_signal_many(uint32_t* const* flags_dev, int n, uint32_t const* epoch_dev, cudaStream_t s)
{
    if (n <= 0) return;
    launch_k(signal_many_kernel, dim3((n + 127) / 128), dim3(128), 0, s, flags_dev, n, epoch_dev);
    ES_CUDA_CHECK(cudaGetLastError());
}

void launch_wait_many(uint32_t* const* flags_dev, int n, uint32_t const* epoch_dev, uint32_t limit_ms, cudaStream_t s)
{
    if (n <= 0) return;
    launch_k(wait_many_kernel, dim3(1), dim3(std::min(n, 256)), 0, s, flags_dev, n, epoch_dev, limit_cycles_of(limit_ms));
    ES_CUDA_CHECK(cudaGetLastError());
}

void launch_pull_batch(pull_item_t const* items_dev,
                       uint32_t*          counters_dev,
                       int                n,
                       uint32_t           max_ctas,
                       uint32_t const*    epoch_dev,
                       uint32_t           limit_ms,
                       cudaStream_t       s)
{
    if (n <= 0) return;
    dim3 grid(max_ctas, (unsigned)n);
    launch_k(pull_batch_kernel, grid, dim3(256), 0, s, items_dev, counters_dev, epoch_dev, limit_cycles_of(limit_ms));
    ES_CUDA_CHECK(cudaGetLastError());
}

unsigned int read_and_clear_exchange_error()
{
    unsigned int v = 0, zero = 0;
    ES_CUDA_CHECK(cudaMemcpyFromSymbol(&v, g_exchange_error, sizeof v));
    if (v) ES_CUDA_CHECK(cudaMemcpyToSymbol(g_exchange_error, &zero, sizeof zero));
    return v;
}

} // namespace es
