// Row sum ("ab->a", castable add, f32) for callers that must not allocate.
//
// The generated split row reduction needs scratch for its per-chunk partial
// sums, which the caller normally provides as workspace.  Some callers cannot
// get any: an engine that has already handed (nearly) all of the device's
// memory to one big memgraph buffer has nothing left for cudaMalloc to return,
// and an event loop that must never stall cannot afford cudaMalloc's implicit
// device-wide synchronisation.  For them this file carries the same two-pass
// reduction with its scratch in a fixed array that is part of the library image.
//
// Limits and rules (also in include/es_b200.h):
//   * rows * chunks_per_row <= ES_B200_NOALLOC_MAX_PARTIALS (65536 floats,
//     256 KiB per GPU, resident from library load to process exit);
//   * the first call on each device looks up the array's device address; make
//     that first call before starting any stream capture;
//   * all calls on a device share the one array: two calls whose kernels may run
//     at the same time on that GPU race on it.  Every partial is written before
//     it is read, so nothing has to be cleared between calls.
#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>

#include "common.h"
#include "handle.h"

#define ES_B200_NOALLOC_MAX_PARTIALS 65536

// The scratch itself.  In host code this name is only a stand-in for the
// symbol; the address kernels can use comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_scratch[ES_B200_NOALLOC_MAX_PARTIALS];

namespace {

// pass 1: one CTA per (row, chunk); partial sum -> scratch[row * chunks + chunk]
template <bool VEC4>
__global__ void __launch_bounds__(256) noalloc_rowsum_partial(float const* __restrict__ in,
                                                              float* __restrict__ scratch,
                                                              uint64_t cols,
                                                              uint32_t chunks,
                                                              uint64_t chunk_len) // in units of VEC4 ? float4 : float
{
    uint64_t const row = blockIdx.x / chunks;
    uint32_t const chunk = blockIdx.x % chunks;
    uint64_t const units = VEC4 ? cols / 4 : cols;
    uint64_t const begin = (uint64_t)chunk * chunk_len;
    uint64_t const end = min(begin + chunk_len, units);
    float          acc[4] = {0.f, 0.f, 0.f, 0.f};
    if constexpr (VEC4) {
        float4 const* p = reinterpret_cast<float4 const*>(in + row * cols);
#pragma unroll 4
        for (uint64_t i = begin + threadIdx.x; i < end; i += 256) {
            float4 v = p[i];
            acc[0] += v.x;
            acc[1] += v.y;
            acc[2] += v.z;
            acc[3] += v.w;
        }
    } else {
        float const* p = in + row * cols;
#pragma unroll 4
        for (uint64_t i = begin + threadIdx.x; i < end; i += 256) acc[0] += p[i];
    }
    float r = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    __shared__ float red[8];
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = r;
    __syncthreads();
    if (threadIdx.x < 32) {
        r = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
        if (threadIdx.x == 0) scratch[row * chunks + chunk] = r;
    }
}

// pass 2: one thread per row adds that row's partials
__global__ void __launch_bounds__(256)
noalloc_rowsum_final(float const* __restrict__ scratch, float* __restrict__ out, uint64_t rows, uint32_t chunks)
{
    uint64_t row = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    if (row >= rows) return;
    float const* part = scratch + row * chunks;
    float        r = part[0];
    for (uint32_t j = 1; j < chunks; ++j) r += part[j];
    out[row] = r;
}

// Device address of the scratch array, looked up once per device.
float* scratch_address(int device)
{
    static std::mutex mu;
    static float*     addr[64] = {};
    if (device < 0 || device >= 64) es::fail(ES_BAD_ARGUMENT, "device ordinal out of range");
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[device]) {
        // `device` is current here (the caller selected it)
        float*      p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            es::fail(ES_CUDA_ERROR, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
        addr[device] = p;
    }
    return addr[device];
}

} // namespace

extern "C" int es_b200_rowsum_f32_noalloc(es_b200_t*   h,
                                          const float* in,
                                          float*       out,
                                          uint64_t     rows,
                                          uint64_t     cols,
                                          void*        stream)
{
    try {
        if (!h) es::fail(ES_BAD_ARGUMENT, "null handle");
        if (!in || !out) es::fail(ES_BAD_ARGUMENT, "rowsum_noalloc: null pointer");
        if (rows == 0 || cols == 0) es::fail(ES_BAD_DESCRIPTOR, "rowsum_noalloc: empty shape");
        if (rows > ES_B200_NOALLOC_MAX_PARTIALS)
            es::fail(ES_NOT_SUPPORTED,
                     "rowsum_noalloc: " + std::to_string(rows) + " rows exceed the built-in scratch of " +
                         std::to_string(ES_B200_NOALLOC_MAX_PARTIALS) +
                         " partial sums; use es_b200_launch_einsummable with a workspace");
        if (cols > (1ull << 40)) es::fail(ES_NOT_SUPPORTED, "rowsum_noalloc: row too long");
        ES_CUDA_CHECK(cudaSetDevice(h->device));
        float* scratch = scratch_address(h->device);
        bool   vec4 = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) & 15) == 0);
        uint64_t units = vec4 ? cols / 4 : cols;
        // enough CTAs to fill the GPU, at least 4 loop trips per thread, and never
        // more partials than the scratch holds
        uint64_t chunks = std::min<uint64_t>((148ull * 8 + rows - 1) / rows, std::max<uint64_t>(units / 1024, 1));
        chunks = std::min<uint64_t>(chunks, ES_B200_NOALLOC_MAX_PARTIALS / rows);
        chunks = std::max<uint64_t>(chunks, 1);
        uint64_t chunk_len = (units + chunks - 1) / chunks;
        chunks = (units + chunk_len - 1) / chunk_len;
        if (rows * chunks > 0x7fffffffull) es::fail(ES_NOT_SUPPORTED, "rowsum_noalloc: grid too large");
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        unsigned     grid = (unsigned)(rows * chunks);
        if (vec4) noalloc_rowsum_partial<true><<<grid, 256, 0, s>>>(in, scratch, cols, (uint32_t)chunks, chunk_len);
        else noalloc_rowsum_partial<false><<<grid, 256, 0, s>>>(in, scratch, cols, (uint32_t)chunks, chunk_len);
        ES_CUDA_CHECK(cudaGetLastError());
        noalloc_rowsum_final<<<(unsigned)((rows + 255) / 256), 256, 0, s>>>(scratch, out, rows, (uint32_t)chunks);
        ES_CUDA_CHECK(cudaGetLastError());
        h->counters[0] += 2;
        return ES_OK;
    } catch (es::es_error const& e) {
        es::set_last_error(e.what());
        return e.status;
    } catch (std::exception const& e) {
        es::set_last_error(e.what());
        return ES_BAD_ARGUMENT;
    }
}
