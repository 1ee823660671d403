// The attention chain of a transformer layer as one kernel (sm_100a, tcgen05 / TMEM / TMA):
//
//   S[b,h,i,j] = sum_d Q[b,i,h,d] K[b,j,h,d]              (f16, f32 accumulate, rounded to f16)
//   X          = S + mask[i,j]                            (f16 add), taken to f32
//   P          = exp(X - max_j X) / sum_j exp(X - max_j X)
//   O[b,h,i,d] = sum_j f16(P)[b,h,i,j] V[b,j,h,d]
//
// which the reference runs as five apply nodes -- a contraction, a max reduction, a sum reduction,
// an elementwise node and a second contraction (softmax: src/einsummable/gwriter.cc:830-855,
// attention: llama/modules.cc:285-383) -- with the [b,h,i,j] scores written and read four times.
// Here they never leave the SM.
//
// One CTA per (128 query rows, head, batch), 5 warps:
//   warps 0-3: one thread per query row (its TMEM lane): reads the 64 scores of a key block from
//              TMEM, adds the mask, keeps the running row maximum and row sum ("online" softmax),
//              rescales the output accumulator in TMEM when the maximum moved, writes exp(x - max)
//              as f16 into shared memory in the 128B-swizzled K-major layout the second MMA reads
//   warp 4   : one lane issues the TMA tile copies (Q once; K and V per block of 64 keys, the next
//              block's tiles while the current one is being worked on) and the MMAs: Q K^T into TMEM
//              columns 0..63, P V accumulated into the columns behind them
// The row sum is applied once at the end (O / sum).  Two CTAs fit on an SM (80 KiB of shared
// memory, 256 TMEM columns), so one CTA's exponentials overlap the other's copies and MMAs.
// Every wait is bounded; on expiry the kernel records an error code, lets copies in flight land,
// frees its TMEM and returns.
#include "attention.h"

#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <climits>
#include <cstring>
#include <string>

#include "jit.h"
#include "pdl.h"
#include "tc_ptx.h"

namespace es {

namespace {

constexpr uint32_t ROWS_PER_CTA = 128;
constexpr uint32_t KEYS_PER_BLOCK = 64;
constexpr int      SOFTMAX_THREADS = 128;
constexpr int      ATTN_THREADS = 160;
constexpr uint64_t ATTN_WAIT_LIMIT_CYCLES = 4000000000ull; // ~2 s at 2 GHz

struct alignas(64) attn_params_t {
    CUtensorMap tm_q, tm_k, tm_v;
    uint32_t    batch, heads, rows, keys, d;
    int64_t     out_stride[3]; // batch, head, row (elements)
    int64_t     mask_stride;
    int32_t     skip_from;     // keys j > i - skip_from hold -inf in the mask; INT32_MIN: unknown
    // position (1..3) of the row, head and batch coordinate in each operand's tensor map
    int8_t      q_pos[3], k_pos[3], v_pos[3];
    int8_t      pad[3];
    uint32_t    tmem_cols;
};

struct attn_ctrl_t {
    uint64_t bar_q, bar_k, bar_v, bar_s, bar_o, bar_p;
    uint32_t tmem_base;
    uint32_t abort_flag;
};

__device__ unsigned int g_attn_error; // 0x11..0x16: which bounded wait gave up

__device__ __forceinline__ bool
attn_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t code)
{
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    uint32_t  spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0x3ff) == 0) {
            if (*abort_flag) return false;
            if ((uint64_t)(clock64() - t0) > ATTN_WAIT_LIMIT_CYCLES) {
                *abort_flag = code;
                atomicCAS(&g_attn_error, 0u, code);
                return false;
            }
        }
    }
    return true;
}

// coordinates (1..3) of a 4-D copy from (row, head, batch) and their positions in the map
__device__ __forceinline__ void
coords(int8_t const (&pos)[3], int row, int head, int batch, int& c1, int& c2, int& c3)
{
    c1 = pos[0] == 1 ? row : (pos[1] == 1 ? head : batch);
    c2 = pos[0] == 2 ? row : (pos[1] == 2 ? head : batch);
    c3 = pos[0] == 3 ? row : (pos[1] == 3 ? head : batch);
}

__device__ __forceinline__ __half2 as_h2(uint32_t w)
{
    return *reinterpret_cast<__half2*>(&w);
}
__device__ __forceinline__ uint32_t as_u32(__half2 h)
{
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int DPAD> // head dim rounded up to 64 or 128 (the copies fill the rest with zeros)
__global__ void __launch_bounds__(ATTN_THREADS, 2)
attention_kernel(const __grid_constant__ attn_params_t p, uint16_t* __restrict__ out, uint16_t const* __restrict__ mask)
{
    constexpr uint32_t KB = DPAD / 64;           // 64-element blocks of the head dim
    constexpr uint32_t Q_BYTES = KB * 16384;     // 128 rows x 128 bytes per block
    constexpr uint32_t K_BYTES = KB * 8192;      // 64 keys x 128 bytes per block
    constexpr uint32_t V_BYTES = KB * 8192;      // per column block: 64 keys x 128 bytes of head dim
    constexpr uint32_t P_BYTES = 16384;          // 128 rows x 64 keys f16
    extern __shared__ uint8_t smem_raw[];
    uint8_t*     smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    attn_ctrl_t* ctrl = reinterpret_cast<attn_ctrl_t*>(smem + Q_BYTES + K_BYTES + V_BYTES + P_BYTES);
    volatile uint32_t* abort_flag = &ctrl->abort_flag;
    uint32_t const sQ = smem_u32(smem), sK = sQ + Q_BYTES, sV = sK + K_BYTES, sP = sV + V_BYTES;
    uint32_t const bar_q = smem_u32(&ctrl->bar_q), bar_k = smem_u32(&ctrl->bar_k), bar_v = smem_u32(&ctrl->bar_v);
    uint32_t const bar_s = smem_u32(&ctrl->bar_s), bar_o = smem_u32(&ctrl->bar_o), bar_p = smem_u32(&ctrl->bar_p);

    int const warp = threadIdx.x >> 5;
    int const lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(bar_q, 1);
        mbar_init(bar_k, 1);
        mbar_init(bar_v, 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        mbar_init(bar_p, SOFTMAX_THREADS);
        ctrl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&ctrl->tmem_base)), "r"(p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    ES_PDL_WAIT(); // shared memory and TMEM only above; global memory from here on
    uint32_t const tmem_base = ctrl->tmem_base;
    uint32_t const tmem_s = tmem_base;                   // scores of one key block: 64 columns
    uint32_t const tmem_o = tmem_base + KEYS_PER_BLOCK;  // output accumulator: DPAD columns

    // heavier tiles (more key blocks under a lower-triangular mask) first
    uint32_t const q_tile = gridDim.x - 1 - blockIdx.x;
    uint32_t const head = blockIdx.y, batch = blockIdx.z;
    uint32_t const q0 = q_tile * ROWS_PER_CTA;
    uint32_t       nblk = (p.keys + KEYS_PER_BLOCK - 1) / KEYS_PER_BLOCK;
    if (p.skip_from != INT32_MIN) {
        // the last key any row of this tile may see
        long long const last_row = (long long)min(q0 + ROWS_PER_CTA - 1, p.rows - 1);
        long long const last_key = last_row - (long long)p.skip_from;
        uint32_t const  need = last_key < 0 ? 1u : (uint32_t)(last_key / KEYS_PER_BLOCK) + 1u;
        nblk = min(nblk, need);
    }

    if (warp == 4) {
        // ------------------------------------------------------------ copies and MMAs
        if (lane == 0) {
            uint64_t const tm_q = reinterpret_cast<uint64_t>(&p.tm_q);
            uint64_t const tm_k = reinterpret_cast<uint64_t>(&p.tm_k);
            uint64_t const tm_v = reinterpret_cast<uint64_t>(&p.tm_v);
            auto load_k = [&](uint32_t j) {
                int c1, c2, c3;
                coords(p.k_pos, (int)(j * KEYS_PER_BLOCK), (int)head, (int)batch, c1, c2, c3);
                mbar_arrive_expect_tx(bar_k, K_BYTES);
#pragma unroll
                for (uint32_t kb = 0; kb < KB; ++kb) tma_load4(sK + kb * 8192, tm_k, bar_k, (int)(kb * 64), c1, c2, c3);
            };
            auto load_v = [&](uint32_t j) {
                int c1, c2, c3;
                coords(p.v_pos, (int)(j * KEYS_PER_BLOCK), (int)head, (int)batch, c1, c2, c3);
                mbar_arrive_expect_tx(bar_v, V_BYTES);
#pragma unroll
                for (uint32_t kb = 0; kb < KB; ++kb) tma_load4(sV + kb * 8192, tm_v, bar_v, (int)(kb * 64), c1, c2, c3);
            };
            // shared-memory descriptors: 128B swizzle, 1024 bytes between 8-row groups, version 1
            uint64_t const desc_hi = (uint64_t)((1024u >> 4) | (1u << 14) | (2u << 29)) << 32;
            uint64_t const desc_v = desc_hi | ((uint64_t)(8192u >> 4) << 16); // + distance between column blocks
            // instruction descriptors: D = f32, A / B = f16, N >> 3, M >> 4; P V reads V with the head
            // dim (its N) contiguous
            uint32_t const idesc_s = (1u << 4) | ((KEYS_PER_BLOCK >> 3) << 17) | ((ROWS_PER_CTA >> 4) << 24);
            uint32_t const idesc_o = (1u << 4) | (1u << 16) | ((uint32_t)(DPAD >> 3) << 17) | ((ROWS_PER_CTA >> 4) << 24);
            auto issue_s = [&]() {
#pragma unroll
                for (uint32_t kb = 0; kb < KB; ++kb) {
#pragma unroll
                    for (uint32_t ks = 0; ks < 4; ++ks) {
                        uint64_t const da = desc_hi | (uint64_t)((sQ + kb * 16384 + ks * 32) >> 4);
                        uint64_t const db = desc_hi | (uint64_t)((sK + kb * 8192 + ks * 32) >> 4);
                        umma<0>(tmem_s, da, db, idesc_s, (kb | ks) ? 1u : 0u);
                    }
                }
                umma_commit(bar_s);
            };
            auto issue_o = [&](bool keep) {
#pragma unroll
                for (uint32_t ks = 0; ks < 4; ++ks) { // 16 keys per MMA
                    uint64_t const da = desc_hi | (uint64_t)((sP + ks * 32) >> 4);
                    uint64_t const db = desc_v | (uint64_t)((sV + ks * 2048) >> 4);
                    umma<0>(tmem_o, da, db, idesc_o, (keep || ks) ? 1u : 0u);
                }
                umma_commit(bar_o);
            };
            bool ok = true;
            {
                int c1, c2, c3;
                coords(p.q_pos, (int)q0, (int)head, (int)batch, c1, c2, c3);
                mbar_arrive_expect_tx(bar_q, Q_BYTES);
#pragma unroll
                for (uint32_t kb = 0; kb < KB; ++kb) tma_load4(sQ + kb * 16384, tm_q, bar_q, (int)(kb * 64), c1, c2, c3);
            }
            load_k(0);
            load_v(0);
            ok = attn_wait(bar_q, 0, abort_flag, 0x11) && attn_wait(bar_k, 0, abort_flag, 0x12);
            if (ok) {
                tc_fence_after();
                issue_s();
            }
            for (uint32_t j = 0; j < nblk && ok; ++j) {
                bool const more = j + 1 < nblk;
                // scores of block j are in TMEM: the K tile is free
                if (!attn_wait(bar_s, j & 1, abort_flag, 0x13)) { ok = false; break; }
                if (more) load_k(j + 1);
                // P of block j is in shared memory (and the scores have been read)
                if (!attn_wait(bar_p, j & 1, abort_flag, 0x14)) { ok = false; break; }
                if (!attn_wait(bar_v, j & 1, abort_flag, 0x15)) { ok = false; break; }
                tc_fence_after();
                issue_o(j != 0);
                if (more) {
                    if (!attn_wait(bar_k, (j + 1) & 1, abort_flag, 0x12)) { ok = false; break; }
                    tc_fence_after();
                    issue_s();
                }
                // P V of block j done: V and P tiles are free
                if (!attn_wait(bar_o, j & 1, abort_flag, 0x16)) { ok = false; break; }
                if (more) load_v(j + 1);
            }
        }
    } else {
        // ------------------------------------------------------------ softmax: one thread per row
        uint32_t const r_tile = threadIdx.x;
        uint32_t const row = q0 + r_tile;
        bool const     valid_row = row < p.rows;
        uint32_t const trow_s = tmem_s + ((uint32_t)(warp * 32) << 16);
        uint32_t const trow_o = tmem_o + ((uint32_t)(warp * 32) << 16);
        uint32_t const p_row = sP + r_tile * 128u;
        float          m_run = -INFINITY, l_run = 0.f;
        bool           ok = true;
        for (uint32_t j = 0; j < nblk; ++j) {
            ok = __all_sync(0xffffffffu, attn_wait(bar_s, j & 1, abort_flag, 0x13));
            if (!ok) break;
            tc_fence_after();
            uint32_t xh[32]; // the block's 64 scores of this row as f16 pairs
            {
                uint32_t r[32];
                tmem_ld32(trow_s, r);
#pragma unroll
                for (int i = 0; i < 16; ++i) xh[i] = pack_h2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                tmem_ld32(trow_s + 32, r);
#pragma unroll
                for (int i = 0; i < 16; ++i) xh[16 + i] = pack_h2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
            }
            uint32_t const key0 = j * KEYS_PER_BLOCK;
            uint32_t const n_valid = p.keys - key0; // >= 1
            if (mask != nullptr && valid_row) {
                uint16_t const* mrow = mask + (int64_t)row * p.mask_stride + key0;
                if (n_valid >= KEYS_PER_BLOCK && (reinterpret_cast<uintptr_t>(mrow) & 15) == 0) {
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        uint4 const mv = __ldg(reinterpret_cast<uint4 const*>(mrow) + c);
                        xh[4 * c + 0] = as_u32(__hadd2(as_h2(xh[4 * c + 0]), as_h2(mv.x)));
                        xh[4 * c + 1] = as_u32(__hadd2(as_h2(xh[4 * c + 1]), as_h2(mv.y)));
                        xh[4 * c + 2] = as_u32(__hadd2(as_h2(xh[4 * c + 2]), as_h2(mv.z)));
                        xh[4 * c + 3] = as_u32(__hadd2(as_h2(xh[4 * c + 3]), as_h2(mv.w)));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        uint32_t const lo = (uint32_t)(2 * i) < n_valid ? mrow[2 * i] : 0u;
                        uint32_t const hi = (uint32_t)(2 * i + 1) < n_valid ? mrow[2 * i + 1] : 0u;
                        xh[i] = as_u32(__hadd2(as_h2(xh[i]), as_h2(lo | (hi << 16))));
                    }
                }
            }
            if (n_valid < KEYS_PER_BLOCK) { // keys beyond the tensor: -inf
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if ((uint32_t)(2 * i) >= n_valid) xh[i] = 0xfc00fc00u;
                    else if ((uint32_t)(2 * i + 1) >= n_valid) xh[i] = (xh[i] & 0xffffu) | 0xfc000000u;
                }
            }
            __half2 mx = as_h2(xh[0]);
#pragma unroll
            for (int i = 1; i < 32; ++i) mx = __hmax2(mx, as_h2(xh[i]));
            float const m_new = fmaxf(m_run, fmaxf(__low2float(mx), __high2float(mx)));
            float const m_use = m_new == -INFINITY ? 0.f : m_new; // a row with nothing but -inf so far
            float const alpha = __expf(m_run - m_use);
            m_run = m_new;
            if (j > 0) {
                // P V of the block before has landed: the P tile is free and the accumulator complete
                ok = __all_sync(0xffffffffu, attn_wait(bar_o, (j - 1) & 1, abort_flag, 0x16));
                if (!ok) break;
                tc_fence_after();
                if (!__all_sync(0xffffffffu, alpha == 1.f)) {
#pragma unroll
                    for (int c = 0; c < DPAD / 32; ++c) {
                        uint32_t r[32];
                        tmem_ld32(trow_o + c * 32, r);
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_st32(trow_o + c * 32, r);
                    }
                }
            }
            l_run *= alpha;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint32_t w[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float2 const xf = __half22float2(as_h2(xh[4 * c + k]));
                    float const  p0 = __expf(xf.x - m_use), p1 = __expf(xf.y - m_use);
                    l_run += p0 + p1;
                    w[k] = pack_h2(p0, p1);
                }
                uint32_t const dst = p_row + ((uint32_t)(c ^ (int)(r_tile & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                             ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            mbar_arrive(bar_p);
        }
        if (ok) ok = __all_sync(0xffffffffu, attn_wait(bar_o, (nblk - 1) & 1, abort_flag, 0x16));
        if (ok) {
            tc_fence_after();
            float const inv = 1.f / l_run;
            uint16_t*   orow = out + (int64_t)batch * p.out_stride[0] + (int64_t)head * p.out_stride[1] +
                             (int64_t)row * p.out_stride[2];
#pragma unroll
            for (int c = 0; c < DPAD / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(trow_o + c * 32, r);
                if (valid_row) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) { // 8 values = 16 bytes per store; d is a multiple of 8
                        uint4 w;
                        w.x = pack_h2(__uint_as_float(r[8 * q + 0]) * inv, __uint_as_float(r[8 * q + 1]) * inv);
                        w.y = pack_h2(__uint_as_float(r[8 * q + 2]) * inv, __uint_as_float(r[8 * q + 3]) * inv);
                        w.z = pack_h2(__uint_as_float(r[8 * q + 4]) * inv, __uint_as_float(r[8 * q + 5]) * inv);
                        w.w = pack_h2(__uint_as_float(r[8 * q + 6]) * inv, __uint_as_float(r[8 * q + 7]) * inv);
                        uint32_t const col = (uint32_t)(c * 32 + q * 8);
                        if (col < p.d) *reinterpret_cast<uint4*>(orow + col) = w;
                    }
                }
            }
        }
    }

    // ------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (ctrl->abort_flag) {
        // a bounded wait expired: give copies already issued time to land before the shared
        // memory is released (bounded: ~1 ms)
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 4) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
    }
}

using encode_fn_t = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, cuuint64_t const*,
                                 cuuint64_t const*, cuuint32_t const*, cuuint32_t const*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A [batch, head, row, d] view with arbitrary (16-byte multiple) strides and d contiguous as a 4-D
// map: dim 0 = d, the others in order of increasing stride; pos[] tells the kernel where the row,
// head and batch coordinates go.  Box: 64 elements of d x `box_rows` rows.
void encode_operand(CUtensorMap* tm, int8_t (&pos)[3], void const* base, uint32_t d, uint64_t rows, uint64_t heads,
                    uint64_t batch, int64_t const (&stride)[3] /* batch, head, row */, uint32_t box_rows)
{
    static encode_fn_t fn = (encode_fn_t)driver_entry("cuTensorMapEncodeTiled");
    struct dim_t {
        uint64_t extent;
        int64_t  stride;
        int      what; // 0 row, 1 head, 2 batch
    } dims3[3] = {{rows, stride[2], 0}, {heads, stride[1], 1}, {batch, stride[0], 2}};
    // extent-1 dims last (their stride is arbitrary), the others by stride
    std::stable_sort(dims3, dims3 + 3, [](dim_t const& a, dim_t const& b) {
        bool const a1 = a.extent == 1, b1 = b.extent == 1;
        if (a1 != b1) return b1;
        return !a1 && a.stride < b.stride;
    });
    cuuint64_t gdims[4] = {d, 1, 1, 1};
    cuuint64_t gstrides[3];
    cuuint32_t box[4] = {64, 1, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    uint64_t   below = (uint64_t)d * 2;
    for (int i = 0; i < 3; ++i) {
        gdims[i + 1] = dims3[i].extent;
        uint64_t sb = (uint64_t)dims3[i].stride * 2;
        if (dims3[i].extent == 1) sb = (below + 15) & ~uint64_t(15); // any valid value
        gstrides[i] = sb;
        below = sb * dims3[i].extent;
        pos[dims3[i].what] = (int8_t)(i + 1);
        if (dims3[i].what == 0) box[i + 1] = box_rows;
    }
    CUresult rc = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), gdims, gstrides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) fail(ES_CUDA_ERROR, "attention: cuTensorMapEncodeTiled failed with code " + std::to_string((int)rc));
}

} // namespace

void check_attention(es_attention_t const& a, void const* out, void const* q, void const* k, void const* v,
                     void const* mask)
{
    if (!out || !q || !k || !v) fail(ES_BAD_ARGUMENT, "attention: null pointer");
    if (!a.batch || !a.heads || !a.rows || !a.keys || !a.head_dim) fail(ES_BAD_DESCRIPTOR, "attention: empty extent");
    if (a.head_dim > 128 || a.head_dim % 8) fail(ES_NOT_SUPPORTED, "attention: head dim must be a multiple of 8 up to 128");
    if (a.batch > 65535 || a.heads > 65535) fail(ES_NOT_SUPPORTED, "attention: more than 65535 heads or batches");
    auto strides_ok = [](int64_t const (&s)[3]) { return s[0] >= 0 && s[1] >= 0 && s[2] > 0 && !(s[0] % 8) && !(s[1] % 8) && !(s[2] % 8); };
    if (!strides_ok(a.q_stride) || !strides_ok(a.k_stride) || !strides_ok(a.v_stride) || !strides_ok(a.out_stride))
        fail(ES_NOT_SUPPORTED, "attention: strides must be multiples of 8 elements (16 bytes)");
    if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
         reinterpret_cast<uintptr_t>(v)) & 15)
        fail(ES_BAD_ARGUMENT, "attention: operands must be 16-byte aligned");
    if (mask && (a.mask_stride < (int64_t)a.keys || (reinterpret_cast<uintptr_t>(mask) & 1)))
        fail(ES_BAD_DESCRIPTOR, "attention: mask row stride below the number of keys");
}

void launch_attention(es_attention_t const& a, cudaStream_t stream, void* out, void const* q, void const* k,
                      void const* v, void const* mask)
{
    check_attention(a, out, q, k, v, mask);
    attn_params_t p;
    std::memset(&p, 0, sizeof p);
    p.batch = a.batch;
    p.heads = a.heads;
    p.rows = a.rows;
    p.keys = a.keys;
    p.d = a.head_dim;
    for (int i = 0; i < 3; ++i) p.out_stride[i] = a.out_stride[i];
    p.mask_stride = a.mask_stride;
    p.skip_from = (mask && a.skip_known) ? a.skip_from : INT32_MIN;
    encode_operand(&p.tm_q, p.q_pos, q, a.head_dim, a.rows, a.heads, a.batch, a.q_stride, ROWS_PER_CTA);
    encode_operand(&p.tm_k, p.k_pos, k, a.head_dim, a.keys, a.heads, a.batch, a.k_stride, KEYS_PER_BLOCK);
    encode_operand(&p.tm_v, p.v_pos, v, a.head_dim, a.keys, a.heads, a.batch, a.v_stride, KEYS_PER_BLOCK);
    bool const wide = a.head_dim > 64;
    p.tmem_cols = wide ? 256 : 128;
    uint32_t const kb = wide ? 2 : 1;
    uint32_t const smem = kb * (16384 + 8192 + 8192) + 16384 + (uint32_t)sizeof(attn_ctrl_t) + 1024;
    dim3 const     grid((a.rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA, a.heads, a.batch);
    auto launch = [&](auto kernel, int slot) {
        static bool attr_set[2][64] = {};
        int         dev = 0;
        cudaGetDevice(&dev);
        if (!attr_set[slot][dev & 63]) {
            ES_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024));
            attr_set[slot][dev & 63] = true;
        }
        launch_k(kernel, grid, dim3(ATTN_THREADS), smem, stream, p, static_cast<uint16_t*>(out),
                 static_cast<uint16_t const*>(mask));
    };
    if (wide) launch(attention_kernel<128>, 0);
    else launch(attention_kernel<64>, 1);
    ES_CUDA_CHECK(cudaGetLastError());
}

unsigned int read_and_clear_attention_error()
{
    unsigned int v = 0, zero = 0;
    ES_CUDA_CHECK(cudaMemcpyFromSymbol(&v, g_attn_error, sizeof v));
    if (v) ES_CUDA_CHECK(cudaMemcpyToSymbol(g_attn_error, &zero, sizeof zero));
    return v;
}

} // namespace es
