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
//              rescales the output accumulator in TMEM when the maximum has moved far enough, and
//              writes 2^(x log2 e - max) -- f16 pair arithmetic, one ex2 per two scores -- into shared
//              memory in the 128B-swizzled K-major layout the second MMA reads
//   warp 4   : one lane issues the TMA tile copies (Q once; K double-buffered and V per block of 64
//              keys) and the MMAs: Q K^T of block j + 1 into the second of two 64-column score
//              buffers in TMEM while the softmax warps work on block j, P V accumulated into the
//              columns behind them
// The row sum is applied once at the end (O / sum).  Two CTAs fit on an SM (96 KiB of shared
// memory, 256 TMEM columns each).
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
    CUtensorMap tm_q, tm_k, tm_v, tm_o;
    uint32_t    batch, heads, rows, keys, d;
    int64_t     out_stride[3]; // batch, head, row (elements)
    int64_t     mask_stride;
    int32_t     skip_from;     // keys j > i - skip_from hold -inf in the mask; INT32_MIN: unknown
    // position (1..3) of the row, head and batch coordinate in each operand's tensor map
    int8_t      q_pos[3], k_pos[3], v_pos[3], o_pos[3];
    uint32_t    tmem_cols;
};

struct attn_ctrl_t {
    uint64_t bar_q, bar_k[2], bar_v, bar_s[2], bar_o, bar_p;
    uint32_t tmem_base;
    uint32_t abort_flag;
};

__device__ unsigned int g_attn_error; // 0x11..0x16: which bounded wait gave up

// Opt-in clock trace (builds with -DES_B200_TRACE only): the CTA of the last query tile of head 0,
// batch 0 records clock64() per key block, 16 slots of 32 entries:
//   slots 0-6  (softmax warp 0): block start, scores seen, scores read and packed, mask and maximum
//              done, P V of the block before seen (accumulator rescaled), exponentials stored, arrived
//   slots 8-14 (issuer): iteration start, next block's scores issued, this block's scores seen and the
//              K copy after next issued, P seen, V seen and P V issued, P V seen, next V copy issued
#ifdef ES_B200_TRACE
__device__ unsigned long long g_attn_trace[16 * 32 + 4 * 1024]; // + per CTA: SM, start ns, end ns, key blocks
#define AT_TR(slot, idx)                                                                           \
    do {                                                                                           \
        if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (threadIdx.x & 31) == 0 && (idx) < 32) \
            g_attn_trace[(slot) * 32 + (idx)] = clock64();                                          \
    } while (0)
#else
#define AT_TR(slot, idx) do { } while (0)
#endif

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
// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// 2^x for both halves
__device__ __forceinline__ __half2 ex2_h2(__half2 x)
{
    uint32_t r;
    asm("ex2.approx.f16x2 %0, %1;" : "=r"(r) : "r"(as_u32(x)));
    return as_h2(r);
}

// the KB copies of one tile (64-element blocks of the head dim, `step` bytes apart in shared memory)
template <int KB>
__device__ __forceinline__ void tma_tile(uint32_t dst, uint32_t step, uint64_t desc, uint32_t bar, int c1, int c2, int c3)
{
    tma_load4(dst, desc, bar, 0, c1, c2, c3);
    if constexpr (KB == 2) tma_load4(dst + step, desc, bar, 64, c1, c2, c3);
}

// An accumulator that was rescaled for a new row maximum only when the maximum moved by more than
// this many powers of two: in between, the exponentials are taken against the older maximum and may
// reach 2^8, well inside f16.
constexpr float RESCALE_STEP = 8.f;

template <int DPAD> // head dim rounded up to 64 or 128 (the copies fill the rest with zeros)
__global__ void __launch_bounds__(ATTN_THREADS, 2)
attention_kernel(const __grid_constant__ attn_params_t p, uint16_t* __restrict__ out, uint16_t const* __restrict__ mask)
{
    constexpr uint32_t KB = DPAD / 64;           // 64-element blocks of the head dim
    constexpr uint32_t Q_BYTES = KB * 16384;     // 128 rows x 128 bytes per block
    constexpr uint32_t K_BYTES = KB * 8192;      // 64 keys x 128 bytes per block; two buffers
    constexpr uint32_t V_BYTES = KB * 8192;      // per column block: 64 keys x 128 bytes of head dim
    constexpr uint32_t P_BYTES = 16384;          // 128 rows x 64 keys f16
    extern __shared__ uint8_t smem_raw[];
    uint8_t*     smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    attn_ctrl_t* ctrl = reinterpret_cast<attn_ctrl_t*>(smem + Q_BYTES + 2 * K_BYTES + V_BYTES + P_BYTES);
    volatile uint32_t* abort_flag = &ctrl->abort_flag;
    uint32_t const sQ = smem_u32(smem), sK = sQ + Q_BYTES, sV = sK + 2 * K_BYTES, sP = sV + V_BYTES;
    uint32_t const bar_q = smem_u32(&ctrl->bar_q), bar_k0 = smem_u32(&ctrl->bar_k[0]), bar_v = smem_u32(&ctrl->bar_v);
    uint32_t const bar_s0 = smem_u32(&ctrl->bar_s[0]), bar_o = smem_u32(&ctrl->bar_o), bar_p = smem_u32(&ctrl->bar_p);

    int const warp = threadIdx.x >> 5;
#ifdef ES_B200_TRACE
    unsigned long long cta_t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(cta_t0));
#endif

    if (warp == 0) AT_TR(7, 0);
    // heavier tiles (more key blocks under a lower-triangular mask) first
    uint32_t const q_tile = gridDim.x - 1 - blockIdx.x;
    uint32_t const head = blockIdx.y, batch = blockIdx.z;
    uint32_t const q0 = q_tile * ROWS_PER_CTA;
    uint32_t       nblk = (p.keys + KEYS_PER_BLOCK - 1) / KEYS_PER_BLOCK;
    bool const     tri = p.skip_from != INT32_MIN; // the mask is a lower-triangular fill: 0 / -inf
    if (tri) {
        // the last key any row of this tile may see
        long long const last_row = (long long)min(q0 + ROWS_PER_CTA - 1, p.rows - 1);
        long long const last_key = last_row - (long long)p.skip_from;
        uint32_t const  need = last_key < 0 ? 1u : (uint32_t)(last_key / KEYS_PER_BLOCK) + 1u;
        nblk = min(nblk, need);
    }
    uint64_t const tm_q = reinterpret_cast<uint64_t>(&p.tm_q);
    uint64_t const tm_k = reinterpret_cast<uint64_t>(&p.tm_k);
    uint64_t const tm_v = reinterpret_cast<uint64_t>(&p.tm_v);
    bool           leader = false; // warp 4: the lane that issues copies and MMAs
    int            kc1 = 0, kc2 = 0, kc3 = 0, kstep1 = 0, kstep2 = 0, kstep3 = 0; // K coordinates of block 0, step per block
    if (warp == 4) {
        // The whole warp runs the issuing role and every address, coordinate and descriptor is computed
        // by all of its lanes from CTA-wide values, so that they can live in uniform registers; only the
        // copy / MMA / commit instructions themselves sit under the one-lane predicate.
        leader = elect_one();
        if (leader) {
            mbar_init(bar_q, 1);
            mbar_init(bar_k0, 1);
            mbar_init(bar_k0 + 8, 1);
            mbar_init(bar_v, 1);
            mbar_init(bar_s0, 1);
            mbar_init(bar_s0 + 8, 1);
            mbar_init(bar_o, 1);
            mbar_init(bar_p, SOFTMAX_THREADS);
            ctrl->abort_flag = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        ES_PDL_WAIT(); // the operands may come from the kernel before this one
        // Q and the first K tile are on their way before the TMEM allocation and the CTA barrier
        coords(p.k_pos, 0, (int)head, (int)batch, kc1, kc2, kc3);
        coords(p.k_pos, (int)KEYS_PER_BLOCK, 0, 0, kstep1, kstep2, kstep3);
        int qc1, qc2, qc3;
        coords(p.q_pos, (int)q0, (int)head, (int)batch, qc1, qc2, qc3);
        if (leader) {
            mbar_arrive_expect_tx(bar_q, Q_BYTES);
            tma_tile<KB>(sQ, 16384, tm_q, bar_q, qc1, qc2, qc3);
            mbar_arrive_expect_tx(bar_k0, K_BYTES);
            tma_tile<KB>(sK, 8192, tm_k, bar_k0, kc1, kc2, kc3);
        }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&ctrl->tmem_base)), "r"(p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        AT_TR(7, 1);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) AT_TR(7, 2);
    if (warp != 4) ES_PDL_WAIT();
    uint32_t const tmem_base = ctrl->tmem_base;
    uint32_t const tmem_s = tmem_base;                       // scores: two buffers of 64 columns
    uint32_t const tmem_o = tmem_base + 2 * KEYS_PER_BLOCK;  // output accumulator: DPAD columns

    if (warp == 4) {
        // ------------------------------------------------------------ copies and MMAs
        leader = elect_one(); // again, inside the region that uses it
        int vc1, vc2, vc3, vstep1, vstep2, vstep3;
        coords(p.v_pos, 0, (int)head, (int)batch, vc1, vc2, vc3);
        coords(p.v_pos, (int)KEYS_PER_BLOCK, 0, 0, vstep1, vstep2, vstep3);
        auto load_k = [&](uint32_t j) { // into buffer j & 1
            uint32_t const bar = bar_k0 + (j & 1) * 8, dst = sK + (j & 1) * K_BYTES;
            int const      c1 = kc1 + (int)j * kstep1, c2 = kc2 + (int)j * kstep2, c3 = kc3 + (int)j * kstep3;
            if (leader) {
                mbar_arrive_expect_tx(bar, K_BYTES);
                tma_tile<KB>(dst, 8192, tm_k, bar, c1, c2, c3);
            }
        };
        auto load_v = [&](uint32_t j) {
            int const c1 = vc1 + (int)j * vstep1, c2 = vc2 + (int)j * vstep2, c3 = vc3 + (int)j * vstep3;
            if (leader) {
                mbar_arrive_expect_tx(bar_v, V_BYTES);
                tma_tile<KB>(sV, 8192, tm_v, bar_v, c1, c2, c3);
            }
        };
        // shared-memory descriptors: 128B swizzle, 1024 bytes between 8-row groups, version 1
        uint64_t const desc_hi = (uint64_t)((1024u >> 4) | (1u << 14) | (2u << 29)) << 32;
        uint64_t const desc_v = desc_hi | ((uint64_t)(8192u >> 4) << 16); // + distance between column blocks
        // instruction descriptors: D = f32, A / B = f16, N >> 3, M >> 4; P V reads V with the head
        // dim (its N) contiguous
        uint32_t const idesc_s = (1u << 4) | ((KEYS_PER_BLOCK >> 3) << 17) | ((ROWS_PER_CTA >> 4) << 24);
        uint32_t const idesc_o = (1u << 4) | (1u << 16) | ((uint32_t)(DPAD >> 3) << 17) | ((ROWS_PER_CTA >> 4) << 24);
        // every descriptor is formed here, by the whole warp, outside the one-lane region (formed inside
        // it -- per MMA, or chained inside one asm statement -- issuing was 1.5x slower)
        uint64_t da_s[KB * 4], db_s[KB * 4], da_p[4], db_v[4]; // db_s: K buffer 0
#pragma unroll
        for (uint32_t kb = 0; kb < KB; ++kb) {
#pragma unroll
            for (uint32_t ks = 0; ks < 4; ++ks) {
                da_s[kb * 4 + ks] = desc_hi | (uint64_t)((sQ + kb * 16384 + ks * 32) >> 4);
                db_s[kb * 4 + ks] = desc_hi | (uint64_t)((sK + kb * 8192 + ks * 32) >> 4);
            }
        }
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks) { // 16 keys per MMA
            da_p[ks] = desc_hi | (uint64_t)((sP + ks * 32) >> 4);
            db_v[ks] = desc_v | (uint64_t)((sV + ks * 2048) >> 4);
        }
        auto issue_s = [&](uint32_t j) { // K buffer and score buffer j & 1
            uint32_t const d_tmem = tmem_s + (j & 1) * KEYS_PER_BLOCK;
            uint64_t const k_off = (uint64_t)(((j & 1) * K_BYTES) >> 4); // stays inside the address field
            uint32_t const bar = bar_s0 + (j & 1) * 8;
            if (leader) {
#pragma unroll
                for (uint32_t i = 0; i < KB * 4; ++i) umma<0>(d_tmem, da_s[i], db_s[i] + k_off, idesc_s, i ? 1u : 0u);
                umma_commit(bar);
            }
        };
        auto issue_o = [&](uint32_t keep) {
            if (leader) {
#pragma unroll
                for (uint32_t ks = 0; ks < 4; ++ks) umma<0>(tmem_o, da_p[ks], db_v[ks], idesc_o, (keep | ks) ? 1u : 0u);
                umma_commit(bar_o);
            }
        };
        auto wait_all = [&](uint32_t bar, uint32_t parity, uint32_t code) {
            return __all_sync(0xffffffffu, attn_wait(bar, parity, abort_flag, code)) != 0;
        };
        bool ok = wait_all(bar_q, 0, 0x11) && wait_all(bar_k0, 0, 0x12);
        if (ok) {
            tc_fence_after();
            issue_s(0);
        }
        if (nblk > 1) load_k(1);
        load_v(0);
        for (uint32_t j = 0; j < nblk && ok; ++j) {
            AT_TR(8, j);
            // the scores of block j + 1 are computed while the softmax warps work on block j: its
            // score buffer was last read for block j - 1 (bar_p of that block has been seen)
            if (j + 1 < nblk) {
                if (!wait_all(bar_k0 + ((j + 1) & 1) * 8, ((j + 1) >> 1) & 1, 0x12)) { ok = false; break; }
                tc_fence_after();
                issue_s(j + 1);
            }
            AT_TR(9, j);
            // scores of block j are in TMEM: its K buffer is free for block j + 2
            if (!wait_all(bar_s0 + (j & 1) * 8, (j >> 1) & 1, 0x13)) { ok = false; break; }
            if (j + 2 < nblk) load_k(j + 2);
            AT_TR(10, j);
            // P of block j is in shared memory (and the accumulator has been rescaled)
            if (!wait_all(bar_p, j & 1, 0x14)) { ok = false; break; }
            AT_TR(11, j);
            if (!wait_all(bar_v, j & 1, 0x15)) { ok = false; break; }
            tc_fence_after();
            issue_o(j != 0 ? 1u : 0u);
            AT_TR(12, j);
            // P V of block j done: the V and P tiles are free
            if (!wait_all(bar_o, j & 1, 0x16)) { ok = false; break; }
            AT_TR(13, j);
            if (j + 1 < nblk) load_v(j + 1);
            AT_TR(14, j);
        }
    } else {
        // ------------------------------------------------------------ softmax: one thread per row
        uint32_t const r_tile = threadIdx.x;
        uint32_t const row = q0 + r_tile;
        bool const     valid_row = row < p.rows;
        uint32_t const trow_s = tmem_s + ((uint32_t)(warp * 32) << 16);
        uint32_t const trow_o = tmem_o + ((uint32_t)(warp * 32) << 16);
        uint32_t const p_row = sP + r_tile * 128u;
        // log2(e) as an f16 pair hi + lo: x * log2(e) - M is formed by two fused multiply-adds whose
        // rounding errors are relative to the result, i.e. small where the exponential is large
        float const   LOG2E = 1.4426950408889634f;
        __half2 const c_hi = __float2half2_rn(LOG2E);
        __half2 const c_lo = __float2half2_rn(LOG2E - __low2float(c_hi)); // > 0: -inf stays -inf
        float         m_used = -INFINITY; // the row maximum (times log2 e, an f16 value) the exponentials are taken against
        float         l_run = 0.f;
        bool          ok = true;
        for (uint32_t j = 0; j < nblk; ++j) {
            if (warp == 0) AT_TR(0, j);
            ok = __all_sync(0xffffffffu, attn_wait(bar_s0 + (j & 1) * 8, (j >> 1) & 1, abort_flag, 0x13));
            if (!ok) break;
            tc_fence_after();
            if (warp == 0) AT_TR(1, j);
            uint32_t xh[32]; // the block's 64 scores of this row as f16 pairs
            {
                uint32_t r[32];
                tmem_ld32(trow_s + (j & 1) * KEYS_PER_BLOCK, r);
#pragma unroll
                for (int i = 0; i < 16; ++i) xh[i] = pack_h2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                tmem_ld32(trow_s + (j & 1) * KEYS_PER_BLOCK + 32, r);
#pragma unroll
                for (int i = 0; i < 16; ++i) xh[16 + i] = pack_h2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
            }
            if (warp == 0) AT_TR(2, j);
            uint32_t const key0 = j * KEYS_PER_BLOCK;
            uint32_t const n_valid = p.keys - key0; // >= 1
            // keys of this block the row may see: all that exist; under a lower-triangular mask (0 below
            // and on the shifted diagonal, -inf above: nothing to read) those up to the row's diagonal
            int n_allow = (int)min(n_valid, KEYS_PER_BLOCK);
            if (tri) {
                long long const lim = (long long)row - (long long)p.skip_from - (long long)key0 + 1;
                n_allow = (int)max(0ll, min((long long)n_allow, lim));
            } else if (mask != nullptr && valid_row) {
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
            if (__any_sync(0xffffffffu, n_allow < (int)KEYS_PER_BLOCK)) { // the others: -inf (no branch per element)
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    int const      keep = max(0, min(2, n_allow - 2 * i));                 // 0, 1 or 2 halves stay
                    uint32_t const kill = (uint32_t)(0xffffffffull << (16 * keep));         // bits that become -inf
                    xh[i] = (xh[i] & ~kill) | (0xfc00fc00u & kill);
                }
            }
            __half2 mx; // a tree, not a chain of 31 dependent maxima
            {
                __half2 t[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) t[i] = __hmax2(as_h2(xh[i]), as_h2(xh[16 + i]));
#pragma unroll
                for (int w = 8; w >= 1; w >>= 1) {
#pragma unroll
                    for (int i = 0; i < w; ++i) t[i] = __hmax2(t[i], t[i + w]);
                }
                mx = t[0];
            }
            float const m_blk = fmaxf(__low2float(mx), __high2float(mx));
            // this block's maximum in the exponent's units, as an f16 value
            float const cand = __half2float(__float2half_rn(m_blk * LOG2E));
            if (warp == 0) AT_TR(3, j);
            if (j == 0) {
                m_used = cand;
            } else {
                // P V of the block before has landed: the P tile is free and the accumulator complete
                bool const need = __any_sync(0xffffffffu, cand > m_used + RESCALE_STEP);
                ok = __all_sync(0xffffffffu, attn_wait(bar_o, (j - 1) & 1, abort_flag, 0x16));
                if (!ok) break;
                tc_fence_after();
                if (need) {
                    float const m_new = fmaxf(m_used, cand);
                    float const alpha = m_new == -INFINITY ? 1.f : exp2f(m_used - m_new);
                    m_used = m_new;
                    l_run *= alpha;
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
            if (warp == 0) AT_TR(4, j);
            // a row with nothing but -inf so far: any finite reference point gives exp = 0
            __half2 const neg_m = __float2half2_rn(m_used == -INFINITY ? 0.f : -m_used);
            __half2 s8 = __float2half2_rn(0.f); // sums of 8 pairs in f16 (<= 16 x 2^8), then on in f32
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                __half2 e[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    __half2 const x = as_h2(xh[4 * c + k]);
                    e[k] = ex2_h2(__hfma2(x, c_lo, __hfma2(x, c_hi, neg_m)));
                }
                __half2 const s4 = __hadd2(__hadd2(e[0], e[1]), __hadd2(e[2], e[3]));
                if (c & 1) {
                    s8 = __hadd2(s8, s4);
                    l_run += __low2float(s8) + __high2float(s8);
                } else {
                    s8 = s4;
                }
                uint32_t const dst = p_row + ((uint32_t)(c ^ (int)(r_tile & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                             ::"r"(dst), "r"(as_u32(e[0])), "r"(as_u32(e[1])), "r"(as_u32(e[2])), "r"(as_u32(e[3])) : "memory");
            }
            if (warp == 0) AT_TR(5, j);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            mbar_arrive(bar_p);
            if (warp == 0) AT_TR(6, j);
        }
        if (ok) ok = __all_sync(0xffffffffu, attn_wait(bar_o, (nblk - 1) & 1, abort_flag, 0x16));
        if (warp == 0) AT_TR(15, 0);
        if (ok) {
            // The result goes out through the Q tile's shared memory (every scores MMA has finished) in
            // the copy unit's 128B-swizzled layout and from there with one tiled store per 64 columns,
            // which also clips rows and columns beyond the tensor; 128 threads storing one row each
            // straight to global memory took ~2600 cycles here.
            tc_fence_after();
            float const inv = 1.f / l_run;
#pragma unroll
            for (int c = 0; c < DPAD / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(trow_o + c * 32, r);
#pragma unroll
                for (int q = 0; q < 4; ++q) { // 8 values = 16 bytes
                    uint32_t const w0 = pack_h2(__uint_as_float(r[8 * q + 0]) * inv, __uint_as_float(r[8 * q + 1]) * inv);
                    uint32_t const w1 = pack_h2(__uint_as_float(r[8 * q + 2]) * inv, __uint_as_float(r[8 * q + 3]) * inv);
                    uint32_t const w2 = pack_h2(__uint_as_float(r[8 * q + 4]) * inv, __uint_as_float(r[8 * q + 5]) * inv);
                    uint32_t const w3 = pack_h2(__uint_as_float(r[8 * q + 6]) * inv, __uint_as_float(r[8 * q + 7]) * inv);
                    uint32_t const chunk = (uint32_t)((c & 1) * 4 + q); // 16-byte chunk inside the 64-column block
                    uint32_t const dst = sQ + (uint32_t)(c >> 1) * 16384u + r_tile * 128u + ((chunk ^ (r_tile & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        // the four softmax warps meet (also after a failed wait), then one lane issues the stores
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ok && threadIdx.x == 0 && ctrl->abort_flag == 0) {
            uint64_t const tm_o = reinterpret_cast<uint64_t>(&p.tm_o);
            int c1, c2, c3;
            coords(p.o_pos, (int)q0, (int)head, (int)batch, c1, c2, c3);
#pragma unroll
            for (uint32_t kb = 0; kb < KB; ++kb) tma_store4(tm_o, sQ + kb * 16384, (int)(kb * 64), c1, c2, c3);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); // the tile has been read: smem may go
        }
    }

    if (warp == 0) AT_TR(15, 1);
#ifdef ES_B200_TRACE
    {
        uint32_t const cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        if (threadIdx.x == 0 && cta < 1024) {
            unsigned long long t;
            uint32_t           sm;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
            g_attn_trace[16 * 32 + 4 * cta + 0] = sm;
            g_attn_trace[16 * 32 + 4 * cta + 1] = cta_t0;
            g_attn_trace[16 * 32 + 4 * cta + 2] = t;
            g_attn_trace[16 * 32 + 4 * cta + 3] = nblk;
        }
    }
#endif
    // ------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (ctrl->abort_flag) {
        // a bounded wait expired: give copies already issued time to land before the shared
        // memory is released (bounded: ~1 ms)
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 0) AT_TR(15, 2);
    if (warp == 4) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
        AT_TR(15, 3);
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
    encode_operand(&p.tm_o, p.o_pos, out, a.head_dim, a.rows, a.heads, a.batch, a.out_stride, ROWS_PER_CTA);
    bool const wide = a.head_dim > 64;
    p.tmem_cols = 256; // 2 x 64 score columns + 64 or 128 accumulator columns, rounded to a power of two
    uint32_t const kb = wide ? 2 : 1;
    uint32_t const smem = kb * (16384 + 2 * 8192 + 8192) + 16384 + (uint32_t)sizeof(attn_ctrl_t) + 1024;
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

int read_attention_trace(unsigned long long* out, int n)
{
#ifdef ES_B200_TRACE
    if (n > 16 * 32 + 4 * 1024) n = 16 * 32 + 4 * 1024;
    ES_CUDA_CHECK(cudaDeviceSynchronize());
    ES_CUDA_CHECK(cudaMemcpyFromSymbol(out, g_attn_trace, sizeof(unsigned long long) * (size_t)n));
    return n;
#else
    (void)out;
    (void)n;
    return -1;
#endif
}

unsigned int read_and_clear_attention_error()
{
    unsigned int v = 0, zero = 0;
    ES_CUDA_CHECK(cudaMemcpyFromSymbol(&v, g_attn_error, sizeof v));
    if (v) ES_CUDA_CHECK(cudaMemcpyToSymbol(g_attn_error, &zero, sizeof zero));
    return v;
}

} // namespace es
