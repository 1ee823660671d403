// Contraction einsummables on the 5th-generation tensor cores (sm_100a).
//
//   C[outer, m, n] = sum_k A[..] * B[..]       (join = x0*x1, castable add)
//
// replaces the reference's cublas{H,S}gemm / cutensorContract calls
// (src/engine/gpu/gpu_kernel_manager.cc:1454-1609).  Neither operand is ever
// permuted in memory: each keeps its own row-major layout and is described to
// the TMA unit by a <=5-D tensor map built from its own mode order; whether its
// innermost mode is a contracted mode ("K-major") or an output mode
// ("MN-major") selects the major-ness bits of the tcgen05 shared-memory and
// instruction descriptors, so ij,jk / ij,kj / ji,jk / ji,kj and the attention
// contractions (acbe,adbe->abcd; abce,aebd->abcd; adbe,cde->abc) all run
// without a transpose pass.
//
// One persistent CTA per SM, 10 warps:
//   warp 0   : TMA producer  (cp.async.bulk.tensor -> 128B-swizzled smem ring, mbarrier tx)
//   warp 1   : MMA issuer    (one lane issues tcgen05.mma, accumulators in TMEM, 2 stages)
//   warps 2-9: epilogue      (tcgen05.ld -> convert -> swizzled smem staging -> TMA store; plain
//                            stores when the output is not TMA-describable), overlapped with the
//                            next tile's main loop through the second TMEM stage
// f16 inputs accumulate in f32.  f32 inputs run as TF32: by default split into
// hi + lo parts by a pre-pass into the workspace and multiplied with three MMAs
// (hi*hi + hi*lo + lo*hi, ~fp32 accuracy); a single TF32 MMA is an opt-in policy.
//
// Every wait on an mbarrier is bounded by a clock limit; on expiry the kernel
// records an error word, lets in-flight copies land, frees its TMEM and returns.
#include "contraction.h"
#include "pdl.h"
#include "tc_ptx.h"

#include <cuda.h>

#include <algorithm>
#include <cstring>

#include "jit.h"

namespace es {

namespace {

constexpr int      BM = 128;
constexpr int      NUM_THREADS = 320; // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue (two per TMEM quarter)
constexpr int      MAX_STAGES = 8;
constexpr int      MAX_LOOP_MODES = 6;
constexpr uint32_t STAGING_BYTES = 8 * 4096; // one 32-row x 128-byte staging tile per epilogue warp
constexpr uint64_t WAIT_LIMIT_CYCLES = 4000000000ull; // ~2 s at 2 GHz

enum src_kind_t : int8_t { SRC_ZERO = 0, SRC_MN_TILE = 1, SRC_K_BLOCK = 2, SRC_N_TILE = 3, SRC_OUTER0 = 8, SRC_KOUTER0 = 24 };

struct operand_t {
    uint32_t n_boxes;       // TMA copies per stage (per term)
    uint32_t box_bytes;     // bytes landed by one copy
    uint32_t box_step;      // coordinate step along `box_dim` between copies
    int32_t  box_dim;       // TMA dim the step applies to
    uint32_t tile_bytes;    // smem bytes of one term's tile
    uint32_t k_step_bytes;  // start-address advance per MMA k-step
    uint32_t desc_hi;       // upper 32 bits of the smem descriptor (SBO, version, swizzle)
    uint32_t desc_lbo;      // LBO field (bytes >> 4), goes to bits 16..29
    int32_t  nd;            // tensor-map rank
    int8_t   src[5];        // where each coordinate comes from
    int8_t   pad[3];
};

// Exact division of numerators below 2^31 by a fixed divisor: q = umulhi(n, m) >> s with
// l = ceil(log2 d), m = ceil(2^(31+l) / d), s = l - 1 (d <= 1: q = n).
struct fd_t {
    uint32_t m, s, d;
};

struct alignas(64) tc_params_t {
    CUtensorMap tm_a[2];    // [0] = hi (or the only) term, [1] = lo term
    CUtensorMap tm_b[2];
    operand_t   a, b;
    uint32_t    n_outer;
    uint32_t    outer_extent[MAX_LOOP_MODES];
    int64_t     outer_out_stride[MAX_LOOP_MODES];
    uint32_t    n_kouter;
    uint32_t    kouter_extent[4];
    uint32_t    m_tiles, n_tiles, k_blocks, kouter_total;
    fd_t        fd_m_tiles, fd_n_tiles, fd_m_pairs, fd_outer[MAX_LOOP_MODES];
    // digits of the grid size in the mixed radix (m_tiles, n_tiles, outer extents): a CTA steps from
    // one of its tiles to the next by adding them with carries instead of decoding the tile index
    uint32_t    step_m, step_n, step_outer[MAX_LOOP_MODES];
    uint32_t    m_extent, n_extent;
    int64_t     out_stride_m, out_stride_n;
    uint32_t    total_tiles;
    uint32_t    bn, bk_elems, stages, tmem_cols;
    uint32_t    idesc;
    uint32_t    stage_bytes;
    uint32_t    out_is_f32;
    uint32_t    n_terms;
    uint32_t    k_chunk;    // k-iterations accumulated in TMEM before the epilogue takes the partial sum
    // epilogue through TMA stores (output's innermost mode is the N mode and its layout is TMA-describable)
    CUtensorMap tm_out;
    uint32_t    out_tma;
    int32_t     out_nd;
    int8_t      out_src[8]; // SRC_MN_TILE (row), SRC_N_TILE (column) or SRC_OUTER0+j per TMA dim
    uint32_t    staging_offset; // byte offset of the epilogue staging buffers inside dynamic smem
    // 256-row work items ("big": two 128-row halves that share one B tile in shared memory, each
    // with its own accumulator slot) followed by 128-row items for the tail of the schedule
    uint32_t    mh;          // 2 when big items exist (the A region of a stage then holds two tiles)
    uint32_t    m_pairs;     // m_tiles / 2
    uint32_t    n_big;       // big items come first in the item order
    uint32_t    pair_small;  // 128-row items cut from the row pairs that are not big items
    uint32_t    total_items;
};

__device__ unsigned int g_tc_error; // nonzero = a bounded wait expired (code, see below)

// Opt-in clock trace (builds with -DES_B200_TRACE only): CTA 0 records clock64() at the role
// boundaries of its first events, 8 slots of 1000 entries.
//   slot 0 / 1: producer before / after the wait for a free stage, per k-iteration
//               (entries 500..: top of a tile / coordinates ready, per tile)
//   slot 2 / 3: MMA issuer before / after the wait for a full stage; slot 4: after the stage's commit
//               (slot 2 entries 500..: producer after the copies of a k-iteration were issued)
//   slot 5 / 6 / 7: epilogue warp 2 before / after the wait for an accumulator, after releasing it
#ifdef ES_B200_TRACE
__device__ unsigned long long g_trace[8000];
#define ES_TR(slot, idx)                                                                           \
    do {                                                                                           \
        if (blockIdx.x == 0 && (idx) < 1000) g_trace[(slot) * 1000 + (idx)] = clock64();            \
    } while (0)
#else
#define ES_TR(slot, idx) do { } while (0)
#endif

// Bounded wait.  Returns false (and raises the CTA-wide abort flag) when the
// limit expires or another role already aborted.
__device__ __forceinline__ bool
mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t code)
{
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    uint32_t  spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0x3ff) == 0) {
            if (*abort_flag) return false;
            if ((uint64_t)(clock64() - t0) > WAIT_LIMIT_CYCLES) {
                *abort_flag = code;
                atomicCAS(&g_tc_error, 0u, code);
                return false;
            }
        }
    }
    return true;
}

// smem control block placed after the stage ring
struct ctrl_t {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

// All index arrays below are only ever indexed by compile-time constants inside
// fully unrolled loops, so they live in registers: a version with run-time
// indexing put them in local memory and the dependent local-memory round trips
// (~2300 cycles per k-block) made the producer, not the tensor pipe, the bottleneck.
__device__ __forceinline__ uint32_t fd_div(uint32_t n, fd_t const& f)
{
    return f.d <= 1 ? n : (__umulhi(n, f.m) >> f.s);
}

// t -> (t / d, t % d)
__device__ __forceinline__ uint32_t fd_divmod(uint32_t& t, fd_t const& f)
{
    uint32_t const q = fd_div(t, f), r = t - q * f.d;
    t = q;
    return r;
}

__device__ __forceinline__ void
decode_rest(tc_params_t const& p, uint32_t t, uint32_t& n_tile, uint32_t (&outer)[MAX_LOOP_MODES])
{
    n_tile = fd_divmod(t, p.fd_n_tiles);
#pragma unroll
    for (int j = MAX_LOOP_MODES - 1; j >= 0; --j) outer[j] = j < (int)p.n_outer ? fd_divmod(t, p.fd_outer[j]) : 0u;
}

__device__ __forceinline__ void
decode_tile(tc_params_t const& p, uint32_t tile, uint32_t& m_tile, uint32_t& n_tile, uint32_t (&outer)[MAX_LOOP_MODES])
{
    m_tile = fd_divmod(tile, p.fd_m_tiles);
    decode_rest(p, tile, n_tile, outer);
}

// (m_tile, n_tile, outer) of tile t  ->  of tile t + gridDim.x  (schedules without 256-row items)
template <bool BIG>
__device__ __forceinline__ void
step_tile(tc_params_t const& p, uint32_t& m_tile, uint32_t& n_tile, uint32_t (&outer)[MAX_LOOP_MODES])
{
    if constexpr (!BIG) {
        uint32_t v = m_tile + p.step_m;
        uint32_t c = v >= p.m_tiles ? 1u : 0u;
        m_tile = c ? v - p.m_tiles : v;
        v = n_tile + p.step_n + c;
        c = v >= p.n_tiles ? 1u : 0u;
        n_tile = c ? v - p.n_tiles : v;
#pragma unroll
        for (int j = MAX_LOOP_MODES - 1; j >= 0; --j) {
            if (j < (int)p.n_outer) {
                v = outer[j] + p.step_outer[j] + c;
                c = v >= p.outer_extent[j] ? 1u : 0u;
                outer[j] = c ? v - p.outer_extent[j] : v;
            }
        }
    }
}

// Work item -> (first 128-row tile, halves, column tile, outer indices).  Without big items this is
// decode_tile.  With them: items [0, n_big) are row pairs (2j, 2j+1) of one column tile; the next
// pair_small items are the single rows of the remaining pairs; the rest is the unpaired last row.
template <bool BIG>
__device__ __forceinline__ void decode_item(tc_params_t const& p, uint32_t it, uint32_t& m_tile, uint32_t& halves,
                                            uint32_t& n_tile, uint32_t (&outer)[MAX_LOOP_MODES])
{
    halves = 1;
    if constexpr (!BIG) {
        decode_tile(p, it, m_tile, n_tile, outer);
        return;
    }
    uint32_t rest;
    if (it < p.n_big) {
        halves = 2;
        rest = it;
        m_tile = 2 * fd_divmod(rest, p.fd_m_pairs);
    } else if (it - p.n_big < p.pair_small) {
        uint32_t const s = it - p.n_big;
        rest = p.n_big + (s >> 1);
        m_tile = 2 * fd_divmod(rest, p.fd_m_pairs) + (s & 1);
    } else {
        m_tile = p.m_tiles - 1;
        rest = it - p.n_big - p.pair_small;
    }
    decode_rest(p, rest, n_tile, outer);
}

__device__ __forceinline__ uint32_t pick6(uint32_t const (&v)[MAX_LOOP_MODES], int i)
{
    uint32_t r = v[0];
#pragma unroll
    for (int j = 1; j < MAX_LOOP_MODES; ++j) r = (i == j) ? v[j] : r;
    return r;
}

__device__ __forceinline__ uint32_t pick4(uint32_t const (&v)[4], int i)
{
    uint32_t r = v[0];
#pragma unroll
    for (int j = 1; j < 4; ++j) r = (i == j) ? v[j] : r;
    return r;
}

// The producer warp issues one k-block's copies as one SIMT instruction: lane l owns copy l (operand,
// 128-row half, term, column block).  Everything a lane needs is read from the kernel parameters
// once and kept in registers (arrays are only ever indexed by compile-time constants), so the loop
// touches no parameter memory.  Issued one after the other by a single lane, with parameter reads,
// selects and a switch on the rank in between, a copy cost ~370 cycles, which - not the tensor pipe
// and not the memory system - bounded every contraction.
struct prod_lane_t {
    uint64_t desc;     // tensor map of this lane's term
    uint32_t dst_off;  // byte offset of the copy's destination inside a stage
    uint32_t half;     // 128-row half of a 256-row item (A copies only)
    uint32_t is_a;
    uint32_t active;
    int      src[5];   // where each coordinate comes from
    int      kinc[5];  // coordinate advance per k-block
    int      off[5];   // constant coordinate offset of this copy (second half, column block)
};

template <bool BIG>
__device__ __forceinline__ prod_lane_t make_prod_lane(tc_params_t const& p, uint32_t lane, uint32_t a_region)
{
    uint32_t const n_terms = p.n_terms;
    uint32_t const nA1 = n_terms * p.a.n_boxes; // copies of one 128-row A tile
    uint32_t const nA = nA1 * (BIG ? 2u : 1u);
    uint32_t const nB = n_terms * p.b.n_boxes;
    prod_lane_t r;
    r.is_a = lane < nA ? 1u : 0u;
    r.active = lane < nA + nB ? 1u : 0u;
    uint32_t const idx = r.is_a ? lane : lane - nA;
    r.half = r.is_a ? idx / nA1 : 0u;
    uint32_t const idx1 = r.is_a ? idx - r.half * nA1 : idx;
    uint32_t const n_boxes = r.is_a ? p.a.n_boxes : p.b.n_boxes;
    uint32_t const term = idx1 / n_boxes, box = idx1 - term * n_boxes;
    uint32_t const tile_bytes = r.is_a ? p.a.tile_bytes : p.b.tile_bytes;
    uint32_t const box_bytes = r.is_a ? p.a.box_bytes : p.b.box_bytes;
    uint32_t const box_step = r.is_a ? p.a.box_step : p.b.box_step;
    int const      box_dim = r.is_a ? p.a.box_dim : p.b.box_dim;
    CUtensorMap const* tm = r.is_a ? p.tm_a : p.tm_b;
    r.desc = reinterpret_cast<uint64_t>(term ? &tm[1] : &tm[0]);
    // stage layout: A tiles (half 0 / term 0, then half 1 or term 1), then B tiles
    r.dst_off = (r.is_a ? 0u : a_region) + (r.half + term) * tile_bytes + box * box_bytes;
#pragma unroll
    for (int d = 0; d < 5; ++d) {
        int const sa = p.a.src[d], sb = p.b.src[d];
        r.src[d] = r.is_a ? sa : sb;
        r.kinc[d] = r.src[d] == SRC_K_BLOCK ? (int)p.bk_elems : 0;
        // column blocks step along TMA dim 0 (an operand with several copies is MN-major)
        r.off[d] = (d == box_dim ? (int)(r.half * BM) : 0) + (d == 0 ? (int)(box * box_step) : 0);
    }
    return r;
}

// Coordinates of a lane's copy for (tile origin, outer indices, outer-K indices) at k block 0.
__device__ __forceinline__ void lane_coords(prod_lane_t const& o,
                                            uint32_t           mn_elems,
                                            uint32_t const (&outer)[MAX_LOOP_MODES],
                                            uint32_t const (&kouter)[4],
                                            int (&c)[5])
{
#pragma unroll
    for (int d = 0; d < 5; ++d) {
        int const s = o.src[d];
        int       v = 0;
        if (s == SRC_MN_TILE) v = (int)mn_elems;
        else if (s >= SRC_KOUTER0) v = (int)pick4(kouter, s - SRC_KOUTER0);
        else if (s >= SRC_OUTER0) v = (int)pick6(outer, s - SRC_OUTER0);
        c[d] = v + o.off[d];
    }
}

template <int KIND, bool PROMOTE, bool BIG> // BIG: the schedule holds 256-row items (p.mh == 2)
__global__ void __launch_bounds__(NUM_THREADS, 1)
tc_contraction_kernel(const __grid_constant__ tc_params_t p, void* __restrict__ out_)
{
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the 128B swizzle atoms
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // layout: [stage ring][epilogue staging, 4 warps x 2 x 4 KiB][control block]
    ctrl_t*  ctrl = reinterpret_cast<ctrl_t*>(smem + (size_t)p.stages * p.stage_bytes + STAGING_BYTES);
    volatile uint32_t* abort_flag = &ctrl->abort_flag;

    int const warp = threadIdx.x >> 5;
    int const lane = threadIdx.x & 31;
    uint32_t const smem_base = smem_u32(smem);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&ctrl->full[s]), 1);
            mbar_init(smem_u32(&ctrl->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&ctrl->tmem_full[a]), 1);
            mbar_init(smem_u32(&ctrl->tmem_empty[a]), 8);
        }
        ctrl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&ctrl->tmem_base)), "r"(p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // everything above touched shared memory and TMEM only; global memory from here on
    ES_PDL_WAIT();
    uint32_t const tmem_base = ctrl->tmem_base;

    uint32_t const k_iters = p.k_blocks * p.kouter_total;
    uint32_t const term_a_bytes = p.a.tile_bytes, term_b_bytes = p.b.tile_bytes;
    uint32_t const a_region = term_a_bytes * p.n_terms * (BIG ? 2u : 1u); // A tiles first, then B tiles

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        {
            uint32_t stage = 0, phase = 0;
            [[maybe_unused]] uint32_t tr_k = 0, tr_t = 0; // trace indices: k-iterations, tiles
            bool     ok = true;
            prod_lane_t const me = make_prod_lane<BIG>(p, (uint32_t)lane, a_region);
            uint32_t const stages = p.stages, stage_bytes = p.stage_bytes, bn = p.bn;
            uint32_t const k_blocks = p.k_blocks, n_kouter = p.n_kouter;
            uint32_t const kouter_extent[4] = {p.kouter_extent[0], p.kouter_extent[1], p.kouter_extent[2],
                                               p.kouter_extent[3]};
            uint32_t const full0 = smem_u32(&ctrl->full[0]), empty0 = smem_u32(&ctrl->empty[0]);
            uint32_t m_tile = 0, halves = 1, n_tile = 0, outer[MAX_LOOP_MODES] = {0, 0, 0, 0, 0, 0};
            if constexpr (!BIG) decode_tile(p, blockIdx.x, m_tile, n_tile, outer);
            for (uint32_t tile = blockIdx.x; tile < p.total_items && ok;
                 tile += gridDim.x, step_tile<BIG>(p, m_tile, n_tile, outer)) {
                if (lane == 0) ES_TR(0, 500 + tr_t);
                if constexpr (BIG) decode_item<true>(p, tile, m_tile, halves, n_tile, outer);
                uint32_t const tx_bytes = stage_bytes - ((BIG ? 2u : 1u) - halves) * term_a_bytes;
                bool const     mine = me.active && me.half < halves; // a 128-row item has no second half
                uint32_t const mn_elems = me.is_a ? m_tile * BM : n_tile * bn;
                // odometer over (outer K modes ..., k block): the last entry runs fastest
                uint32_t kb = 0, kouter[4] = {0, 0, 0, 0};
                int      c[5];
                lane_coords(me, mn_elems, outer, kouter, c);
                if (lane == 0) ES_TR(1, 500 + tr_t);
                ++tr_t;
                for (uint32_t ki = 0; ki < k_iters; ++ki) {
                    // lane 0 waits for the stage and announces the bytes; then every lane issues its copy
                    uint32_t const bar = full0 + stage * 8u;
                    uint32_t       go = 1;
                    if (lane == 0) {
                        ES_TR(0, tr_k);
                        go = mbar_wait(empty0 + stage * 8u, phase ^ 1, abort_flag, 1) ? 1u : 0u;
                        ES_TR(1, tr_k);
                        if (go) mbar_arrive_expect_tx(bar, tx_bytes);
                    }
                    go = __shfl_sync(0xffffffffu, go, 0);
                    if (!go) { ok = false; break; }
                    if (mine) tma_load5(smem_base + stage * stage_bytes + me.dst_off, me.desc, bar, c[0], c[1], c[2], c[3], c[4]);
                    if (lane == 0) ES_TR(2, 500 + tr_k);
                    ++tr_k;
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                    if (ki + 1 == k_iters) break; // the next tile computes its own coordinates
                    if (++kb == k_blocks) {
                        kb = 0;
                        bool carry = true;
#pragma unroll
                        for (int j = 3; j >= 0; --j) {
                            if (carry && j < (int)n_kouter) {
                                if (++kouter[j] == kouter_extent[j]) kouter[j] = 0;
                                else carry = false;
                            }
                        }
                        lane_coords(me, mn_elems, outer, kouter, c);
                    } else {
#pragma unroll
                        for (int d = 0; d < 5; ++d) c[d] += me.kinc[d];
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, use0 = 0, use1 = 0; // uses of each accumulator slot so far
            [[maybe_unused]] uint32_t tr_k = 0;
            bool     ok = true;
            constexpr uint32_t NT = PROMOTE ? 3u : 1u; // MMAs per k-step: (lo*hi, hi*lo, hi*hi) or one
            uint64_t const a_hi = ((uint64_t)p.a.desc_hi << 32) | ((uint64_t)p.a.desc_lbo << 16);
            uint64_t const b_hi = ((uint64_t)p.b.desc_hi << 32) | ((uint64_t)p.b.desc_lbo << 16);
            // descriptor start-address fields are in 16-byte units; shared addresses stay below 2^18
            uint32_t const a_kstep = p.a.k_step_bytes >> 4, b_kstep = p.b.k_step_bytes >> 4;
            uint32_t const a_term = term_a_bytes >> 4, b_term = term_b_bytes >> 4;
            uint32_t const idesc = p.idesc, stages = p.stages, stage_units = p.stage_bytes >> 4;
            uint32_t const a_region_units = a_region >> 4, base_units = smem_base >> 4;
            for (uint32_t tile = blockIdx.x; tile < p.total_items && ok; tile += gridDim.x) {
                uint32_t halves = 1;
                if constexpr (BIG) {
                    uint32_t m_tile, n_tile, outer[MAX_LOOP_MODES];
                    decode_item<true>(p, tile, m_tile, halves, n_tile, outer);
                }
                for (uint32_t ki0 = 0; ki0 < k_iters && ok; ki0 += p.k_chunk) {
                    // accumulator slots: a big item takes both (one per half); anything else the
                    // slot used less often so far, which alternates 0, 1, 0, ... between big items
                    uint32_t slot0, par0, par1 = 0;
                    if (BIG && halves == 2) { slot0 = 0; par0 = use0++ & 1; par1 = use1++ & 1; }
                    else if (use0 <= use1) { slot0 = 0; par0 = use0++ & 1; }
                    else { slot0 = 1; par0 = use1++ & 1; }
                    if (!mbar_wait(smem_u32(&ctrl->tmem_empty[slot0]), par0 ^ 1, abort_flag, 2)) { ok = false; break; }
                    tc_fence_after();
                    uint32_t const tmem_d = tmem_base + slot0 * p.bn;
                    uint32_t const ki1 = min(ki0 + p.k_chunk, k_iters);
                    for (uint32_t ki = ki0; ki < ki1; ++ki) {
                        uint32_t const s = stage;
                        ES_TR(2, tr_k);
                        if (!mbar_wait(smem_u32(&ctrl->full[s]), phase, abort_flag, 3)) { ok = false; break; }
                        ES_TR(3, tr_k);
                        if (++stage == stages) { stage = 0; phase ^= 1; }
                        tc_fence_after();
                        uint32_t const a0 = base_units + s * stage_units;
                        uint32_t const b0 = a0 + a_region_units;
                        uint32_t const keep = ki != ki0; // the first MMA of a chunk overwrites the accumulator
#pragma unroll
                        for (uint32_t ks = 0; ks < 4; ++ks) { // a 128-byte swizzle row holds four MMA k-steps
#pragma unroll
                            for (uint32_t t = 0; t < NT; ++t) {
                                uint32_t const ta = (NT == 1) ? 0 : (t == 0 ? 1 : 0);
                                uint32_t const tb = (NT == 1) ? 0 : (t == 1 ? 1 : 0);
                                uint64_t const da = a_hi | (uint64_t)(a0 + ta * a_term + ks * a_kstep);
                                uint64_t const db = b_hi | (uint64_t)(b0 + tb * b_term + ks * b_kstep);
                                umma<KIND>(tmem_d, da, db, idesc, (ks == 0 && t == 0) ? keep : 1u);
                            }
                        }
                        if (BIG && halves == 2) {
                            // second 128 rows: its own A tile and accumulator slot, the same B tile
                            if (ki == ki0) {
                                if (!mbar_wait(smem_u32(&ctrl->tmem_empty[1]), par1 ^ 1, abort_flag, 2)) { ok = false; break; }
                                tc_fence_after();
                            }
#pragma unroll
                            for (uint32_t ks = 0; ks < 4; ++ks) {
                                uint64_t const da = a_hi | (uint64_t)(a0 + a_term + ks * a_kstep);
                                uint64_t const db = b_hi | (uint64_t)(b0 + ks * b_kstep);
                                umma<KIND>(tmem_base + p.bn, da, db, idesc, ks == 0 ? keep : 1u);
                            }
                        }
                        umma_commit(smem_u32(&ctrl->empty[s])); // frees the smem stage when these MMAs retire
                        ES_TR(4, tr_k);
                        ++tr_k;
                    }
                    if (ok) {
                        umma_commit(smem_u32(&ctrl->tmem_full[slot0]));
                        if (BIG && halves == 2) umma_commit(smem_u32(&ctrl->tmem_full[1]));
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..9)
        // Two warps share each TMEM lane quarter and take alternate 128-byte pieces of the tile's
        // columns, so that short-K contractions (attention) are not bound by one warp's epilogue.
        uint32_t const quarter = warp & 3; // TMEM lanes 32*quarter .. +31 belong to this warp
        uint32_t const half = (uint32_t)(warp - 2) >> 2;
        uint32_t use0 = 0, use1 = 0, store_seq = 0; // accumulator slot uses: the MMA issuer's rule
        [[maybe_unused]] uint32_t tr_u = 0;
        bool     ok = true;
        // PROMOTE: partial sums of each k-chunk are added in registers with
        // round-to-nearest f32 adds.  The tensor core's own accumulation truncates,
        // which over hundreds of MMAs biases a long f32 sum beyond 1e-5.
        float accr[PROMOTE ? 2 : 1][32];
        // A "piece" is 128 bytes of one output row: 64 f16 or 32 f32 columns.
        uint32_t const piece_cols = p.out_is_f32 ? 32u : 64u;
        uint32_t const pieces = p.bn / piece_cols;
        // per-warp staging for TMA stores: 32 rows x 128 bytes, 128B-swizzled
        uint32_t const stage_buf = smem_base + p.staging_offset + (uint32_t)(warp - 2) * 4096u;
        // per-tile work below reads registers only (parameter reads per tile cost the epilogue
        // warps ~1000 cycles, which shows when a tile is two k-blocks long)
        uint32_t const out_tma = p.out_tma, bn = p.bn, m_extent = p.m_extent, n_extent = p.n_extent;
        uint64_t const out_desc = reinterpret_cast<uint64_t>(&p.tm_out);
        int osrc[5];
#pragma unroll
        for (int d = 0; d < 5; ++d) osrc[d] = p.out_src[d];
        uint32_t m_first = 0, halves = 1, n_tile = 0, outer[MAX_LOOP_MODES] = {0, 0, 0, 0, 0, 0};
        if constexpr (!BIG) decode_tile(p, blockIdx.x, m_first, n_tile, outer);
        for (uint32_t tile = blockIdx.x; tile < p.total_items && ok;
             tile += gridDim.x, step_tile<BIG>(p, m_first, n_tile, outer)) {
            if constexpr (BIG) decode_item<true>(p, tile, m_first, halves, n_tile, outer);
            int64_t base = 0;
            if (!out_tma) {
#pragma unroll
                for (int j = 0; j < MAX_LOOP_MODES; ++j)
                    if (j < (int)p.n_outer) base += (int64_t)outer[j] * p.outer_out_stride[j];
            }
          for (uint32_t hf = 0; hf < halves && ok; ++hf) {
            uint32_t const m_tile = m_first + hf;
            uint32_t const m_warp = m_tile * BM + quarter * 32;
            uint32_t const m = m_warp + lane;
            uint32_t const n0 = n_tile * bn;
            int oc[5]; // TMA store coordinates; the column entry is filled per piece
#pragma unroll
            for (int d = 0; d < 5; ++d) {
                int const sk = osrc[d];
                oc[d] = sk == SRC_MN_TILE ? (int)m_warp
                        : (sk >= SRC_OUTER0 ? (int)pick6(outer, sk - SRC_OUTER0) : 0);
            }
            for (uint32_t ki0 = 0; ki0 < k_iters && ok; ki0 += p.k_chunk) {
                uint32_t acc, acc_ph;
                if (BIG && halves == 2) { acc = hf; acc_ph = (hf == 0 ? use0++ : use1++) & 1; }
                else if (use0 <= use1) { acc = 0; acc_ph = use0++ & 1; }
                else { acc = 1; acc_ph = use1++ & 1; }
                bool const first_chunk = ki0 == 0, last_chunk = ki0 + p.k_chunk >= k_iters;
                if (warp == 2 && lane == 0) ES_TR(5, tr_u);
                if (!mbar_wait(smem_u32(&ctrl->tmem_full[acc]), acc_ph, abort_flag, 4)) { ok = false; break; }
                if (warp == 2 && lane == 0) ES_TR(6, tr_u);
                tc_fence_after();
                uint32_t const trow = tmem_base + ((quarter * 32u) << 16) + acc * p.bn;
                if constexpr (PROMOTE) {
                    // this chunk's partial sums join the running sums in registers; piece slots are
                    // compile-time indices (bn <= 128: at most 4 pieces, 2 per warp)
#pragma unroll
                    for (int c2 = 0; c2 < 2; ++c2) {
                        uint32_t const pc = half + 2u * (uint32_t)c2;
                        if (pc < pieces) {
                            uint32_t r[32];
                            tmem_ld32(trow + pc * 32, r);
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                float const v = __uint_as_float(r[j]);
                                accr[c2][j] = first_chunk ? v : __fadd_rn(accr[c2][j], v);
                            }
                        }
                    }
                }
                for (uint32_t pc = half; pc < pieces && (last_chunk || !PROMOTE); pc += 2) {
                    uint4 w[8]; // this lane's 128 bytes of the piece, in the output dtype
                    if (p.out_is_f32) {
                        uint32_t r[32];
                        if constexpr (PROMOTE) {
                            bool const second = (pc >> 1) != 0;
#pragma unroll
                            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(second ? accr[1][j] : accr[0][j]);
                        } else {
                            tmem_ld32(trow + pc * 32, r);
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) w[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    } else {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            uint32_t r[32];
                            tmem_ld32(trow + pc * 64 + h * 32, r);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                w[h * 4 + j].x = pack_h2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1]));
                                w[h * 4 + j].y = pack_h2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                                w[h * 4 + j].z = pack_h2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                                w[h * 4 + j].w = pack_h2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                            }
                        }
                    }
                    if (!last_chunk) continue;
                    uint32_t const n = n0 + pc * piece_cols;
                    if (out_tma) {
                        // 32 rows x 128 bytes -> swizzled staging -> one TMA store per warp and piece
                        // (rows / columns beyond the tensor are clipped by the TMA unit)
                        uint32_t const buf = stage_buf;
                        if (store_seq >= 1) { // the previous store of this warp must have read the tile
                            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                            __syncwarp();
                        }
                        ++store_seq;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            uint32_t dst = buf + lane * 128u + ((uint32_t)(j ^ (lane & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                         ::"r"(dst), "r"(w[j].x), "r"(w[j].y), "r"(w[j].z), "r"(w[j].w) : "memory");
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0 && n < n_extent && m_warp < m_extent) {
                            int cc[5];
#pragma unroll
                            for (int d = 0; d < 5; ++d) cc[d] = (osrc[d] == SRC_N_TILE) ? (int)n : oc[d];
                            tma_store5(out_desc, buf, cc[0], cc[1], cc[2], cc[3], cc[4]);
                        }
                    } else if (m < m_extent && n < n_extent) {
                        int64_t off = base + (int64_t)m * p.out_stride_m + (int64_t)n * p.out_stride_n;
                        bool    full = n + piece_cols <= n_extent;
                        if (p.out_is_f32) {
                            float* o = static_cast<float*>(out_) + off;
                            if (p.out_stride_n == 1 && full && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
                                for (int j = 0; j < 8; ++j) *reinterpret_cast<uint4*>(o + 4 * j) = w[j];
                            } else {
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    uint32_t const e4[4] = {w[j].x, w[j].y, w[j].z, w[j].w};
#pragma unroll
                                    for (int i = 0; i < 4; ++i)
                                        if (n + 4 * j + i < n_extent)
                                            o[(int64_t)(4 * j + i) * p.out_stride_n] = __uint_as_float(e4[i]);
                                }
                            }
                        } else {
                            uint16_t* o = static_cast<uint16_t*>(out_) + off;
                            if (p.out_stride_n == 1 && full && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
                                for (int j = 0; j < 8; ++j) *reinterpret_cast<uint4*>(o + 8 * j) = w[j];
                            } else {
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    uint32_t const e4[4] = {w[j].x, w[j].y, w[j].z, w[j].w};
#pragma unroll
                                    for (int i = 0; i < 8; ++i)
                                        if (n + 8 * j + i < n_extent)
                                            o[(int64_t)(8 * j + i) * p.out_stride_n] =
                                                (uint16_t)((i & 1) ? (e4[i >> 1] >> 16) : (e4[i >> 1] & 0xffffu));
                                }
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctrl->tmem_empty[acc]));
                if (warp == 2 && lane == 0) ES_TR(7, tr_u);
                ++tr_u;
            }
          }
        }
        // all of this warp's stores must have read their staging buffers before smem goes away
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
    }

    // ------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (ctrl->abort_flag) {
        // a bounded wait expired: give copies already issued time to land before the
        // shared memory is released (bounded: ~1 ms)
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
    }
}

// f32 -> (hi, lo) with hi = tf32(x) (round to nearest), lo = x - hi (exact in f32)
__global__ void __launch_bounds__(256) split_tf32_kernel(float const* x, float* hi, float* __restrict__ lo,
                                                         uint64_t n4) // hi may alias x (in-place split)
{
    ES_PDL_PROLOGUE();
    uint64_t nth = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += nth) {
        float4 v = reinterpret_cast<float4 const*>(x)[i];
        float4 h, l;
        uint32_t t;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(t) : "f"(v.x)); h.x = __uint_as_float(t); l.x = v.x - h.x;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(t) : "f"(v.y)); h.y = __uint_as_float(t); l.y = v.y - h.y;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(t) : "f"(v.z)); h.z = __uint_as_float(t); l.z = v.z - h.z;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(t) : "f"(v.w)); h.w = __uint_as_float(t); l.w = v.w - h.w;
        reinterpret_cast<float4*>(hi)[i] = h;
        reinterpret_cast<float4*>(lo)[i] = l;
    }
}

// ------------------------------------------------------------------ host side
struct tc_plan_t {
    tc_params_t p;
    int         kind;          // 0 f16, 1 tf32
    uint32_t    smem_bytes;
    uint32_t    grid;
    // tensor-map recipes (the base pointer is only known at launch)
    struct map_recipe_t {
        uint32_t nd;
        uint64_t dims[5];
        uint64_t strides_bytes[4];
        uint32_t box[5];
        int      dtype; // CUtensorMapDataType
    } ra, rb, rout;
    int      out_tma;
    uint64_t a_elems, b_elems; // for the split pre-pass
    int      swap;             // the second input plays the A (128-row) role
    int      promote;          // chunked accumulation with register promotion (3xTF32)
    int      a_perm, b_perm;   // operand is first copied K-major into the workspace
    uint64_t ws_b_offset;      // float offset of B's workspace region
};

using encode_fn_t = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, cuuint64_t const*,
                                 cuuint64_t const*, cuuint32_t const*, cuuint32_t const*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// pad5: encode with five dims, the missing outer ones with extent 1 (operand maps: the producer
// always issues the 5-D form of the copy)
void encode_map(CUtensorMap* tm, tc_plan_t::map_recipe_t const& r, void const* base, bool pad5 = false)
{
    static encode_fn_t fn = (encode_fn_t)driver_entry("cuTensorMapEncodeTiled");
    cuuint32_t         elem_strides[5] = {1, 1, 1, 1, 1};
    cuuint64_t         dims[5];
    cuuint64_t         strides[4];
    cuuint32_t         box[5];
    for (uint32_t i = 0; i < r.nd; ++i) {
        dims[i] = r.dims[i];
        box[i] = r.box[i];
        if (i + 1 < r.nd) strides[i] = r.strides_bytes[i];
    }
    uint32_t nd = r.nd;
    if (pad5) {
        uint64_t const esize = r.dtype == CU_TENSOR_MAP_DATA_TYPE_FLOAT16 ? 2 : 4;
        for (; nd < 5; ++nd) {
            // stride of a new outermost dim of extent 1: the byte size of everything below it,
            // rounded up to the 16 bytes a stride must be a multiple of
            uint64_t below = nd == 1 ? dims[0] * esize : strides[nd - 2] * dims[nd - 1];
            strides[nd - 1] = (below + 15) & ~uint64_t(15);
            dims[nd] = 1;
            box[nd] = 1;
        }
    }
    CUresult rc = fn(tm, (CUtensorMapDataType)r.dtype, nd, const_cast<void*>(base), dims, strides, box,
                     elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) fail(ES_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)rc));
}

enum mode_class_t { MC_BATCH, MC_M, MC_N, MC_K, MC_BAD };

fd_t make_fd(uint32_t d)
{
    fd_t f{0, 0, d};
    if (d > 1) {
        // with e = m*d - 2^(31+l) in [0, d) and n < 2^31: n*e < 2^(31+l), so the quotient is exact
        uint32_t l = 0;
        while ((1ull << l) < d) ++l;
        f.m = (uint32_t)(((1ull << (31 + l)) + d - 1) / d);
        f.s = l - 1;
    }
    return f;
}

} // namespace

bool plan_contraction(einsum_t const& e, int f32_policy, contraction_plan_t& plan)
{
    if (!e.is_contraction()) return false;
    int dt = e.out_dtype();
    if (dt != ES_F16 && dt != ES_F32) return false;
    if (e.inn_dtype(0) != dt || e.inn_dtype(1) != dt) return false;
    int const      r = e.join_rank();
    int const      esize = dtype_size(dt);
    // The product is symmetric in its operands.  When the first input has very
    // few rows along its innermost output mode (e.g. the last-token vocabulary
    // projection, 4 x 32000 x 4096) the roles are swapped so that the long mode
    // fills the 128-row side of the MMA tile.
    bool swap = false;
    {
        auto extent_of_innermost_out_mode = [&](int k) {
            auto const& t = e.inns[k];
            auto const  other = e.inn_strides(1 - k);
            for (int i = (int)t.size() - 1; i >= 0; --i)
                if (t[i] < e.out_rank && other[t[i]] == 0) return e.join_shape[t[i]];
            return (uint64_t)0;
        };
        uint64_t m0 = extent_of_innermost_out_mode(0), n0 = extent_of_innermost_out_mode(1);
        swap = m0 > 0 && n0 > 0 && m0 <= 64 && n0 > m0;
    }
    int const      ia = swap ? 1 : 0, ib = swap ? 0 : 1;
    auto const     sa_orig = e.inn_strides(ia), sb_orig = e.inn_strides(ib), so = e.out_strides();
    auto const&    A_orig = e.inns[ia];
    auto const&    B_orig = e.inns[ib];
    if (A_orig.size() > 5 || B_orig.size() > 5 || A_orig.size() < 2 || B_orig.size() < 2) return false;

    std::vector<mode_class_t> cls(r);
    for (int m = 0; m != r; ++m) {
        bool ia = sa_orig[m] != 0, ib = sb_orig[m] != 0, io = m < e.out_rank;
        if (ia && ib && io) cls[m] = MC_BATCH;
        else if (ia && !ib && io) cls[m] = MC_M;
        else if (!ia && ib && io) cls[m] = MC_N;
        else if (ia && ib && !io) cls[m] = MC_K;
        else return false;
        if (e.join_shape[m] > 0x7fffffffull) return false;
    }
    // innermost (smallest stride) M mode of A, N mode of B, K mode of each
    auto innermost = [&](std::vector<int> const& modes, mode_class_t c) {
        for (int i = (int)modes.size() - 1; i >= 0; --i)
            if (cls[modes[i]] == c) return modes[i];
        return -1;
    };
    int m_in = innermost(A_orig, MC_M), n_in = innermost(B_orig, MC_N);
    int k_in = innermost(A_orig, MC_K);
    if (m_in < 0 || n_in < 0 || k_in < 0 || innermost(B_orig, MC_K) != k_in) return false;
    bool a_mn = A_orig.back() == m_in, b_mn = B_orig.back() == n_in;
    if (!a_mn && A_orig.back() != k_in) return false;
    if (!b_mn && B_orig.back() != k_in) return false;

    // f32 operands run as TF32 with K-major tiles only: an operand whose innermost
    // mode is an output mode is copied (pre-pass, generated permutation kernel)
    // into the workspace with the contracted mode moved innermost.
    std::vector<int>      A = A_orig, B = B_orig;
    std::vector<uint64_t> sa = sa_orig, sb = sb_orig;
    bool const            a_perm = dt == ES_F32 && a_mn, b_perm = dt == ES_F32 && b_mn;
    auto k_last = [&](std::vector<int>& modes, std::vector<uint64_t>& st) {
        modes.erase(std::find(modes.begin(), modes.end(), k_in));
        modes.push_back(k_in);
        std::fill(st.begin(), st.end(), 0);
        uint64_t s = 1;
        for (int i = (int)modes.size() - 1; i >= 0; --i) {
            st[modes[i]] = s;
            s *= e.join_shape[modes[i]];
        }
    };
    if (a_perm) { k_last(A, sa); a_mn = false; }
    if (b_perm) { k_last(B, sb); b_mn = false; }
    auto perm_plan = [&](std::vector<int> const& orig, std::vector<int> const& eff) {
        einsum_t pe;
        pe.out_rank = (int)eff.size();
        pe.castable = ES_CASTABLE_NONE;
        pe.join = scalarop_t::parse("hole|f32@0");
        std::vector<int> in_modes;
        for (int m : eff) pe.join_shape.push_back(e.join_shape[m]);
        for (int m : orig) in_modes.push_back((int)(std::find(eff.begin(), eff.end(), m) - eff.begin()));
        pe.inns.push_back(in_modes);
        return plan_pointwise(pe.merge_adjacent_dims(), false);
    };

    // TMA: every non-innermost stride must be a multiple of 16 bytes
    for (int m : A)
        if (m != A.back() && (sa[m] * esize) % 16) return false;
    for (int m : B)
        if (m != B.back() && (sb[m] * esize) % 16) return false;

    tc_plan_t tp;
    std::memset(&tp, 0, sizeof tp);
    tc_params_t& p = tp.p;
    tp.kind = dt == ES_F16 ? 0 : 1;
    p.n_terms = (dt == ES_F32 && f32_policy == ES_F32_3XTF32) ? 2 : 1; // number of operand copies (hi, lo)
    uint32_t const row_elems = 128 / esize;   // elements in one 128-byte swizzle row
    p.bk_elems = row_elems;
    uint64_t const M = e.join_shape[m_in], Nn = e.join_shape[n_in], K = e.join_shape[k_in];
    uint32_t bn;
    if (p.n_terms == 2) bn = Nn > 64 ? 128 : 64;
    else bn = Nn > 128 ? 256 : (Nn > 64 ? 128 : 64);
    p.bn = bn;
    p.m_extent = (uint32_t)M;
    p.n_extent = (uint32_t)Nn;
    p.m_tiles = (uint32_t)((M + BM - 1) / BM);
    p.n_tiles = (uint32_t)((Nn + bn - 1) / bn);
    p.k_blocks = (uint32_t)((K + row_elems - 1) / row_elems);
    p.out_stride_m = (int64_t)so[m_in];
    p.out_stride_n = (int64_t)so[n_in];
    p.out_is_f32 = dt == ES_F32;

    // loop modes
    std::vector<int> outer_idx(r, -1), kouter_idx(r, -1);
    uint64_t         total = (uint64_t)p.m_tiles * p.n_tiles;
    p.kouter_total = 1;
    for (int m = 0; m != r; ++m) {
        if (m == m_in || m == n_in || m == k_in) continue;
        if (cls[m] == MC_K) {
            if (p.n_kouter >= 4) return false;
            kouter_idx[m] = (int)p.n_kouter;
            p.kouter_extent[p.n_kouter++] = (uint32_t)e.join_shape[m];
            if ((uint64_t)p.kouter_total * e.join_shape[m] > 0x7fffffffull) return false;
            p.kouter_total *= (uint32_t)e.join_shape[m];
        } else {
            if (p.n_outer >= MAX_LOOP_MODES) return false;
            outer_idx[m] = (int)p.n_outer;
            p.outer_extent[p.n_outer] = (uint32_t)e.join_shape[m];
            p.outer_out_stride[p.n_outer] = (int64_t)so[m];
            ++p.n_outer;
            total *= e.join_shape[m];
        }
    }
    if (total > 0x7fffffffull) return false;
    p.total_tiles = (uint32_t)total;

    // operands
    auto setup = [&](std::vector<int> const& modes, std::vector<uint64_t> const& st, bool mn_major, int mn_mode,
                     uint32_t tile_mn, operand_t& o, tc_plan_t::map_recipe_t& rc) {
        int nd = (int)modes.size();
        o.nd = nd;
        rc.nd = nd;
        rc.dtype = dt == ES_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
        for (int d = 0; d < 5; ++d) o.src[d] = SRC_ZERO;
        for (int d = 0; d != nd; ++d) {
            int m = modes[nd - 1 - d]; // TMA dim 0 = innermost
            rc.dims[d] = e.join_shape[m];
            if (d > 0) rc.strides_bytes[d - 1] = st[m] * esize;
            rc.box[d] = 1;
            if (m == mn_mode) o.src[d] = SRC_MN_TILE;
            else if (m == k_in) o.src[d] = SRC_K_BLOCK;
            else if (kouter_idx[m] >= 0) o.src[d] = (int8_t)(SRC_KOUTER0 + kouter_idx[m]);
            else o.src[d] = (int8_t)(SRC_OUTER0 + outer_idx[m]);
            if (m == mn_mode) o.box_dim = d;
        }
        int k_dim = -1, mn_dim = o.box_dim;
        for (int d = 0; d != nd; ++d)
            if (modes[nd - 1 - d] == k_in) k_dim = d;
        uint32_t const version = 1u << 14; // descriptor version field (bit 46 of the 64-bit word)
        uint32_t const sw128 = 2u << 29;   // layout type SWIZZLE_128B (bits 61..63)
        uint32_t const sbo = (1024u >> 4); // 8 rows x 128 bytes between core-matrix groups
        o.tile_bytes = tile_mn * 128;
        if (!mn_major) {
            // K-major: rows of the tile are MN indices, 128 bytes of K each
            rc.box[k_dim] = row_elems;
            rc.box[mn_dim] = tile_mn; // <= 256
            o.n_boxes = 1;
            o.box_bytes = tile_mn * 128;
            o.box_step = 0;
            o.k_step_bytes = 32;
            o.desc_lbo = 0;
            o.desc_hi = sbo | version | sw128;
        } else {
            // MN-major: rows are K indices, 128 bytes of MN each; one copy per 128-byte column block
            rc.box[mn_dim] = row_elems;
            rc.box[k_dim] = row_elems; // BK rows (BK = elements per 128 bytes of K in the other operand)
            o.n_boxes = tile_mn / row_elems;
            o.box_bytes = row_elems * 128;
            o.box_step = row_elems;
            o.k_step_bytes = (32 / esize) * 128; // UMMA_K rows
            o.desc_lbo = (o.box_bytes >> 4);     // byte distance between column blocks
            o.desc_hi = sbo | version | sw128;
        }
        return true;
    };
    setup(A, sa, a_mn, m_in, BM, p.a, tp.ra);
    setup(B, sb, b_mn, n_in, bn, p.b, tp.rb);
    // the K extent of one block must be the same for both operands: row_elems elements
    p.stage_bytes = (p.a.tile_bytes + p.b.tile_bytes) * p.n_terms;
    uint32_t const smem_budget = 227 * 1024 - 1024 /*alignment*/ - STAGING_BYTES - (uint32_t)sizeof(ctrl_t) - 64;
    // 256-row items.  A 128 x 256 tile streams 48 KiB per k-block for 512 cycles of MMA work; the
    // copies were measured at 750 cycles per k-block (64 bytes per clock into the SM), so the tile
    // is bound by its operand stream, not by the tensor pipe.  Two 128-row halves that share the
    // B tile stream 64 KiB for 1024 cycles of MMA work.  They take both accumulator slots, so the
    // epilogue of an item overlaps the next item only half by half; and items twice as large
    // quantise worse over 148 SMs, so the tail of the schedule falls back to 128-row items.  The
    // split is chosen by the estimated makespan of the round-robin schedule.
    p.mh = 1;
    p.total_items = p.total_tiles;
    {
        uint32_t const k_iters = p.k_blocks * p.kouter_total;
        uint32_t const big_stage = 2 * p.a.tile_bytes + p.b.tile_bytes;
        bool const     eligible = dt == ES_F16 && p.n_terms == 1 && bn == 256 && p.m_tiles >= 2 && k_iters >= 16 &&
                              smem_budget / big_stage >= 3;
        if (eligible) {
            uint32_t const G = 148;
            uint64_t const rest = total / p.m_tiles;              // column tiles x outer indices
            uint32_t const m_pairs = p.m_tiles / 2;
            uint64_t const pairs = (uint64_t)m_pairs * rest;      // candidate big items
            uint64_t const odd_rows = (p.m_tiles & 1) ? rest : 0; // items of the unpaired last row
            double const   cost_small = 750.0, cost_big = 1140.0; // cycles per k-block (incl. epilogue stall)
            auto makespan = [&](uint64_t n_big) {
                uint64_t const n_small = 2 * (pairs - n_big) + odd_rows;
                double         worst = 0;
                for (uint32_t c = 0; c < G; ++c) {
                    uint64_t big_c = n_big / G + (c < n_big % G ? 1 : 0);
                    // small item j runs on CTA (n_big + j) % G
                    uint64_t first = (c + G - n_big % G) % G; // smallest j with (n_big + j) % G == c
                    uint64_t small_c = n_small > first ? (n_small - first + G - 1) / G : 0;
                    worst = std::max(worst, big_c * cost_big + small_c * cost_small);
                }
                return worst;
            };
            uint64_t best = 0;
            double   best_t = makespan(0);
            for (uint64_t cand : {pairs, pairs / G * G}) {
                double t = makespan(cand);
                if (t < best_t) { best_t = t; best = cand; }
            }
            if (best > 0) {
                p.mh = 2;
                p.m_pairs = m_pairs;
                p.n_big = (uint32_t)best;
                p.pair_small = (uint32_t)(2 * (pairs - best));
                p.total_items = (uint32_t)(best + 2 * (pairs - best) + odd_rows);
                p.stage_bytes = big_stage;
            }
        }
    }
    p.stages = std::min<uint32_t>(MAX_STAGES, smem_budget / p.stage_bytes);
    if (p.stages < 2) return false;
    p.fd_m_tiles = make_fd(p.m_tiles);
    p.fd_n_tiles = make_fd(p.n_tiles);
    p.fd_m_pairs = make_fd(p.m_pairs);
    for (uint32_t j = 0; j < MAX_LOOP_MODES; ++j) p.fd_outer[j] = make_fd(j < p.n_outer ? p.outer_extent[j] : 1u);
    p.tmem_cols = 2 * bn < 32 ? 32 : 2 * bn; // 128, 256 or 512: powers of two
    // 3xTF32: promote the partial sum to registers every 8 k-blocks (256 contracted elements)
    tp.promote = p.n_terms == 2 ? 1 : 0;
    p.k_chunk = tp.promote ? 8u : (p.k_blocks * p.kouter_total);
    // instruction descriptor: D=f32, A/B format, majors, N>>3, M>>4
    uint32_t fmt = dt == ES_F16 ? 0u : 2u;
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
              ((bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    p.staging_offset = p.stages * p.stage_bytes;
    tp.smem_bytes = p.stages * p.stage_bytes + STAGING_BYTES + (uint32_t)sizeof(ctrl_t) + 1024;
    // epilogue through TMA stores when the output's innermost mode is the N mode and every other
    // output stride is a multiple of 16 bytes
    {
        bool ok_tma = so[n_in] == 1 && e.out_rank <= 5 && e.out_rank >= 2;
        for (int m = 0; m != e.out_rank; ++m)
            if (m != n_in && (so[m] * esize) % 16) ok_tma = false;
        tp.out_tma = ok_tma ? 1 : 0;
        if (ok_tma) {
            auto& rc = tp.rout;
            rc.nd = e.out_rank;
            p.out_nd = e.out_rank;
            rc.dtype = dt == ES_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
            // output modes sorted by stride: the output is row-major over modes 0..out_rank-1
            for (int d = 0; d != e.out_rank; ++d) {
                int m = e.out_rank - 1 - d;
                rc.dims[d] = e.join_shape[m];
                if (d > 0) rc.strides_bytes[d - 1] = so[m] * esize;
                rc.box[d] = 1;
                if (m == n_in) {
                    rc.box[d] = row_elems;
                    p.out_src[d] = SRC_N_TILE;
                } else if (m == m_in) {
                    rc.box[d] = 32;
                    p.out_src[d] = SRC_MN_TILE;
                } else {
                    p.out_src[d] = (int8_t)(SRC_OUTER0 + outer_idx[m]);
                }
            }
        }
    }
    tp.grid = std::min<uint32_t>(p.total_items, 148);
    {
        uint32_t g = tp.grid;
        p.step_m = g % p.m_tiles;
        g /= p.m_tiles;
        p.step_n = g % p.n_tiles;
        g /= p.n_tiles;
        for (int j = (int)p.n_outer - 1; j >= 0; --j) {
            p.step_outer[j] = g % p.outer_extent[j];
            g /= p.outer_extent[j];
        }
    }
    tp.a_elems = e.inn_nelem(ia);
    tp.b_elems = e.inn_nelem(ib);
    tp.swap = swap ? 1 : 0;

    plan.kind = dt == ES_F16 ? "contraction_tc_f16" : (p.n_terms == 2 ? "contraction_tc_3xtf32" : "contraction_tc_tf32");
    plan.n_launches = 1;
    plan.pre_plans.clear();
    tp.a_perm = a_perm;
    tp.b_perm = b_perm;
    if (a_perm) plan.pre_plans.push_back(perm_plan(A_orig, A));
    if (b_perm) plan.pre_plans.push_back(perm_plan(B_orig, B));
    plan.n_launches += (int)plan.pre_plans.size();
    // workspace (floats): [A copy / A hi][A lo][B copy / B hi][B lo], parts present as needed
    uint64_t a_ws = 0, b_ws = 0;
    if (p.n_terms == 2) {
        if ((tp.a_elems % 4) || (tp.b_elems % 4)) return false;
        a_ws = 2 * tp.a_elems;
        b_ws = 2 * tp.b_elems;
        plan.n_launches += 2;
    } else {
        a_ws = a_perm ? tp.a_elems : 0;
        b_ws = b_perm ? tp.b_elems : 0;
    }
    a_ws = (a_ws + 3) & ~3ull; // keep the B region 16-byte aligned
    tp.ws_b_offset = a_ws;
    plan.workspace_bytes = (a_ws + b_ws) * 4;
    plan.info = "bm=128,bn=" + std::to_string(bn) + ",bk=" + std::to_string(row_elems) + ",stages=" +
                std::to_string(p.stages) + ",tiles=" + std::to_string(p.total_tiles) +
                (p.mh == 2 ? ",items256=" + std::to_string(p.n_big) + ",items128=" +
                                 std::to_string(p.total_items - p.n_big)
                           : std::string()) +
                ",a=" +
                (a_mn ? "mn" : "k") + "-major,b=" + (b_mn ? "mn" : "k") + "-major" + (swap ? ",swapped" : "") +
                (a_perm ? ",a-prepermuted" : "") + (b_perm ? ",b-prepermuted" : "");
    plan.blob.resize(sizeof tp);
    std::memcpy(plan.blob.data(), &tp, sizeof tp);
    return true;
}

void launch_contraction(contraction_plan_t const& plan,
                        cudaStream_t              stream,
                        void*                     out,
                        void const*               lhs,
                        void const*               rhs,
                        void*                     workspace)
{
    tc_plan_t tp;
    std::memcpy(&tp, plan.blob.data(), sizeof tp);
    tc_params_t& p = tp.p;
    if (tp.swap) std::swap(lhs, rhs);
    if ((reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs)) & 15)
        fail(ES_BAD_ARGUMENT, "tensor-core contraction needs 16-byte aligned operands");
    {
        float* w = static_cast<float*>(workspace);
        auto   blocks = [](uint64_t n4) { return (unsigned)std::min<uint64_t>((n4 + 255) / 256, 148ull * 8); };
        size_t pre = 0;
        auto   stage = [&](void const* src, int perm, uint64_t elems, float* region, CUtensorMap* tm,
                         tc_plan_t::map_recipe_t const& rc) {
            float const* cur = static_cast<float const*>(src);
            if (perm) {
                // generated permutation kernel: (out, x0, workspace)
                plan_t const& pp = plan.pre_plans[pre];
                void*         o = region;
                void*         x = const_cast<void*>(src);
                void*         none = nullptr;
                void*         args[3] = {&o, &x, &none};
                for (size_t i = 0; i != pp.launches.size(); ++i)
                    launch_function(plan.pre_functions[pre][i], pp.launches[i].grid, pp.launches[i].block,
                                    pp.launches[i].smem, stream, args);
                cur = region;
                ++pre;
            }
            if (p.n_terms == 2) {
                float* hi = region;
                float* lo = region + elems;
                launch_k(split_tf32_kernel, dim3(blocks(elems / 4)), dim3(256), 0, stream, cur, hi, lo, elems / 4);
                encode_map(&tm[0], rc, hi, true);
                encode_map(&tm[1], rc, lo, true);
            } else {
                encode_map(&tm[0], rc, cur, true);
                tm[1] = tm[0];
            }
        };
        stage(lhs, tp.a_perm, tp.a_elems, w, p.tm_a, tp.ra);
        stage(rhs, tp.b_perm, tp.b_elems, w + tp.ws_b_offset, p.tm_b, tp.rb);
    }
    p.out_tma = 0;
    if (tp.out_tma && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        encode_map(&p.tm_out, tp.rout, out, true);
        p.out_tma = 1;
    }
    auto launch = [&](auto kernel, int slot) {
        static bool attr_set[4][64] = {};
        int         dev = 0;
        cudaGetDevice(&dev);
        if (!attr_set[slot][dev & 63]) {
            ES_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            attr_set[slot][dev & 63] = true;
        }
        launch_k(kernel, dim3(tp.grid), dim3(NUM_THREADS), tp.smem_bytes, stream, p, out);
    };
    if (tp.kind == 0 && p.mh == 2) launch(tc_contraction_kernel<0, false, true>, 3);
    else if (tp.kind == 0) launch(tc_contraction_kernel<0, false, false>, 0);
    else if (tp.promote) launch(tc_contraction_kernel<1, true, false>, 1);
    else launch(tc_contraction_kernel<1, false, false>, 2);
    ES_CUDA_CHECK(cudaGetLastError());
}

int read_trace(unsigned long long* out, int n)
{
#ifdef ES_B200_TRACE
    if (n > 8000) n = 8000;
    ES_CUDA_CHECK(cudaDeviceSynchronize());
    ES_CUDA_CHECK(cudaMemcpyFromSymbol(out, g_trace, sizeof(unsigned long long) * (size_t)n));
    return n;
#else
    (void)out;
    (void)n;
    return -1;
#endif
}

unsigned int read_and_clear_tc_error()
{
    unsigned int v = 0, zero = 0;
    ES_CUDA_CHECK(cudaMemcpyFromSymbol(&v, g_tc_error, sizeof v));
    if (v) ES_CUDA_CHECK(cudaMemcpyToSymbol(g_tc_error, &zero, sizeof zero));
    return v;
}

} // namespace es
