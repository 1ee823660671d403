// touch_t copy-region kernels, fills and the move pull-copy for sm_100a.
//
// touch: for every index i of the region, out[off_out+i] (=|+=|*=|min=|max=) inn[off_inn+i]
// (semantics of execute_touch, src/engine/touch.cc:155-237).  After
// touch_t::simplify the innermost dim is contiguous on both sides, so the
// region is a set of rows; a row is moved in 16-byte (or narrower, when the
// region's alignment demands) vectors, consecutive threads on consecutive
// vectors of a row, up to three outer dims folded into the flat slot index with
// exact multiply-high divisions.  Replaces touch1..4 of
// src/engine/gpu/cuda_kernels.cu:99-246 (per-element dtype switch, threadIdx.x
// on the slowest dim for rank 3/4).
#include "kernels.h"
#include "pdl.h"

#include <algorithm>
#include <cstring>

namespace es {

namespace {

__host__ fastdiv_t make_fastdiv(uint32_t d)
{
    fastdiv_t f;
    f.d = d;
    f.pad = 0;
    f.m = 0;
    f.s = 0;
    if (d > 1) {
        // with e = m*d - 2^(31+l) in [0, d) and n < 2^31: n*e < 2^(31+l), so the quotient is exact
        uint32_t l = 0;
        while ((1ull << l) < d) ++l;
        f.m = (uint32_t)(((1ull << (31 + l)) + d - 1) / d);
        f.s = l - 1;
    }
    return f;
}

__device__ __forceinline__ uint32_t fdiv(uint32_t n, fastdiv_t const& f)
{
    return f.d <= 1 ? n : (__umulhi(n, f.m) >> f.s);
}

template <int W> struct word_t;
template <> struct word_t<16> { using type = uint4; };
template <> struct word_t<8> { using type = uint2; };
template <> struct word_t<4> { using type = uint32_t; };
template <> struct word_t<2> { using type = uint16_t; };

__device__ __forceinline__ float h2f(uint16_t h)
{
    float f;
    asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h));
    return f;
}
__device__ __forceinline__ uint16_t f2h(float f)
{
    uint16_t h;
    asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f));
    return h;
}

// out <- castable(out, inn), one element.  IEEE operations without fused
// multiply-add so that results equal the CPU executor's bit for bit.
template <int CAST> __device__ __forceinline__ float op_f32(float o, float i)
{
    if constexpr (CAST == ES_CASTABLE_ADD) return __fadd_rn(o, i);
    if constexpr (CAST == ES_CASTABLE_MUL) return __fmul_rn(o, i);
    if constexpr (CAST == ES_CASTABLE_MIN) return (i < o) ? i : o;
    return (o < i) ? i : o;
}
template <int CAST> __device__ __forceinline__ double op_f64(double o, double i)
{
    if constexpr (CAST == ES_CASTABLE_ADD) return __dadd_rn(o, i);
    if constexpr (CAST == ES_CASTABLE_MUL) return __dmul_rn(o, i);
    if constexpr (CAST == ES_CASTABLE_MIN) return (i < o) ? i : o;
    return (o < i) ? i : o;
}
template <int CAST> __device__ __forceinline__ uint16_t op_f16(uint16_t o, uint16_t i)
{
    // f16 (+,*) f16 is exact in f32, so one rounding back equals f16 arithmetic
    return f2h(op_f32<CAST>(h2f(o), h2f(i)));
}
template <int CAST> __device__ __forceinline__ void op_c64(float& ore, float& oim, float ire, float iim)
{
    if constexpr (CAST == ES_CASTABLE_ADD) {
        ore = __fadd_rn(ore, ire);
        oim = __fadd_rn(oim, iim);
    } else {
        float re = __fsub_rn(__fmul_rn(ore, ire), __fmul_rn(oim, iim));
        float im = __fadd_rn(__fmul_rn(ore, iim), __fmul_rn(oim, ire));
        ore = re;
        oim = im;
    }
}

// combine NW 32-bit words
template <int DT, int CAST, int NW>
__device__ __forceinline__ void combine32(uint32_t* o, uint32_t const* i)
{
    if constexpr (DT == ES_F16) {
#pragma unroll
        for (int k = 0; k < NW; ++k) {
            uint16_t lo = op_f16<CAST>((uint16_t)(o[k] & 0xffffu), (uint16_t)(i[k] & 0xffffu));
            uint16_t hi = op_f16<CAST>((uint16_t)(o[k] >> 16), (uint16_t)(i[k] >> 16));
            o[k] = (uint32_t)lo | ((uint32_t)hi << 16);
        }
    } else if constexpr (DT == ES_F32) {
#pragma unroll
        for (int k = 0; k < NW; ++k)
            o[k] = __float_as_uint(op_f32<CAST>(__uint_as_float(o[k]), __uint_as_float(i[k])));
    } else if constexpr (DT == ES_F64) {
#pragma unroll
        for (int k = 0; k < NW; k += 2) {
            double a = __hiloint2double((int)o[k + 1], (int)o[k]);
            double b = __hiloint2double((int)i[k + 1], (int)i[k]);
            double r = op_f64<CAST>(a, b);
            o[k] = (uint32_t)__double2loint(r);
            o[k + 1] = (uint32_t)__double2hiint(r);
        }
    } else {
#pragma unroll
        for (int k = 0; k < NW; k += 2) {
            float re = __uint_as_float(o[k]), im = __uint_as_float(o[k + 1]);
            constexpr int C = CAST == ES_CASTABLE_ADD ? ES_CASTABLE_ADD : ES_CASTABLE_MUL;
            op_c64<C>(re, im, __uint_as_float(i[k]), __uint_as_float(i[k + 1]));
            o[k] = __float_as_uint(re);
            o[k + 1] = __float_as_uint(im);
        }
    }
}

template <int W, int DT, int CAST>
__device__ __forceinline__ typename word_t<W>::type combine(typename word_t<W>::type o,
                                                            typename word_t<W>::type i)
{
    if constexpr (W == 2) {
        return op_f16<CAST>(o, i); // only f16 has 2-byte vectors
    } else {
        constexpr int NW = W / 4;
        uint32_t      ow[NW], iw[NW];
        memcpy(ow, &o, W);
        memcpy(iw, &i, W);
        combine32<DT, CAST, NW>(ow, iw);
        memcpy(&o, ow, W);
        return o;
    }
}

constexpr int TOUCH_UNROLL = 4;
constexpr int TOUCH_BLOCK = 256;

template <int W>
__device__ __forceinline__ bool
touch_locate(touch_args_t const& a, uint32_t slot, char const*& pin, char*& pout)
{
    if (slot >= (uint32_t)a.total_slots) return false;
    uint32_t seg = slot >> a.seg_shift;
    uint32_t lane = slot & ((1u << a.seg_shift) - 1u);
    uint32_t row = fdiv(seg, a.div_segs);
    uint32_t col = ((seg - row * a.segs_per_row) << a.seg_shift) + lane;
    if (col >= a.row_vecs) return false;
    uint32_t t = fdiv(row, a.div_n2);
    uint32_t i2 = row - t * a.div_n2.d;
    uint32_t i0 = fdiv(t, a.div_n1);
    uint32_t i1 = t - i0 * a.div_n1.d;
    uint64_t cb = (uint64_t)col * W;
    pin = a.inn + i0 * a.sin[0] + i1 * a.sin[1] + i2 * a.sin[2] + cb;
    pout = a.out + i0 * a.sout[0] + i1 * a.sout[1] + i2 * a.sout[2] + cb;
    return true;
}

template <int W, int DT, int CAST>
__device__ __forceinline__ void touch_body(touch_args_t const& a, uint32_t slot0, uint32_t stride)
{
    using V = typename word_t<W>::type;
    V     vi[TOUCH_UNROLL], vo[TOUCH_UNROLL];
    char* po[TOUCH_UNROLL];
    bool  ok[TOUCH_UNROLL];
#pragma unroll
    for (int u = 0; u < TOUCH_UNROLL; ++u) {
        char const* pi;
        ok[u] = touch_locate<W>(a, slot0 + u * stride, pi, po[u]);
        if (ok[u]) {
            vi[u] = *reinterpret_cast<V const*>(pi);
            if constexpr (CAST != ES_CASTABLE_NONE) vo[u] = *reinterpret_cast<V const*>(po[u]);
        }
    }
#pragma unroll
    for (int u = 0; u < TOUCH_UNROLL; ++u) {
        if (ok[u]) {
            if constexpr (CAST == ES_CASTABLE_NONE) *reinterpret_cast<V*>(po[u]) = vi[u];
            else *reinterpret_cast<V*>(po[u]) = combine<W, DT, CAST>(vo[u], vi[u]);
        }
    }
}

template <int W, int DT>
__device__ __forceinline__ void touch_dispatch(touch_args_t const& a, uint32_t slot0, uint32_t stride)
{
    switch (a.castable) {
        case ES_CASTABLE_NONE: touch_body<W, DT, ES_CASTABLE_NONE>(a, slot0, stride); break;
        case ES_CASTABLE_ADD: touch_body<W, DT, ES_CASTABLE_ADD>(a, slot0, stride); break;
        case ES_CASTABLE_MUL: touch_body<W, DT, ES_CASTABLE_MUL>(a, slot0, stride); break;
        case ES_CASTABLE_MIN:
            if constexpr (DT != ES_C64) touch_body<W, DT, ES_CASTABLE_MIN>(a, slot0, stride);
            break;
        case ES_CASTABLE_MAX:
            if constexpr (DT != ES_C64) touch_body<W, DT, ES_CASTABLE_MAX>(a, slot0, stride);
            break;
    }
}

// one touch; the descriptor travels in the kernel parameters
template <int W, int DT>
__global__ void __launch_bounds__(TOUCH_BLOCK) touch_kernel(const __grid_constant__ touch_args_t a)
{
    ES_PDL_PROLOGUE();
    uint32_t slot0 = blockIdx.x * (TOUCH_BLOCK * TOUCH_UNROLL) + threadIdx.x;
    touch_dispatch<W, DT>(a, slot0, TOUCH_BLOCK);
    if (a.done != nullptr) {
        // input read from a peer GPU: tell it when the last CTA has finished reading
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            uint32_t old = atomicAdd(a.counter, 1u);
            if (old == gridDim.x - 1) {
                *a.counter = 0;
                uint32_t e = *a.epoch;
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.done), "r"(e) : "memory");
            }
        }
    }
}

// many touches; blockIdx.y selects the descriptor in device memory
template <int W, int DT>
__global__ void __launch_bounds__(TOUCH_BLOCK) touch_batch_kernel(touch_args_t const* items)
{
    ES_PDL_PROLOGUE();
    __shared__ touch_args_t a;
    {
        uint32_t const* src = reinterpret_cast<uint32_t const*>(items + blockIdx.y);
        uint32_t*       dst = reinterpret_cast<uint32_t*>(&a);
        for (int i = threadIdx.x; i < (int)(sizeof(touch_args_t) / 4); i += TOUCH_BLOCK) dst[i] = src[i];
    }
    __syncthreads();
    uint32_t slot0 = blockIdx.x * (TOUCH_BLOCK * TOUCH_UNROLL) + threadIdx.x;
    if ((uint64_t)blockIdx.x * (TOUCH_BLOCK * TOUCH_UNROLL) >= a.total_slots) return;
    touch_dispatch<W, DT>(a, slot0, TOUCH_BLOCK);
}

template <typename T> __global__ void fill_constant_kernel(T* out, T v, uint64_t n)
{
    ES_PDL_PROLOGUE();
    // 16-byte stores over the aligned body, scalar head/tail
    constexpr int PER = 16 / sizeof(T);
    uint64_t      head = ((16 - (reinterpret_cast<uintptr_t>(out) & 15)) & 15) / sizeof(T);
    if (head > n) head = n;
    uint64_t body = (n - head) / PER;
    uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t nth = (uint64_t)gridDim.x * blockDim.x;
    struct alignas(16) pack_t { T v[PER]; };
    pack_t p;
#pragma unroll
    for (int i = 0; i < PER; ++i) p.v[i] = v;
    pack_t* o16 = reinterpret_cast<pack_t*>(out + head);
    for (uint64_t i = tid; i < body; i += nth) o16[i] = p;
    uint64_t tail0 = head + body * PER;
    for (uint64_t i = tid; i < head; i += nth) out[i] = v;
    for (uint64_t i = tail0 + tid; i < n; i += nth) out[i] = v;
}

// out[i,j] = (i - start >= j) ? lower : upper   (reference_fill,
// src/einsummable/reference.cc:485-508; start is signed)
template <typename T>
__global__ void fill_lowertri_kernel(T* out, T lower, T upper, int64_t nrow, int64_t ncol, int64_t start)
{
    ES_PDL_PROLOGUE();
    int64_t n = nrow * ncol;
    int64_t nth = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += nth) {
        int64_t i = e / ncol;
        int64_t j = e - i * ncol;
        out[e] = (i - start >= j) ? lower : upper;
    }
}

__global__ void __launch_bounds__(256) pull_copy_kernel(uint4 const* __restrict__ src,
                                                        uint4* __restrict__ dst,
                                                        uint64_t n16,
                                                        unsigned char const* __restrict__ src_tail,
                                                        unsigned char* __restrict__ dst_tail,
                                                        uint32_t ntail)
{
    ES_PDL_PROLOGUE();
    uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t nth = (uint64_t)gridDim.x * blockDim.x;
    uint64_t i = tid;
    // 4 loads in flight per thread
    for (; i + 3 * nth < n16; i += 4 * nth) {
        uint4 a = src[i], b = src[i + nth], c = src[i + 2 * nth], d = src[i + 3 * nth];
        dst[i] = a;
        dst[i + nth] = b;
        dst[i + 2 * nth] = c;
        dst[i + 3 * nth] = d;
    }
    for (; i < n16; i += nth) dst[i] = src[i];
    if (tid < ntail) dst_tail[tid] = src_tail[tid];
}

__device__ unsigned int g_flag_error; // 1 = a signal gave up, 2 = a wait gave up

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

// expected: the value the flag must have before it is flipped to `next`
__global__ void flag_kernel(uint32_t* flag, uint32_t expected, uint32_t next, unsigned long long limit_cycles,
                            unsigned int code)
{
    ES_PDL_PROLOGUE();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    long long t0 = clock64();
    while (ld_acquire_sys(flag) != expected) {
        if ((unsigned long long)(clock64() - t0) > limit_cycles) {
            atomicCAS(&g_flag_error, 0u, code);
            return; // give up: the flag is left alone, the stream goes on, the host sees the error word
        }
        __nanosleep(64);
    }
    __threadfence_system();
    st_release_sys(flag, next);
}

uint32_t ceil_log2(uint32_t v)
{
    uint32_t s = 0;
    while ((1u << s) < v) ++s;
    return s;
}

void finish_args(touch_args_t& a, uint32_t n0, uint32_t n1, uint32_t n2, uint64_t row_vecs)
{
    if (row_vecs > 0xffffffffull) fail(ES_NOT_SUPPORTED, "touch row too long");
    a.row_vecs = (uint32_t)row_vecs;
    uint32_t seg = std::min<uint64_t>(256, 1ull << ceil_log2((uint32_t)std::max<uint64_t>(row_vecs, 1)));
    a.seg_shift = ceil_log2(seg);
    a.segs_per_row = (uint32_t)((row_vecs + seg - 1) / seg);
    uint64_t rows = (uint64_t)n0 * n1 * n2;
    if (rows > 0x7fffffffull || ((rows * a.segs_per_row) << a.seg_shift) >= 0x7fffffffull)
        fail(ES_NOT_SUPPORTED, "touch region too large for one launch (2^31 vectors)");
    a.n_rows = (uint32_t)rows;
    a.div_n1 = make_fastdiv(n1);
    a.div_n2 = make_fastdiv(n2);
    a.div_segs = make_fastdiv(a.segs_per_row);
    a.total_slots = (rows * a.segs_per_row) << a.seg_shift;
}

} // namespace

int simplify_touch(es_touchdim_t const* dims, int rank, es_touchdim_t* out)
{
    if (rank < 1) fail(ES_BAD_DESCRIPTOR, "touch rank must be >= 1");
    int r = 0;
    out[r++] = dims[0];
    for (int i = 1; i != rank; ++i) {
        es_touchdim_t const& td = dims[i];
        bool dummy = td.d_inn == td.d_out && td.offset_inn == 0 && td.offset_out == 0 &&
                     td.d_inn == td.size;
        if (dummy) {
            es_touchdim_t& b = out[r - 1];
            b.d_inn *= td.d_inn;
            b.d_out *= td.d_inn;
            b.offset_inn *= td.d_inn;
            b.offset_out *= td.d_inn;
            b.size *= td.d_inn;
        } else {
            out[r++] = td;
        }
    }
    return r;
}

int prepare_touch(es_touchdim_t const* dims_in,
                  int                  rank_in,
                  int                  castable,
                  int                  dtype,
                  void*                out,
                  void const*          inn,
                  touch_args_t&        a)
{
    if (!dims_in || rank_in < 1 || rank_in > 16) fail(ES_BAD_DESCRIPTOR, "touch: bad rank");
    if (!out || !inn) fail(ES_BAD_ARGUMENT, "touch: null pointer");
    if (castable < -1 || castable > 3) fail(ES_BAD_DESCRIPTOR, "touch: bad castable");
    if (dtype == ES_C64 && (castable == ES_CASTABLE_MIN || castable == ES_CASTABLE_MAX))
        fail(ES_BAD_DESCRIPTOR, "touch: min/max castable is not defined for complex");
    uint64_t ds = dtype_size(dtype);
    for (int i = 0; i != rank_in; ++i) {
        es_touchdim_t const& td = dims_in[i];
        if (td.size == 0 || td.offset_inn + td.size > td.d_inn || td.offset_out + td.size > td.d_out)
            fail(ES_BAD_DESCRIPTOR, "touch: region exceeds a dimension (or is empty)");
    }
    es_touchdim_t d[16];
    int           rank = simplify_touch(dims_in, rank_in, d);
    if (rank > 4) fail(ES_NOT_SUPPORTED, "touch: more than 4 dims remain after simplify");

    // element strides of every dim, row-major
    uint64_t sin[4], sout[4];
    {
        uint64_t si = 1, so = 1;
        for (int i = rank - 1; i >= 0; --i) {
            sin[i] = si;
            sout[i] = so;
            si *= d[i].d_inn;
            so *= d[i].d_out;
        }
    }
    uint64_t off_in = 0, off_out = 0;
    for (int i = 0; i != rank; ++i) {
        off_in += d[i].offset_inn * sin[i];
        off_out += d[i].offset_out * sout[i];
    }
    std::memset(&a, 0, sizeof a);
    a.inn = static_cast<char const*>(inn) + off_in * ds;
    a.out = static_cast<char*>(out) + off_out * ds;
    a.castable = castable;
    // outer dims -> slots 0..2 (right-aligned so that slot 2 is the dim next to the row)
    uint32_t n[3] = {1, 1, 1};
    for (int i = 0; i != rank - 1; ++i) {
        int slot = 3 - (rank - 1) + i;
        if (d[i].size > 0xffffffffull) fail(ES_NOT_SUPPORTED, "touch: dim too large");
        n[slot] = (uint32_t)d[i].size;
        a.sin[slot] = sin[i] * ds;
        a.sout[slot] = sout[i] * ds;
    }
    uint64_t row_bytes = d[rank - 1].size * ds;
    // widest vector width every row start and the row length are multiples of
    uint64_t bits = reinterpret_cast<uintptr_t>(a.inn) | reinterpret_cast<uintptr_t>(a.out) | row_bytes;
    for (int s = 0; s != 3; ++s)
        if (n[s] > 1) bits |= a.sin[s] | a.sout[s];
    int w = 16;
    while (w > (int)ds && (bits & (uint64_t)(w - 1))) w /= 2;
    if (bits & (ds - 1)) fail(ES_BAD_ARGUMENT, "touch: pointer not aligned to the element size");
    // stash n0 (needed by narrow_touch) in pad-free fields: n_rows/n1/n2 recover it
    finish_args(a, n[0], n[1], n[2], row_bytes / w);
    return w;
}

void narrow_touch(touch_args_t& a, int w_from, int w_to)
{
    if (w_to == w_from) return;
    uint64_t row_vecs = (uint64_t)a.row_vecs * w_from / w_to;
    uint32_t n1 = a.div_n1.d, n2 = a.div_n2.d;
    uint32_t n0 = a.n_rows / (n1 * n2);
    finish_args(a, n0, n1, n2, row_vecs);
}

template <int W, int DT> static void launch_touch_wd(touch_args_t const& a, cudaStream_t s)
{
    uint64_t per = (uint64_t)TOUCH_BLOCK * TOUCH_UNROLL;
    uint64_t grid = (a.total_slots + per - 1) / per;
    if (grid > 0x7fffffffull) fail(ES_NOT_SUPPORTED, "touch grid too large");
    launch_k(touch_kernel<W, DT>, dim3((unsigned)grid), dim3(TOUCH_BLOCK), 0, s, a);
}

template <int W, int DT>
static void launch_batch_wd(touch_args_t const* items, int n, uint64_t max_slots, cudaStream_t s)
{
    uint64_t per = (uint64_t)TOUCH_BLOCK * TOUCH_UNROLL;
    uint64_t gx = (max_slots + per - 1) / per;
    if (gx > 0x7fffffffull || n > 65535) fail(ES_NOT_SUPPORTED, "touch batch grid too large");
    dim3 grid((unsigned)gx, (unsigned)n, 1);
    launch_k(touch_batch_kernel<W, DT>, grid, dim3(TOUCH_BLOCK), 0, s, items);
}

#define ES_TOUCH_SWITCH(FN, ...)                                                                   \
    switch (dtype) {                                                                               \
        case ES_F16:                                                                               \
            switch (width) {                                                                       \
                case 16: FN<16, ES_F16>(__VA_ARGS__); break;                                       \
                case 8: FN<8, ES_F16>(__VA_ARGS__); break;                                         \
                case 4: FN<4, ES_F16>(__VA_ARGS__); break;                                         \
                default: FN<2, ES_F16>(__VA_ARGS__); break;                                        \
            }                                                                                      \
            break;                                                                                 \
        case ES_F32:                                                                               \
            switch (width) {                                                                       \
                case 16: FN<16, ES_F32>(__VA_ARGS__); break;                                       \
                case 8: FN<8, ES_F32>(__VA_ARGS__); break;                                         \
                default: FN<4, ES_F32>(__VA_ARGS__); break;                                        \
            }                                                                                      \
            break;                                                                                 \
        case ES_F64:                                                                               \
            if (width == 16) FN<16, ES_F64>(__VA_ARGS__);                                          \
            else FN<8, ES_F64>(__VA_ARGS__);                                                       \
            break;                                                                                 \
        default:                                                                                   \
            if (width == 16) FN<16, ES_C64>(__VA_ARGS__);                                          \
            else FN<8, ES_C64>(__VA_ARGS__);                                                       \
            break;                                                                                 \
    }

void launch_touch(touch_args_t const& a, int width, int dtype, cudaStream_t stream)
{
    ES_TOUCH_SWITCH(launch_touch_wd, a, stream);
    ES_CUDA_CHECK(cudaGetLastError());
}

void launch_touch_batch(touch_args_t const* items_dev,
                        int                 n,
                        uint64_t            max_slots,
                        int                 width,
                        int                 dtype,
                        cudaStream_t        stream)
{
    ES_TOUCH_SWITCH(launch_batch_wd, items_dev, n, max_slots, stream);
    ES_CUDA_CHECK(cudaGetLastError());
}

template <typename T> static void fill_const_t(void* out, void const* v8, uint64_t n, cudaStream_t s)
{
    T v;
    std::memcpy(&v, v8, sizeof(T));
    uint64_t per = 16 / sizeof(T);
    uint64_t blocks = std::min<uint64_t>((n / per + 255) / 256 + 1, 148ull * 8);
    launch_k(fill_constant_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, s, static_cast<T*>(out), v, n);
}

void launch_fill_constant(int dtype, void const* value8, uint64_t nelem, cudaStream_t s, void* out)
{
    if (!out || !value8) fail(ES_BAD_ARGUMENT, "fill: null pointer");
    if (nelem == 0) return;
    switch (dtype) {
        case ES_F16: fill_const_t<uint16_t>(out, value8, nelem, s); break;
        case ES_F32: fill_const_t<uint32_t>(out, value8, nelem, s); break;
        case ES_F64:
        case ES_C64: fill_const_t<uint64_t>(out, value8, nelem, s); break;
        default: fail(ES_BAD_DESCRIPTOR, "fill: bad dtype");
    }
    ES_CUDA_CHECK(cudaGetLastError());
}

template <typename T>
static void fill_tri_t(void* out, void const* lo8, void const* up8, uint64_t nrow, uint64_t ncol,
                       int64_t start, cudaStream_t s)
{
    T lo, up;
    std::memcpy(&lo, lo8, sizeof(T));
    std::memcpy(&up, up8, sizeof(T));
    uint64_t n = nrow * ncol;
    uint64_t blocks = std::min<uint64_t>((n + 255) / 256, 148ull * 8);
    launch_k(fill_lowertri_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, s, static_cast<T*>(out), lo, up,
                                                            (int64_t)nrow, (int64_t)ncol, start);
}

void launch_fill_lowertri(int          dtype,
                          void const*  lower8,
                          void const*  upper8,
                          uint64_t     nrow,
                          uint64_t     ncol,
                          int64_t      start,
                          cudaStream_t s,
                          void*        out)
{
    if (!out || !lower8 || !upper8) fail(ES_BAD_ARGUMENT, "fill: null pointer");
    if (nrow == 0 || ncol == 0) return;
    if (nrow > (1ull << 40) || ncol > (1ull << 40)) fail(ES_BAD_DESCRIPTOR, "fill: shape too large");
    switch (dtype) {
        case ES_F16: fill_tri_t<uint16_t>(out, lower8, upper8, nrow, ncol, start, s); break;
        case ES_F32: fill_tri_t<uint32_t>(out, lower8, upper8, nrow, ncol, start, s); break;
        case ES_F64:
        case ES_C64: fill_tri_t<uint64_t>(out, lower8, upper8, nrow, ncol, start, s); break;
        default: fail(ES_BAD_DESCRIPTOR, "fill: bad dtype");
    }
    ES_CUDA_CHECK(cudaGetLastError());
}

static unsigned long long limit_cycles(uint32_t limit_ms)
{
    // clock64 ticks at the SM clock (<= ~2 GHz here); the limit is an upper bound, not a timer
    return (unsigned long long)(limit_ms ? limit_ms : 2000) * 2000000ull;
}

void launch_flag_signal(uint32_t* flag, uint32_t limit_ms, cudaStream_t s)
{
    if (!flag || (reinterpret_cast<uintptr_t>(flag) & 3)) fail(ES_BAD_ARGUMENT, "flag: null or unaligned pointer");
    launch_k(flag_kernel, dim3(1), dim3(32), 0, s, flag, 0u, 1u, limit_cycles(limit_ms), 1u);
    ES_CUDA_CHECK(cudaGetLastError());
}

void launch_flag_wait(uint32_t* flag, uint32_t limit_ms, cudaStream_t s)
{
    if (!flag || (reinterpret_cast<uintptr_t>(flag) & 3)) fail(ES_BAD_ARGUMENT, "flag: null or unaligned pointer");
    launch_k(flag_kernel, dim3(1), dim3(32), 0, s, flag, 1u, 0u, limit_cycles(limit_ms), 2u);
    ES_CUDA_CHECK(cudaGetLastError());
}

unsigned int read_and_clear_flag_error()
{
    unsigned int v = 0, zero = 0;
    ES_CUDA_CHECK(cudaMemcpyFromSymbol(&v, g_flag_error, sizeof v));
    if (v) ES_CUDA_CHECK(cudaMemcpyToSymbol(g_flag_error, &zero, sizeof zero));
    return v;
}

void launch_pull_copy(void const* src, void* dst, uint64_t bytes, cudaStream_t s)
{
    if (bytes == 0) return;
    bool     aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
    uint64_t n16 = aligned ? bytes / 16 : 0;
    uint64_t tail = bytes - n16 * 16;
    if (tail > 0xffffffffull) fail(ES_NOT_SUPPORTED, "unaligned move too large for the pull kernel");
    uint64_t blocks = std::max<uint64_t>(std::min<uint64_t>((n16 + 1023) / 1024, 148ull * 4),
                                         (tail + 255) / 256);
    blocks = std::max<uint64_t>(blocks, 1);
    launch_k(pull_copy_kernel, dim3((unsigned)blocks), dim3(256), 0, s,
        static_cast<uint4 const*>(src), static_cast<uint4*>(dst), n16,
        static_cast<unsigned char const*>(src) + n16 * 16,
        static_cast<unsigned char*>(dst) + n16 * 16, (uint32_t)tail);
    ES_CUDA_CHECK(cudaGetLastError());
}

} // namespace es
