#include "codegen.h"

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <limits>

namespace es {

namespace {

// ---------------------------------------------------------------------------
// Device-side helpers shared by every generated kernel.  No CUDA headers are
// included: f16 is handled as raw 16-bit words with cvt instructions, so a
// kernel compiles in a few tens of milliseconds.
// ---------------------------------------------------------------------------
char const* const k_preamble = R"PRE(
typedef unsigned short u16;
typedef unsigned int u32;
typedef unsigned long long u64;
struct __align__(8) cf { float re, im; };
__device__ __forceinline__ cf cf_make(float a, float b) { cf r; r.re = a; r.im = b; return r; }
__device__ __forceinline__ cf cf_add(cf a, cf b) { return cf_make(a.re + b.re, a.im + b.im); }
__device__ __forceinline__ cf cf_mul(cf a, cf b) {
    return cf_make(a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re);
}
__device__ __forceinline__ cf cf_conj(cf a) { return cf_make(a.re, -a.im); }
template <typename T> __device__ __forceinline__ T es_sq(T x) { return x * x; }
template <typename T> __device__ __forceinline__ T es_cube(T x) { return x * x * x; }
__device__ __forceinline__ float es_h2f(u16 h) {
    float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h)); return f;
}
__device__ __forceinline__ u16 es_f2h(float f) {
    u16 h; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h;
}
__device__ __forceinline__ float es_rt_h(float f) { return es_h2f(es_f2h(f)); }
__device__ __forceinline__ void es_unpack2(u32 w, float& a, float& b) {
    asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %2; cvt.f32.f16 %0, lo; cvt.f32.f16 %1, hi;}"
        : "=f"(a), "=f"(b) : "r"(w));
}
__device__ __forceinline__ u32 es_pack2(float a, float b) {
    u32 w; asm("cvt.rn.f16x2.f32 %0, %2, %1;" : "=r"(w) : "f"(a), "f"(b)); return w;
}
// ---- loads: V elements of a storage type into an array of the compute type ----
template <int V> __device__ __forceinline__ void ld_f16(const u16* p, float* o) {
    if constexpr (V == 1) { o[0] = es_h2f(*p); }
    else if constexpr (V == 2) { u32 w = *(const u32*)p; es_unpack2(w, o[0], o[1]); }
    else if constexpr (V == 4) {
        uint2 w = *(const uint2*)p; es_unpack2(w.x, o[0], o[1]); es_unpack2(w.y, o[2], o[3]);
    } else {
        uint4 w = *(const uint4*)p;
        es_unpack2(w.x, o[0], o[1]); es_unpack2(w.y, o[2], o[3]);
        es_unpack2(w.z, o[4], o[5]); es_unpack2(w.w, o[6], o[7]);
        if constexpr (V > 8) ld_f16<V - 8>(p + 8, o + 8);
    }
}
template <int V> __device__ __forceinline__ void ld_f32(const float* p, float* o) {
    if constexpr (V == 1) { o[0] = *p; }
    else if constexpr (V == 2) { float2 w = *(const float2*)p; o[0] = w.x; o[1] = w.y; }
    else {
        float4 w = *(const float4*)p; o[0] = w.x; o[1] = w.y; o[2] = w.z; o[3] = w.w;
        if constexpr (V > 4) ld_f32<V - 4>(p + 4, o + 4);
    }
}
template <int V> __device__ __forceinline__ void ld_f64(const double* p, double* o) {
    if constexpr (V == 1) { o[0] = *p; }
    else {
        double2 w = *(const double2*)p; o[0] = w.x; o[1] = w.y;
        if constexpr (V > 2) ld_f64<V - 2>(p + 2, o + 2);
    }
}
template <int V> __device__ __forceinline__ void ld_c64(const cf* p, cf* o) {
    if constexpr (V == 1) { float2 w = *(const float2*)p; o[0] = cf_make(w.x, w.y); }
    else {
        float4 w = *(const float4*)p; o[0] = cf_make(w.x, w.y); o[1] = cf_make(w.z, w.w);
        if constexpr (V > 2) ld_c64<V - 2>(p + 2, o + 2);
    }
}
// ---- raw (packed) loads: data stays packed in registers until it is used ----
template <int BYTES> struct raw_t { uint4 q[BYTES / 16]; };
template <> struct raw_t<8> { uint2 q[1]; };
template <> struct raw_t<4> { u32 q[1]; };
template <> struct raw_t<2> { u16 q[1]; };
template <int BYTES> __device__ __forceinline__ void ld_raw(const void* p, raw_t<BYTES>& r) {
    if constexpr (BYTES >= 16) {
#pragma unroll
        for (int i = 0; i < BYTES / 16; ++i) r.q[i] = ((const uint4*)p)[i];
    } else if constexpr (BYTES == 8) { r.q[0] = *(const uint2*)p; }
    else if constexpr (BYTES == 4) { r.q[0] = *(const u32*)p; }
    else { r.q[0] = *(const u16*)p; }
}
template <int V> __device__ __forceinline__ void cv_f16(const raw_t<2 * V>& r, float* o) {
    if constexpr (V == 1) { o[0] = es_h2f(r.q[0]); }
    else if constexpr (V == 2) { es_unpack2(r.q[0], o[0], o[1]); }
    else if constexpr (V == 4) { es_unpack2(r.q[0].x, o[0], o[1]); es_unpack2(r.q[0].y, o[2], o[3]); }
    else {
#pragma unroll
        for (int i = 0; i < V / 8; ++i) {
            es_unpack2(r.q[i].x, o[8 * i + 0], o[8 * i + 1]); es_unpack2(r.q[i].y, o[8 * i + 2], o[8 * i + 3]);
            es_unpack2(r.q[i].z, o[8 * i + 4], o[8 * i + 5]); es_unpack2(r.q[i].w, o[8 * i + 6], o[8 * i + 7]);
        }
    }
}
template <int V> __device__ __forceinline__ void cv_f32(const raw_t<4 * V>& r, float* o) {
    if constexpr (V == 1) { o[0] = __uint_as_float(r.q[0]); }
    else if constexpr (V == 2) { o[0] = __uint_as_float(r.q[0].x); o[1] = __uint_as_float(r.q[0].y); }
    else {
#pragma unroll
        for (int i = 0; i < V / 4; ++i) {
            o[4 * i + 0] = __uint_as_float(r.q[i].x); o[4 * i + 1] = __uint_as_float(r.q[i].y);
            o[4 * i + 2] = __uint_as_float(r.q[i].z); o[4 * i + 3] = __uint_as_float(r.q[i].w);
        }
    }
}
template <int V> __device__ __forceinline__ void cv_f64(const raw_t<8 * V>& r, double* o) {
    if constexpr (V == 1) { o[0] = __hiloint2double((int)r.q[0].y, (int)r.q[0].x); }
    else {
#pragma unroll
        for (int i = 0; i < V / 2; ++i) {
            o[2 * i + 0] = __hiloint2double((int)r.q[i].y, (int)r.q[i].x);
            o[2 * i + 1] = __hiloint2double((int)r.q[i].w, (int)r.q[i].z);
        }
    }
}
template <int V> __device__ __forceinline__ void cv_c64(const raw_t<8 * V>& r, cf* o) {
    if constexpr (V == 1) { o[0] = cf_make(__uint_as_float(r.q[0].x), __uint_as_float(r.q[0].y)); }
    else {
#pragma unroll
        for (int i = 0; i < V / 2; ++i) {
            o[2 * i + 0] = cf_make(__uint_as_float(r.q[i].x), __uint_as_float(r.q[i].y));
            o[2 * i + 1] = cf_make(__uint_as_float(r.q[i].z), __uint_as_float(r.q[i].w));
        }
    }
}
__device__ __forceinline__ float es_rcp_approx(float x) {
    float r; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r;
}
// ---- stores ----
template <int V> __device__ __forceinline__ void st_f16(u16* p, const float* o) {
    if constexpr (V == 1) { *p = es_f2h(o[0]); }
    else if constexpr (V == 2) { *(u32*)p = es_pack2(o[0], o[1]); }
    else if constexpr (V == 4) {
        uint2 w; w.x = es_pack2(o[0], o[1]); w.y = es_pack2(o[2], o[3]); *(uint2*)p = w;
    } else {
        uint4 w; w.x = es_pack2(o[0], o[1]); w.y = es_pack2(o[2], o[3]);
        w.z = es_pack2(o[4], o[5]); w.w = es_pack2(o[6], o[7]); *(uint4*)p = w;
        if constexpr (V > 8) st_f16<V - 8>(p + 8, o + 8);
    }
}
template <int V> __device__ __forceinline__ void st_f32(float* p, const float* o) {
    if constexpr (V == 1) { *p = o[0]; }
    else if constexpr (V == 2) { *(float2*)p = make_float2(o[0], o[1]); }
    else {
        *(float4*)p = make_float4(o[0], o[1], o[2], o[3]);
        if constexpr (V > 4) st_f32<V - 4>(p + 4, o + 4);
    }
}
template <int V> __device__ __forceinline__ void st_f64(double* p, const double* o) {
    if constexpr (V == 1) { *p = o[0]; }
    else {
        *(double2*)p = make_double2(o[0], o[1]);
        if constexpr (V > 2) st_f64<V - 2>(p + 2, o + 2);
    }
}
template <int V> __device__ __forceinline__ void st_c64(cf* p, const cf* o) {
    if constexpr (V == 1) { *(float2*)p = make_float2(o[0].re, o[0].im); }
    else {
        *(float4*)p = make_float4(o[0].re, o[0].im, o[1].re, o[1].im);
        if constexpr (V > 2) st_c64<V - 2>(p + 2, o + 2);
    }
}
// ---- warp shuffles of the compute types ----
__device__ __forceinline__ float es_shx(float v, int o) { return __shfl_xor_sync(0xffffffffu, v, o); }
__device__ __forceinline__ double es_shx(double v, int o) { return __shfl_xor_sync(0xffffffffu, v, o); }
__device__ __forceinline__ cf es_shx(cf v, int o) {
    return cf_make(__shfl_xor_sync(0xffffffffu, v.re, o), __shfl_xor_sync(0xffffffffu, v.im, o));
}
)PRE";

struct src_t {
    std::string s;
    void        add(char const* fmt, ...) __attribute__((format(printf, 2, 3)))
    {
        char    buf[4096];
        va_list ap;
        va_start(ap, fmt);
        int n = std::vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        if (n < 0 || n >= (int)sizeof buf) fail(ES_COMPILE_ERROR, "codegen line too long");
        s += buf;
        s += "\n";
    }
    void raw(std::string const& t) { s += t; s += "\n"; }
};

char const* dt_suffix(int d)
{
    switch (d) {
        case ES_F16: return "f16";
        case ES_F32: return "f32";
        case ES_F64: return "f64";
        case ES_C64: return "c64";
    }
    return "?";
}

std::string u64s(uint64_t v)
{
    return std::to_string(v);
}

// literal of the index type
std::string idx_lit(uint64_t v, bool wide)
{
    return std::to_string(v) + (wide ? "ull" : "u");
}

std::string identity_literal(int castable, int dtype)
{
    double const inf = std::numeric_limits<double>::infinity();
    switch (castable) {
        case ES_CASTABLE_ADD: return literal(dtype, 0.0, 0.0);
        case ES_CASTABLE_MUL: return literal(dtype, 1.0, 0.0);
        case ES_CASTABLE_MIN: return literal(dtype == ES_F16 ? ES_F32 : dtype, inf);
        case ES_CASTABLE_MAX: return literal(dtype == ES_F16 ? ES_F32 : dtype, -inf);
    }
    fail(ES_BAD_DESCRIPTOR, "identity: bad castable");
}

// acc <- combine(acc, v), following the reference's update order
// (std::min(out, inn) / std::max(out, inn), src/engine/cpu/kernel_executor.cc:1194-1195)
std::string combine_expr(int castable, int dtype, std::string const& acc, std::string const& v)
{
    bool c = dtype == ES_C64;
    switch (castable) {
        case ES_CASTABLE_ADD: return c ? "cf_add(" + acc + "," + v + ")" : "(" + acc + "+" + v + ")";
        case ES_CASTABLE_MUL: return c ? "cf_mul(" + acc + "," + v + ")" : "(" + acc + "*" + v + ")";
        case ES_CASTABLE_MIN: return "((" + v + "<" + acc + ")?" + v + ":" + acc + ")";
        case ES_CASTABLE_MAX: return "((" + acc + "<" + v + ")?" + v + ":" + acc + ")";
    }
    fail(ES_BAD_DESCRIPTOR, "combine: bad castable");
}

struct ctx_t {
    einsum_t const&                    e;
    int                                r;        // join rank
    int                                n;        // number of inputs
    bool                               wide;     // 64-bit index arithmetic
    std::vector<std::vector<uint64_t>> st;       // st[k][m]
    std::vector<uint64_t>              ost;

    explicit ctx_t(einsum_t const& e_) : e(e_), r(e_.join_rank()), n((int)e_.inns.size())
    {
        uint64_t big = e.join_nelem();
        for (int k = 0; k != n; ++k) {
            st.push_back(e.inn_strides(k));
            big = std::max(big, e.inn_nelem(k));
        }
        ost = e.out_strides();
        wide = big >= (1ull << 31);
    }
    char const* idx() const { return wide ? "u64" : "u32"; }
    std::string lit(uint64_t v) const { return idx_lit(v, wide); }

    bool has_mode(int k, int m) const { return st[k][m] != 0; }

    // kernel signature + typed pointer prologue
    void signature(src_t& s, char const* name, int block) const
    {
        std::string args = "void* out_";
        for (int k = 0; k != n; ++k) args += ", const void* x" + std::to_string(k) + "_";
        args += ", void* ws_";
        s.add("extern \"C\" __global__ void __launch_bounds__(%d) %s(%s) {", block, name,
              args.c_str());
        // programmatic dependent launch (see pdl.h): release the next kernel of the lane, then wait
        // for the one before; both are no-ops for ordinary launches
        s.add("  asm volatile(\"griddepcontrol.launch_dependents;\");");
        s.add("  asm volatile(\"griddepcontrol.wait;\" ::: \"memory\");");
        s.add("  %s* out = (%s*)out_;", storage_type(e.out_dtype()), storage_type(e.out_dtype()));
        for (int k = 0; k != n; ++k) {
            char const* t = storage_type(e.inn_dtype(k));
            s.add("  const %s* x%d = (const %s*)x%d_;", t, k, t, k);
        }
    }

    // emit "idx i{m} = ..." for modes [lo, hi) from the flat index `flat`
    void decompose(src_t& s, char const* flat, int lo, int hi, char const* indent) const
    {
        if (hi - lo == 1) {
            s.add("%sconst %s i%d = %s;", indent, idx(), lo, flat);
            return;
        }
        s.add("%s%s t_%d = %s;", indent, idx(), lo, flat);
        for (int m = hi - 1; m > lo; --m) {
            s.add("%sconst %s i%d = t_%d %% %s; t_%d /= %s;", indent, idx(), m, lo,
                  lit(e.join_shape[m]).c_str(), lo, lit(e.join_shape[m]).c_str());
        }
        s.add("%sconst %s i%d = t_%d;", indent, idx(), lo, lo);
    }

    // "i0*S0+i2*S2" over modes [lo,hi) present in input k; "0" when none
    std::string offset_expr(std::vector<uint64_t> const& strides, int lo, int hi) const
    {
        std::string o;
        for (int m = lo; m != hi; ++m) {
            if (strides[m] == 0) continue;
            if (!o.empty()) o += "+";
            o += "i" + std::to_string(m);
            if (strides[m] != 1) o += "*" + lit(strides[m]);
        }
        return o.empty() ? lit(0) : o;
    }

    bool any_mode_in(int k, int lo, int hi) const
    {
        for (int m = lo; m != hi; ++m)
            if (st[k][m]) return true;
        return false;
    }
};

int pick_vec(einsum_t const& e, uint64_t inner_extent, bool force_scalar)
{
    if (force_scalar) return 1;
    int minsize = dtype_size(e.out_dtype());
    for (size_t k = 0; k != e.inns.size(); ++k) minsize = std::min(minsize, dtype_size(e.inn_dtype(k)));
    int v = 16 / minsize;
    while (v > 1 && inner_extent % v) v /= 2;
    return v;
}

// ---------------------------------------------------------------------------
// elementwise, vectorised along the innermost output mode
// ---------------------------------------------------------------------------
plan_t gen_ew_vec(ctx_t const& c, bool force_scalar)
{
    einsum_t const& e = c.e;
    int             L = c.r - 1;
    int             V = pick_vec(e, e.join_shape[L], force_scalar);
    uint64_t        N = e.out_nelem();
    uint64_t        NV = N / V;
    int             U = NV >= 148ull * 2048 * 4 ? 4 : (NV >= 148ull * 2048 ? 2 : 1);
    int const       B = 256;

    // does any input need the multi-index? (straight inputs use the flat index)
    std::vector<bool> straight(c.n);
    bool              need_idx = false;
    for (int k = 0; k != c.n; ++k) {
        straight[k] = c.st[k] == c.ost;
        need_idx = need_idx || !straight[k];
    }

    src_t s;
    s.raw(k_preamble);
    c.signature(s, "es_ew_vec_k0", B);
    s.add("  const %s NV = %s;", c.idx(), c.lit(NV).c_str());
    s.add("  const %s v0 = (%s)blockIdx.x * %du + threadIdx.x;", c.idx(), c.idx(), B * U);
    for (int k = 0; k != c.n; ++k) {
        bool vec = c.has_mode(k, L);
        if (vec) s.add("  raw_t<%d> q%d[%d];", V * dtype_size(e.inn_dtype(k)), k, U);
        else s.add("  %s b%d[%d];", compute_type(e.inn_dtype(k)), k, U);
    }
    s.add("  #pragma unroll");
    s.add("  for (int u = 0; u < %d; ++u) {", U);
    s.add("    const %s v = v0 + (%s)u * %du;", c.idx(), c.idx(), B);
    s.add("    if (v < NV) {");
    s.add("      const %s ee = v * %du;", c.idx(), V);
    if (need_idx) c.decompose(s, "ee", 0, c.r, "      ");
    for (int k = 0; k != c.n; ++k) {
        std::string off = straight[k] ? std::string("ee") : c.offset_expr(c.st[k], 0, c.r);
        if (c.has_mode(k, L))
            s.add("      ld_raw<%d>(x%d + (%s), q%d[u]);", V * dtype_size(e.inn_dtype(k)), k, off.c_str(), k);
        else
            s.add("      ld_%s<1>(x%d + (%s), &b%d[u]);", dt_suffix(e.inn_dtype(k)), k, off.c_str(),
                  k);
    }
    s.add("    }");
    s.add("  }");
    s.add("  #pragma unroll");
    s.add("  for (int u = 0; u < %d; ++u) {", U);
    s.add("    const %s v = v0 + (%s)u * %du;", c.idx(), c.idx(), B);
    s.add("    if (v < NV) {");
    for (int k = 0; k != c.n; ++k) {
        if (c.has_mode(k, L))
            s.add("      %s a%d[%d]; cv_%s<%d>(q%d[u], a%d);", compute_type(e.inn_dtype(k)), k, V,
                  dt_suffix(e.inn_dtype(k)), V, k, k);
    }
    s.add("      %s r[%d];", compute_type(e.out_dtype()), V);
    s.add("      #pragma unroll");
    s.add("      for (int i = 0; i < %d; ++i) {", V);
    std::vector<std::string> names;
    for (int k = 0; k != c.n; ++k) {
        names.push_back(c.has_mode(k, L) ? "a" + std::to_string(k) + "[i]"
                                         : "b" + std::to_string(k) + "[u]");
    }
    s.add("        r[i] = %s;", e.join.emit(names).c_str());
    s.add("      }");
    s.add("      st_%s<%d>(out + v * %du, r);", dt_suffix(e.out_dtype()), V, V);
    s.add("    }");
    s.add("  }");
    s.add("}");

    plan_t p;
    p.kind = "ew_vec";
    p.source = s.s;
    p.vec = V;
    p.align = V > 1 ? 16 : 1;
    launch_t l;
    l.entry = "es_ew_vec_k0";
    l.block = B;
    uint64_t grid = (NV + uint64_t(B) * U - 1) / (uint64_t(B) * U);
    if (grid > 0x7fffffffull) fail(ES_NOT_SUPPORTED, "elementwise grid too large");
    l.grid = (uint32_t)grid;
    p.launches.push_back(l);
    return p;
}

// ---------------------------------------------------------------------------
// elementwise, one thread per output element, arbitrary input strides
// ---------------------------------------------------------------------------
plan_t gen_ew_gather(ctx_t const& c)
{
    einsum_t const& e = c.e;
    uint64_t        N = e.out_nelem();
    int const       B = 256;
    src_t           s;
    s.raw(k_preamble);
    c.signature(s, "es_ew_gather_k0", B);
    s.add("  const %s ee = (%s)blockIdx.x * %du + threadIdx.x;", c.idx(), c.idx(), B);
    s.add("  if (ee >= %s) return;", c.lit(N).c_str());
    c.decompose(s, "ee", 0, c.r, "  ");
    std::vector<std::string> names;
    for (int k = 0; k != c.n; ++k) {
        s.add("  %s b%d; ld_%s<1>(x%d + (%s), &b%d);", compute_type(e.inn_dtype(k)), k,
              dt_suffix(e.inn_dtype(k)), k, c.offset_expr(c.st[k], 0, c.r).c_str(), k);
        names.push_back("b" + std::to_string(k));
    }
    s.add("  %s r = %s;", compute_type(e.out_dtype()), e.join.emit(names).c_str());
    s.add("  st_%s<1>(out + ee, &r);", dt_suffix(e.out_dtype()));
    s.add("}");
    plan_t p;
    p.kind = "ew_gather";
    p.source = s.s;
    launch_t l;
    l.entry = "es_ew_gather_k0";
    l.block = B;
    uint64_t grid = (N + B - 1) / B;
    if (grid > 0x7fffffffull) fail(ES_NOT_SUPPORTED, "elementwise grid too large");
    l.grid = (uint32_t)grid;
    p.launches.push_back(l);
    return p;
}

// ---------------------------------------------------------------------------
// elementwise where one or more inputs have a different innermost mode than
// the output: shared-memory tiles over the (output-innermost, input-innermost)
// plane so that both the reads and the writes are coalesced.
// ---------------------------------------------------------------------------
plan_t gen_ew_transpose(ctx_t const& c, int P)
{
    // L = innermost output mode; P = innermost mode of the permuted inputs.
    // Tile: 32 (P) x 32 (L).  Block 32x8.  Inputs whose innermost is P are
    // staged through smem; inputs aligned with L (or without L) are read directly.
    einsum_t const& e = c.e;
    int             L = c.r - 1;
    uint64_t        JL = e.join_shape[L], JP = e.join_shape[P];
    uint64_t        tl = (JL + 31) / 32, tp = (JP + 31) / 32;
    uint64_t        outer = e.out_nelem() / (JL * JP);
    src_t           s;
    s.raw(k_preamble);
    c.signature(s, "es_ew_transpose_k0", 256);
    for (int k = 0; k != c.n; ++k) {
        if (c.st[k][P] == 1)
            s.add("  __shared__ %s tile%d[32][33];", compute_type(e.inn_dtype(k)), k);
    }
    s.add("  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;");
    s.add("  %s bid = blockIdx.x;", c.idx());
    s.add("  const %s bl = bid %% %s; bid /= %s;", c.idx(), c.lit(tl).c_str(), c.lit(tl).c_str());
    s.add("  const %s bp = bid %% %s; bid /= %s;", c.idx(), c.lit(tp).c_str(), c.lit(tp).c_str());
    // remaining modes (all but L and P) from bid
    {
        std::vector<int> rest;
        for (int m = 0; m != c.r; ++m)
            if (m != L && m != P) rest.push_back(m);
        s.add("  %s t_r = bid;", c.idx());
        for (int j = (int)rest.size() - 1; j >= 0; --j) {
            int m = rest[j];
            if (j == 0) s.add("  const %s i%d = t_r;", c.idx(), m);
            else
                s.add("  const %s i%d = t_r %% %s; t_r /= %s;", c.idx(), m,
                      c.lit(e.join_shape[m]).c_str(), c.lit(e.join_shape[m]).c_str());
        }
        (void)outer;
    }
    // phase 1: read permuted inputs, coalesced along P
    s.add("  #pragma unroll");
    s.add("  for (int j = 0; j < 32; j += 8) {");
    s.add("    const %s i%d = bp * 32u + tx;", c.idx(), P);
    s.add("    const %s i%d = bl * 32u + ty + j;", c.idx(), L);
    s.add("    if (i%d < %s && i%d < %s) {", P, c.lit(JP).c_str(), L, c.lit(JL).c_str());
    for (int k = 0; k != c.n; ++k) {
        if (c.st[k][P] == 1)
            s.add("      ld_%s<1>(x%d + (%s), &tile%d[ty + j][tx]);", dt_suffix(e.inn_dtype(k)), k,
                  c.offset_expr(c.st[k], 0, c.r).c_str(), k);
    }
    s.add("    }");
    s.add("  }");
    s.add("  __syncthreads();");
    // phase 2: compute + write, coalesced along L
    s.add("  #pragma unroll");
    s.add("  for (int j = 0; j < 32; j += 8) {");
    s.add("    const %s i%d = bl * 32u + tx;", c.idx(), L);
    s.add("    const %s i%d = bp * 32u + ty + j;", c.idx(), P);
    s.add("    if (i%d < %s && i%d < %s) {", P, c.lit(JP).c_str(), L, c.lit(JL).c_str());
    std::vector<std::string> names;
    for (int k = 0; k != c.n; ++k) {
        if (c.st[k][P] == 1) {
            names.push_back("tile" + std::to_string(k) + "[tx][ty + j]");
        } else {
            s.add("      %s b%d; ld_%s<1>(x%d + (%s), &b%d);", compute_type(e.inn_dtype(k)), k,
                  dt_suffix(e.inn_dtype(k)), k, c.offset_expr(c.st[k], 0, c.r).c_str(), k);
            names.push_back("b" + std::to_string(k));
        }
    }
    s.add("      %s r = %s;", compute_type(e.out_dtype()), e.join.emit(names).c_str());
    s.add("      st_%s<1>(out + (%s), &r);", dt_suffix(e.out_dtype()),
          c.offset_expr(c.ost, 0, c.r).c_str());
    s.add("    }");
    s.add("  }");
    s.add("}");
    plan_t p;
    p.kind = "ew_transpose";
    p.source = s.s;
    launch_t l;
    l.entry = "es_ew_transpose_k0";
    l.block = 256;
    uint64_t grid = tl * tp * outer;
    if (grid > 0x7fffffffull) fail(ES_NOT_SUPPORTED, "transpose grid too large");
    l.grid = (uint32_t)grid;
    p.launches.push_back(l);
    return p;
}

// ---------------------------------------------------------------------------
// reductions
// ---------------------------------------------------------------------------
void emit_group_reduce(src_t& s, int G, int castable, int dtype)
{
    char const* ct = compute_type(dtype);
    s.add("  #pragma unroll");
    s.add("  for (int o = 16; o > 0; o >>= 1) { %s w = es_shx(r, o); r = %s; }", ct,
          combine_expr(castable, dtype, "r", "w").c_str());
    if (G > 32) {
        s.add("  __shared__ %s red[%d];", ct, G / 32);
        s.add("  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = r;");
        s.add("  __syncthreads();");
        s.add("  if (threadIdx.x < 32) {");
        s.add("    r = threadIdx.x < %d ? red[threadIdx.x] : %s;", G / 32,
              identity_literal(castable, dtype).c_str());
        s.add("    #pragma unroll");
        s.add("    for (int o = %d; o > 0; o >>= 1) { %s w = es_shx(r, o); r = %s; }", G / 64, ct,
              combine_expr(castable, dtype, "r", "w").c_str());
        s.add("  }");
    }
}

// Row reduction: the last aggregated mode L is the innermost mode of every
// input that has it.  One warp (short rows) or one CTA (long rows) per output
// element; rows that are too few to fill the GPU are split across CTAs with the
// partials combined by a second kernel through the workspace.
plan_t gen_red_row(ctx_t const& c, bool force_scalar)
{
    einsum_t const& e = c.e;
    int             L = c.r - 1;
    int             orank = e.out_rank;
    int             od = e.out_dtype();
    char const*     ct = compute_type(od);
    int             V = pick_vec(e, e.join_shape[L], force_scalar);
    uint64_t        NO = e.out_nelem();
    uint64_t        A = e.join_nelem() / NO;
    uint64_t        AV = A / V;
    int             G = AV <= 256 ? 32 : 256;
    uint64_t        S = 1; // CTAs per row
    if (G == 256 && NO < 148ull * 4 && AV >= 256ull * 16) {
        S = std::min<uint64_t>((148ull * 8 + NO - 1) / NO, AV / (256ull * 4));
        S = std::max<uint64_t>(S, 1);
    }
    uint64_t CH = (AV + S - 1) / S; // vectors per chunk
    S = (AV + CH - 1) / CH;
    int rows_per_cta = 256 / G;

    src_t s;
    s.raw(k_preamble);
    c.signature(s, "es_red_row_k0", 256);
    if (G == 32) {
        s.add("  const int lane = threadIdx.x & 31;");
        // CTAs take the rows from the last to the first: a reduction usually reads what the kernel
        // before it just wrote front to back, and the tail of that tensor is what the 126 MB L2 still
        // holds; the CTAs that start first find it there instead of evicting it with the head
        s.add("  const %s row = (%s)(gridDim.x - 1u - blockIdx.x) * %du + (threadIdx.x >> 5);", c.idx(), c.idx(),
              rows_per_cta);
        s.add("  if (row >= %s) return;", c.lit(NO).c_str());
        s.add("  const %s p_begin = 0, p_end = %s;", c.idx(), c.lit(AV).c_str());
    } else {
        s.add("  const int lane = threadIdx.x;");
        if (S == 1) {
            s.add("  const %s row = gridDim.x - 1u - blockIdx.x;  // last rows first, see above", c.idx());
            s.add("  const %s p_begin = 0, p_end = %s;", c.idx(), c.lit(AV).c_str());
        } else {
            s.add("  const %s row = blockIdx.x / %s;", c.idx(), c.lit(S).c_str());
            s.add("  const %s chunk = blockIdx.x %% %s;", c.idx(), c.lit(S).c_str());
            s.add("  const %s p_begin = chunk * %s;", c.idx(), c.lit(CH).c_str());
            s.add("  const %s p_end = min(p_begin + %s, %s);", c.idx(), c.lit(CH).c_str(),
                  c.lit(AV).c_str());
        }
    }
    c.decompose(s, "row", 0, orank, "  ");
    std::vector<std::string> names(c.n);
    for (int k = 0; k != c.n; ++k) {
        s.add("  const %s base%d = %s;", c.idx(), k, c.offset_expr(c.st[k], 0, orank).c_str());
        if (!c.any_mode_in(k, orank, c.r)) {
            // row-invariant input: read once
            s.add("  %s c%d; ld_%s<1>(x%d + base%d, &c%d);", compute_type(e.inn_dtype(k)), k,
                  dt_suffix(e.inn_dtype(k)), k, k, k);
            names[k] = "c" + std::to_string(k);
        } else if (c.has_mode(k, L)) {
            names[k] = "a" + std::to_string(k) + "[i]";
        } else {
            names[k] = "s" + std::to_string(k);
        }
    }
    s.add("  %s acc[%d];", ct, V);
    s.add("  #pragma unroll");
    s.add("  for (int i = 0; i < %d; ++i) acc[i] = %s;", V,
          identity_literal(e.castable, od).c_str());
    // Loads are issued in batches of NB before any of them is consumed, so that
    // each thread keeps NB 16-byte requests in flight.  Short rows (few trips per
    // thread, known here) are unrolled completely.
    uint64_t const max_trips = ((S == 1 ? AV : CH) + G - 1) / G;
    int const      NB = (int)std::min<uint64_t>(max_trips, 4);
    bool const     whole = S == 1 && max_trips <= 8; // every trip of a thread in one batch
    int const      batch = whole ? (int)max_trips : NB;
    for (int k = 0; k != c.n; ++k) {
        if (c.any_mode_in(k, orank, c.r) && c.has_mode(k, L))
            s.add("  raw_t<%d> q%d[%d];", V * dtype_size(e.inn_dtype(k)), k, batch);
    }
    if (whole) s.add("  {");
    else s.add("  for (%s p0 = p_begin + lane; p0 < p_end; p0 += %du) {", c.idx(), G * batch);
    if (whole) s.add("    const %s p0 = p_begin + lane;", c.idx());
    // load phase
    s.add("    #pragma unroll");
    s.add("    for (int t = 0; t < %d; ++t) {", batch);
    s.add("      const %s p = p0 + (%s)t * %du;", c.idx(), c.idx(), G);
    s.add("      if (p < p_end) {");
    s.add("        const %s ea = p * %du;", c.idx(), V);
    c.decompose(s, "ea", orank, c.r, "        ");
    for (int k = 0; k != c.n; ++k) {
        if (!c.any_mode_in(k, orank, c.r) || !c.has_mode(k, L)) continue;
        s.add("        ld_raw<%d>(x%d + base%d + (%s), q%d[t]);", V * dtype_size(e.inn_dtype(k)), k, k,
              c.offset_expr(c.st[k], orank, c.r).c_str(), k);
    }
    s.add("      }");
    s.add("    }");
    // compute phase
    s.add("    #pragma unroll");
    s.add("    for (int t = 0; t < %d; ++t) {", batch);
    s.add("      const %s p = p0 + (%s)t * %du;", c.idx(), c.idx(), G);
    s.add("      if (p < p_end) {");
    bool need_scalar = false;
    for (int k = 0; k != c.n; ++k)
        if (c.any_mode_in(k, orank, c.r) && !c.has_mode(k, L)) need_scalar = true;
    if (need_scalar) {
        s.add("        const %s ea = p * %du;", c.idx(), V);
        c.decompose(s, "ea", orank, c.r, "        ");
    }
    for (int k = 0; k != c.n; ++k) {
        if (!c.any_mode_in(k, orank, c.r)) continue;
        if (c.has_mode(k, L)) {
            s.add("        %s a%d[%d]; cv_%s<%d>(q%d[t], a%d);", compute_type(e.inn_dtype(k)), k, V,
                  dt_suffix(e.inn_dtype(k)), V, k, k);
        } else {
            s.add("        %s s%d; ld_%s<1>(x%d + base%d + (%s), &s%d);", compute_type(e.inn_dtype(k)),
                  k, dt_suffix(e.inn_dtype(k)), k, k, c.offset_expr(c.st[k], orank, c.r).c_str(), k);
        }
    }
    s.add("        #pragma unroll");
    s.add("        for (int i = 0; i < %d; ++i) {", V);
    s.add("          const %s val = %s;", ct, e.join.emit(names).c_str());
    s.add("          acc[i] = %s;", combine_expr(e.castable, od, "acc[i]", "val").c_str());
    s.add("        }");
    s.add("      }");
    s.add("    }");
    s.add("  }");
    s.add("  %s r = acc[0];", ct);
    s.add("  #pragma unroll");
    s.add("  for (int i = 1; i < %d; ++i) r = %s;", V,
          combine_expr(e.castable, od, "r", "acc[i]").c_str());
    emit_group_reduce(s, G, e.castable, od);
    if (S == 1) {
        s.add("  if (lane == 0) st_%s<1>(out + row, &r);", dt_suffix(od));
    } else {
        s.add("  if (lane == 0) ((%s*)ws_)[row * %s + chunk] = r;", ct, c.lit(S).c_str());
    }
    s.add("}");

    plan_t p;
    p.kind = S == 1 ? "red_row" : "red_split";
    p.vec = V;
    p.align = V > 1 ? 16 : 1;
    launch_t l;
    l.entry = "es_red_row_k0";
    l.block = 256;
    uint64_t grid = G == 32 ? (NO + rows_per_cta - 1) / rows_per_cta : NO * S;
    if (grid > 0x7fffffffull) fail(ES_NOT_SUPPORTED, "reduction grid too large");
    l.grid = (uint32_t)grid;
    p.launches.push_back(l);

    if (S > 1) {
        // second pass: one thread per output combines the S partials
        c.signature(s, "es_red_row_k1", 256);
        s.add("  const %s row = (%s)blockIdx.x * 256u + threadIdx.x;", c.idx(), c.idx());
        s.add("  if (row >= %s) return;", c.lit(NO).c_str());
        s.add("  const %s* part = (const %s*)ws_ + row * %s;", ct, ct, c.lit(S).c_str());
        s.add("  %s r = part[0];", ct);
        s.add("  for (int j = 1; j < %d; ++j) { %s w = part[j]; r = %s; }", (int)S, ct,
              combine_expr(e.castable, od, "r", "w").c_str());
        s.add("  st_%s<1>(out + row, &r);", dt_suffix(od));
        s.add("}");
        launch_t l2;
        l2.entry = "es_red_row_k1";
        l2.block = 256;
        l2.grid = (uint32_t)((NO + 255) / 256);
        p.launches.push_back(l2);
        p.workspace_bytes = NO * S * (od == ES_F64 || od == ES_C64 ? 8 : 4);
    }
    p.source = s.s;
    return p;
}

// Column reduction: the innermost mode of the inputs that carry the innermost
// output mode Lo is Lo itself (e.g. "ba->a").  Threads map to consecutive
// output elements (coalesced reads along Lo), each block covers 32 output
// columns x 8 slices of the aggregated space, combined through shared memory;
// when the outputs are too few to fill the GPU the aggregated space is also
// split across blocks (workspace + second pass).
plan_t gen_red_col(ctx_t const& c)
{
    einsum_t const& e = c.e;
    int             orank = e.out_rank;
    int             od = e.out_dtype();
    char const*     ct = compute_type(od);
    uint64_t        NO = e.out_nelem();
    uint64_t        A = e.join_nelem() / NO;
    uint64_t        col_blocks = (NO + 31) / 32;
    uint64_t        S = 1;
    if (col_blocks < 148ull * 4 && A >= 8 * 16) {
        S = std::min<uint64_t>((148ull * 8 + col_blocks - 1) / col_blocks, A / (8 * 4));
        S = std::max<uint64_t>(S, 1);
    }
    uint64_t CH = (A + S - 1) / S;
    S = (A + CH - 1) / CH;

    src_t s;
    s.raw(k_preamble);
    c.signature(s, "es_red_col_k0", 256);
    s.add("  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;");
    s.add("  const %s cb = blockIdx.x %% %s;", c.idx(), c.lit(col_blocks).c_str());
    s.add("  const %s chunk = blockIdx.x / %s;", c.idx(), c.lit(col_blocks).c_str());
    s.add("  const %s row = cb * 32u + tx;", c.idx());
    s.add("  const bool live = row < %s;", c.lit(NO).c_str());
    s.add("  %s r = %s;", ct, identity_literal(e.castable, od).c_str());
    s.add("  if (live) {");
    c.decompose(s, "row", 0, orank, "    ");
    std::vector<std::string> names(c.n);
    for (int k = 0; k != c.n; ++k) {
        s.add("    const %s base%d = %s;", c.idx(), k, c.offset_expr(c.st[k], 0, orank).c_str());
        if (!c.any_mode_in(k, orank, c.r)) {
            s.add("    %s c%d; ld_%s<1>(x%d + base%d, &c%d);", compute_type(e.inn_dtype(k)), k,
                  dt_suffix(e.inn_dtype(k)), k, k, k);
            names[k] = "c" + std::to_string(k);
        } else {
            names[k] = "s" + std::to_string(k);
        }
    }
    s.add("    const %s q_begin = chunk * %s;", c.idx(), c.lit(CH).c_str());
    s.add("    const %s q_end = min(q_begin + %s, %s);", c.idx(), c.lit(CH).c_str(),
          c.lit(A).c_str());
    s.add("    #pragma unroll 4");
    s.add("    for (%s q = q_begin + ty; q < q_end; q += 8u) {", c.idx());
    c.decompose(s, "q", orank, c.r, "      ");
    for (int k = 0; k != c.n; ++k) {
        if (!c.any_mode_in(k, orank, c.r)) continue;
        s.add("      %s s%d; ld_%s<1>(x%d + base%d + (%s), &s%d);", compute_type(e.inn_dtype(k)), k,
              dt_suffix(e.inn_dtype(k)), k, k, c.offset_expr(c.st[k], orank, c.r).c_str(), k);
    }
    s.add("      const %s val = %s;", ct, e.join.emit(names).c_str());
    s.add("      r = %s;", combine_expr(e.castable, od, "r", "val").c_str());
    s.add("    }");
    s.add("  }");
    s.add("  __shared__ %s red[8][33];", ct);
    s.add("  red[ty][tx] = r;");
    s.add("  __syncthreads();");
    s.add("  if (ty == 0 && live) {");
    s.add("    #pragma unroll");
    s.add("    for (int j = 1; j < 8; ++j) { %s w = red[j][tx]; r = %s; }", ct,
          combine_expr(e.castable, od, "r", "w").c_str());
    if (S == 1) s.add("    st_%s<1>(out + row, &r);", dt_suffix(od));
    else s.add("    ((%s*)ws_)[row * %s + chunk] = r;", ct, c.lit(S).c_str());
    s.add("  }");
    s.add("}");

    plan_t p;
    p.kind = S == 1 ? "red_col" : "red_col_split";
    launch_t l;
    l.entry = "es_red_col_k0";
    l.block = 256;
    uint64_t grid = col_blocks * S;
    if (grid > 0x7fffffffull) fail(ES_NOT_SUPPORTED, "reduction grid too large");
    l.grid = (uint32_t)grid;
    p.launches.push_back(l);
    if (S > 1) {
        c.signature(s, "es_red_col_k1", 256);
        s.add("  const %s row = (%s)blockIdx.x * 256u + threadIdx.x;", c.idx(), c.idx());
        s.add("  if (row >= %s) return;", c.lit(NO).c_str());
        s.add("  const %s* part = (const %s*)ws_ + row * %s;", ct, ct, c.lit(S).c_str());
        s.add("  %s r = part[0];", ct);
        s.add("  for (int j = 1; j < %d; ++j) { %s w = part[j]; r = %s; }", (int)S, ct,
              combine_expr(e.castable, od, "r", "w").c_str());
        s.add("  st_%s<1>(out + row, &r);", dt_suffix(od));
        s.add("}");
        launch_t l2;
        l2.entry = "es_red_col_k1";
        l2.block = 256;
        l2.grid = (uint32_t)((NO + 255) / 256);
        p.launches.push_back(l2);
        p.workspace_bytes = NO * S * (od == ES_F64 || od == ES_C64 ? 8 : 4);
    }
    p.source = s.s;
    return p;
}

} // namespace

plan_t plan_pointwise(einsum_t const& e, bool force_scalar)
{
    ctx_t c(e);
    int   L = c.r - 1;
    if (!e.has_aggregation()) {
        // every input either has the innermost output mode as its own innermost
        // mode or does not have it at all -> vector path
        bool aligned = true;
        int  permuted_inner = -1;
        bool one_inner = true;
        for (int k = 0; k != c.n; ++k) {
            if (c.st[k][L] > 1) {
                aligned = false;
                int inner = e.inns[k].back();
                if (permuted_inner >= 0 && permuted_inner != inner) one_inner = false;
                permuted_inner = inner;
            }
        }
        if (aligned) return gen_ew_vec(c, force_scalar);
        if (one_inner && permuted_inner >= 0) return gen_ew_transpose(c, permuted_inner);
        return gen_ew_gather(c);
    }
    // reductions: row form when L (last aggregated mode) is innermost wherever present
    bool row = true;
    for (int k = 0; k != c.n; ++k) {
        if (c.st[k][L] > 1) row = false;
    }
    if (row) return gen_red_row(c, force_scalar);
    return gen_red_col(c);
}

} // namespace es
