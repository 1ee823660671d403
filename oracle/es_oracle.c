/*
 * TEST INFRASTRUCTURE -- not product code.
 *
 * Plain-C restatement of the reference CPU engine's kernels for the memgraph
 * apply-node path, used (1) as the timed CPU baseline of bench.py and (2) as a
 * second checker beside oracle/es_oracle.py.  Only tests/, the smoke check and
 * bench.py's CPU-baseline leg may load this library.
 *
 * Parity status: PINNED -- tests/test_oracle_c.py checks every function against
 * fixtures produced by the reference's own interpreter (tests/golden).
 *
 * The reference CPU engine runs one kernel per pooled thread and gets its
 * parallelism from the taskgraph's blocks (src/server/cpu/mg_server.cc:13-63,
 * src/engine/cpu/mg/exec_graph.cc:193-220); the `omp parallel for` over row
 * blocks below stands for a placement that splits the outermost dim into one
 * block per thread.  Each function cites the loop it follows.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <omp.h>

typedef _Float16 f16;

int oracle_num_threads(void) { return omp_get_max_threads(); }

/* ---- elementwise: _unary_ew_loop / _binary_ew_loop
 *      (src/engine/cpu/kernel_executor.cc:786-845): out[i] = op(x0[i0], x1[i1]),
 *      "ab,a" reads x1[i], "ab,b" reads x1[j].  Arithmetic in the tensor dtype,
 *      as float16_t arithmetic does (every operation rounds to f16). ---- */

/* join = x0 * (1 + exp(-1 * x0))^-1 * x1   (scalarop_t::make_silu combined with mul) */
void oracle_silu_mul_f16(uint64_t n, f16* out, const f16* x0, const f16* x1)
{
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < n; ++i) {
        f16 a = x0[i];
        f16 neg = (f16)((f16)-1.0f * a);
        f16 ex = (f16)expf((float)neg);
        f16 den = (f16)((f16)1.0f + ex);
        f16 rcp = (f16)(1.0f / (float)den);
        f16 silu = (f16)(a * rcp);
        out[i] = (f16)(silu * x1[i]);
    }
}

void oracle_silu_mul_f32(uint64_t n, float* out, const float* x0, const float* x1)
{
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < n; ++i) {
        float a = x0[i];
        out[i] = (a * (1.0f / (1.0f + expf(-1.0f * a)))) * x1[i];
    }
}

/* "ab,a->ab", join = exp(x0 + -1*x1) */
void oracle_exp_sub_ab_a_f16(uint64_t n1, uint64_t n2, f16* out, const f16* x0, const f16* x1)
{
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < n1; ++i) {
        f16 m = x1[i];
        for (uint64_t j = 0; j < n2; ++j) {
            f16 d = (f16)(x0[i * n2 + j] + (f16)((f16)-1.0f * m));
            out[i * n2 + j] = (f16)expf((float)d);
        }
    }
}

void oracle_exp_sub_ab_a_f32(uint64_t n1, uint64_t n2, float* out, const float* x0, const float* x1)
{
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < n1; ++i) {
        float m = x1[i];
        for (uint64_t j = 0; j < n2; ++j) out[i * n2 + j] = expf(x0[i * n2 + j] + -1.0f * m);
    }
}

/* ---- reductions "ab->a": _real_reduction_ab_a (f64 running total for add/mul)
 *      and _reduction_ab_a (native compare for min/max)
 *      (src/engine/cpu/kernel_executor.cc:1163-1195).  castable: 0 add 1 mul 2 min 3 max ---- */
#define ORACLE_REDUCE(NAME, T)                                                                     \
    void NAME(int castable, uint64_t n1, uint64_t n2, T* out, const T* inn)                        \
    {                                                                                              \
        _Pragma("omp parallel for schedule(static)") for (uint64_t i = 0; i < n1; ++i)             \
        {                                                                                          \
            const T* row = inn + i * n2;                                                           \
            if (castable == 0 || castable == 1) {                                                  \
                double total = (double)row[0];                                                     \
                for (uint64_t j = 1; j < n2; ++j) {                                                \
                    if (castable == 0) total += (double)row[j];                                    \
                    else total *= (double)row[j];                                                  \
                }                                                                                  \
                out[i] = (T)total;                                                                 \
            } else {                                                                               \
                T acc = row[0];                                                                    \
                for (uint64_t j = 1; j < n2; ++j) {                                                \
                    T v = row[j];                                                                  \
                    if (castable == 2) acc = (v < acc) ? v : acc;                                  \
                    else acc = (acc < v) ? v : acc;                                                \
                }                                                                                  \
                out[i] = acc;                                                                      \
            }                                                                                      \
        }                                                                                          \
    }
ORACLE_REDUCE(oracle_reduce_ab_a_f16, f16)
ORACLE_REDUCE(oracle_reduce_ab_a_f32, float)
ORACLE_REDUCE(oracle_reduce_ab_a_f64, double)

/* "ab,a->a" add of exp(x0 - x1): reduce_exp_sub (src/engine/cpu/kernel_executor.cc:1868-1885) */
void oracle_reduce_exp_sub_f32(uint64_t na, uint64_t nb, float* out, const float* lhs, const float* rhs)
{
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < na; ++i) {
        const float* l = lhs + i * nb;
        float        r = rhs[i];
        float        acc = expf(l[0] - r);
        for (uint64_t j = 1; j < nb; ++j) acc += expf(l[j] - r);
        out[i] = acc;
    }
}

/* ---- touch: execute_touch (src/engine/touch.cc:3-237).  dims = rank x
 *      {d_inn, d_out, offset_inn, offset_out, size}, rank <= 4 after simplify.
 *      dtype: 0 f16 1 f32 2 f64 3 c64; castable -1 none 0 add 1 mul 2 min 3 max.
 *      Copy is a memcpy per innermost row; accumulation in the tensor dtype. ---- */
static void touch_row(int castable, int dtype, void* out, const void* inn, uint64_t n)
{
    if (castable < 0) {
        static const int sz[4] = {2, 4, 8, 8};
        memcpy(out, inn, n * sz[dtype]);
        return;
    }
#define ROW(T)                                                                                     \
    {                                                                                              \
        T*       o = (T*)out;                                                                      \
        const T* x = (const T*)inn;                                                                \
        for (uint64_t i = 0; i < n; ++i) {                                                         \
            if (castable == 0) o[i] = (T)(o[i] + x[i]);                                            \
            else if (castable == 1) o[i] = (T)(o[i] * x[i]);                                       \
            else if (castable == 2) o[i] = (x[i] < o[i]) ? x[i] : o[i];                            \
            else o[i] = (o[i] < x[i]) ? x[i] : o[i];                                               \
        }                                                                                          \
    }
    if (dtype == 0) ROW(f16)
    else if (dtype == 1) ROW(float)
    else if (dtype == 2) ROW(double)
    else {
        float*       o = (float*)out;
        const float* x = (const float*)inn;
        for (uint64_t i = 0; i < n; ++i) {
            float ar = o[2 * i], ai = o[2 * i + 1], br = x[2 * i], bi = x[2 * i + 1];
            if (castable == 0) {
                o[2 * i] = ar + br;
                o[2 * i + 1] = ai + bi;
            } else {
                o[2 * i] = ar * br - ai * bi;
                o[2 * i + 1] = ar * bi + ai * br;
            }
        }
    }
#undef ROW
}

int oracle_touch(int rank, const uint64_t* dims, int castable, int dtype, void* out, const void* inn)
{
    if (rank < 1 || rank > 4) return -1;
    static const int sz[4] = {2, 4, 8, 8};
    uint64_t d_inn[4] = {1, 1, 1, 1}, d_out[4] = {1, 1, 1, 1}, oi[4] = {0, 0, 0, 0}, oo[4] = {0, 0, 0, 0},
             n[4] = {1, 1, 1, 1};
    for (int i = 0; i < rank; ++i) {
        int s = 4 - rank + i;
        d_inn[s] = dims[5 * i + 0];
        d_out[s] = dims[5 * i + 1];
        oi[s] = dims[5 * i + 2];
        oo[s] = dims[5 * i + 3];
        n[s] = dims[5 * i + 4];
    }
    uint64_t rows = n[0] * n[1] * n[2];
#pragma omp parallel for schedule(static) if (rows > 1)
    for (uint64_t r = 0; r < rows; ++r) {
        uint64_t i2 = r % n[2], t = r / n[2], i1 = t % n[1], i0 = t / n[1];
        uint64_t pin = (((i0 + oi[0]) * d_inn[1] + (i1 + oi[1])) * d_inn[2] + (i2 + oi[2])) * d_inn[3] + oi[3];
        uint64_t pout = (((i0 + oo[0]) * d_out[1] + (i1 + oo[1])) * d_out[2] + (i2 + oo[2])) * d_out[3] + oo[3];
        touch_row(castable, dtype, (char*)out + pout * sz[dtype], (const char*)inn + pin * sz[dtype], n[3]);
    }
    return 0;
}

/* ---- matmul "ij,jk->ik" f32, beta = 0: matrix_multiply_update's cblas_sgemm
 *      call (src/engine/cpu/kernel_executor.cc:1293-1548) restated as a
 *      cache-blocked triple loop (MKL itself is not available here). ---- */
void oracle_matmul_f32(uint64_t ni, uint64_t nj, uint64_t nk, float* out, const float* lhs, const float* rhs)
{
    const uint64_t BI = 64, BJ = 256;
#pragma omp parallel for schedule(static)
    for (uint64_t i0 = 0; i0 < ni; i0 += BI) {
        uint64_t i1 = i0 + BI < ni ? i0 + BI : ni;
        for (uint64_t i = i0; i < i1; ++i) memset(out + i * nk, 0, nk * sizeof(float));
        for (uint64_t j0 = 0; j0 < nj; j0 += BJ) {
            uint64_t j1 = j0 + BJ < nj ? j0 + BJ : nj;
            for (uint64_t i = i0; i < i1; ++i) {
                for (uint64_t j = j0; j < j1; ++j) {
                    float        a = lhs[i * nj + j];
                    const float* b = rhs + j * nk;
                    float*       o = out + i * nk;
                    for (uint64_t k = 0; k < nk; ++k) o[k] += a * b[k];
                }
            }
        }
    }
}

/* ---- fills: _lowertri_fill / constant_fill
 *      (src/engine/cpu/kernel_executor.cc:1776-1832) on raw element words ---- */
void oracle_fill_lowertri(int elem_bytes, const void* lower, const void* upper, int64_t nrow, int64_t ncol,
                          int64_t start, void* out)
{
    for (int64_t i = 0; i < nrow; ++i)
        for (int64_t j = 0; j < ncol; ++j)
            memcpy((char*)out + (i * ncol + j) * elem_bytes, (i - start >= j) ? lower : upper, elem_bytes);
}
