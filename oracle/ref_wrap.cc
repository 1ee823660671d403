// Test infrastructure, not product code.
//
// A plain-C surface over the reference's own CPU interpreter, compiled against
// the reference's sources where they lie (never copied).  Used only by the test
// suite, the smoke check and the bench's CPU-baseline leg to (1) validate the
// numpy/C restatement in this directory and (2) generate golden fixtures.
//
// Entry points and the reference function each one forwards to:
//   ref_einsummable      -> reference_einsummable_inplace   (src/einsummable/reference.cc:410-483)
//   ref_touch            -> reference_touch                 (src/einsummable/reference.cc:565-607)
//   ref_execute_touch    -> execute_touch                   (src/engine/touch.cc:155-237)
//   ref_touch_simplify   -> touch_t::simplify               (src/einsummable/touch.cc:3-28)
//   ref_fill_constant /
//   ref_fill_lowertri    -> reference_fill                  (src/einsummable/reference.cc:485-508)
//   ref_merge            -> einsummable_t::merge_adjacent_dims (src/einsummable/einsummable.cc:166-218)
//   ref_scalarop_make    -> scalarop_t::make_* builders     (src/einsummable/scalarop.cc:2204-2527)
//   ref_scalarop_info    -> operator<<, to_cppstr, simplify (src/einsummable/scalarop.cc)
//   ref_scalarop_eval    -> scalarop_t::eval                (src/einsummable/scalarop.cc:604-640)
#include "src/einsummable/reference.h"
#include "src/einsummable/einsummable.h"
#include "src/einsummable/touch.h"
#include "src/einsummable/fill.h"
#include "src/engine/touch.h"

#include <cstring>

static thread_local std::string g_err;
static thread_local std::string g_str;

#define GUARD_BEGIN try {
#define GUARD_END                                                                                  \
    }                                                                                              \
    catch (std::exception const& e)                                                                \
    {                                                                                              \
        g_err = e.what();                                                                          \
        return -1;                                                                                 \
    }                                                                                              \
    catch (...)                                                                                    \
    {                                                                                              \
        g_err = "unknown exception";                                                               \
        return -1;                                                                                 \
    }

static dtype_t dtype_of(int code)
{
    switch (code) {
        case 0: return dtype_t::f16;
        case 1: return dtype_t::f32;
        case 2: return dtype_t::f64;
        case 3: return dtype_t::c64;
    }
    throw std::runtime_error("bad dtype code");
}

static optional<castable_t> castable_of(int code)
{
    switch (code) {
        case -1: return std::nullopt;
        case 0: return castable_t::add;
        case 1: return castable_t::mul;
        case 2: return castable_t::min;
        case 3: return castable_t::max;
    }
    throw std::runtime_error("bad castable code");
}

static einsummable_t make_es(int             join_rank,
                             uint64_t const* join_shape,
                             int             n_inn,
                             int const*      inn_ranks,
                             int const*      inn_modes,
                             int             out_rank,
                             char const*     join_text,
                             int             castable)
{
    vector<uint64_t>    js(join_shape, join_shape + join_rank);
    vector<vector<int>> inns;
    int const*          p = inn_modes;
    for (int i = 0; i != n_inn; ++i) {
        inns.emplace_back(p, p + inn_ranks[i]);
        p += inn_ranks[i];
    }
    scalarop_t join = parse_with_ss<scalarop_t>(string(join_text));
    return einsummable_t(js, inns, out_rank, join, castable_of(castable));
}

static touch_t make_touch(int rank, uint64_t const* d5, int castable, int dtype)
{
    vector<touchdim_t> sel;
    for (int i = 0; i != rank; ++i) {
        sel.push_back(touchdim_t{.d_inn = d5[5 * i + 0],
                                 .d_out = d5[5 * i + 1],
                                 .offset_inn = d5[5 * i + 2],
                                 .offset_out = d5[5 * i + 3],
                                 .size = d5[5 * i + 4]});
    }
    return touch_t{.selection = sel, .castable = castable_of(castable), .dtype = dtype_of(dtype)};
}

extern "C" {

char const* ref_last_error()
{
    return g_err.c_str();
}

int ref_einsummable(int                join_rank,
                    uint64_t const*    join_shape,
                    int                n_inn,
                    int const*         inn_ranks,
                    int const*         inn_modes,
                    int                out_rank,
                    char const*        join_text,
                    int                castable,
                    void*              out,
                    void const* const* inns)
{
    GUARD_BEGIN
    einsummable_t e =
        make_es(join_rank, join_shape, n_inn, inn_ranks, inn_modes, out_rank, join_text, castable);
    vector<dbuffer_t> ins;
    for (int i = 0; i != n_inn; ++i) {
        ins.emplace_back(e.inn_dtype(i),
                         make_buffer_reference(const_cast<void*>(inns[i]), e.inn_size(i)));
    }
    dbuffer_t o(e.out_dtype(), make_buffer_reference(out, e.out_size()));
    reference_einsummable_inplace(e, o, ins);
    return 0;
    GUARD_END
}

// Writes "str|join_shape...|out_rank|inn0 modes;inn1 modes" of the merged einsummable.
int ref_merge(int             join_rank,
              uint64_t const* join_shape,
              int             n_inn,
              int const*      inn_ranks,
              int const*      inn_modes,
              int             out_rank,
              char const*     join_text,
              int             castable,
              char*           buf,
              int             buf_len)
{
    GUARD_BEGIN
    einsummable_t e =
        make_es(join_rank, join_shape, n_inn, inn_ranks, inn_modes, out_rank, join_text, castable);
    einsummable_t      m = e.merge_adjacent_dims();
    std::stringstream  ss;
    ss << m.str() << "|";
    for (int i = 0; i != m.join_shape.size(); ++i) {
        ss << (i ? "," : "") << m.join_shape[i];
    }
    ss << "|" << m.out_rank << "|";
    for (int i = 0; i != m.inns.size(); ++i) {
        ss << (i ? ";" : "");
        for (int j = 0; j != m.inns[i].size(); ++j) {
            ss << (j ? "," : "") << m.inns[i][j];
        }
    }
    ss << "|" << e.str() << "|" << int(e.is_contraction()) << int(e.has_aggregation())
       << int(e.is_permutation()) << int(e.is_straight_elementwise()) << int(e.has_broadcast());
    string s = ss.str();
    if ((int)s.size() + 1 > buf_len) {
        throw std::runtime_error("buffer too small");
    }
    std::memcpy(buf, s.c_str(), s.size() + 1);
    return 0;
    GUARD_END
}

int ref_touch(int rank, uint64_t const* d5, int castable, int dtype, void* out, void const* inn)
{
    GUARD_BEGIN
    touch_t  t = make_touch(rank, d5, castable, dtype);
    uint64_t n_out = 1, n_inn = 1;
    for (auto const& td : t.selection) {
        n_out *= td.d_out;
        n_inn *= td.d_inn;
    }
    uint64_t  ds = dtype_size(t.dtype);
    dbuffer_t o(t.dtype, make_buffer_reference(out, n_out * ds));
    dbuffer_t i(t.dtype, make_buffer_reference(const_cast<void*>(inn), n_inn * ds));
    reference_touch(t, o, i);
    return 0;
    GUARD_END
}

int ref_execute_touch(
    int rank, uint64_t const* d5, int castable, int dtype, void* out, void const* inn)
{
    GUARD_BEGIN
    touch_t t = make_touch(rank, d5, castable, dtype).simplify();
    execute_touch(t, out, inn);
    return 0;
    GUARD_END
}

// Returns the simplified rank; out_d5 must hold 5*rank values.
int ref_touch_simplify(int rank, uint64_t const* d5, uint64_t* out_d5)
{
    GUARD_BEGIN
    touch_t t = make_touch(rank, d5, -1, 1).simplify();
    int     r = t.selection.size();
    for (int i = 0; i != r; ++i) {
        auto const& td = t.selection[i];
        out_d5[5 * i + 0] = td.d_inn;
        out_d5[5 * i + 1] = td.d_out;
        out_d5[5 * i + 2] = td.offset_inn;
        out_d5[5 * i + 3] = td.offset_out;
        out_d5[5 * i + 4] = td.size;
    }
    return r;
    GUARD_END
}

int ref_fill_constant(int dtype, char const* value, uint64_t nelem, void* out)
{
    GUARD_BEGIN
    dtype_t   d = dtype_of(dtype);
    fill_t    f = fill_t::make_constant(scalar_t(d, value), {nelem});
    dbuffer_t r = reference_fill(f);
    std::memcpy(out, r.raw(), r.size());
    return 0;
    GUARD_END
}

int ref_fill_lowertri(int         dtype,
                      char const* lower,
                      char const* upper,
                      uint64_t    nrow,
                      uint64_t    ncol,
                      int64_t     start,
                      void*       out)
{
    GUARD_BEGIN
    dtype_t d = dtype_of(dtype);
    // reference_fill on the raw lowertri_t (fill_t's constructor may fold a
    // degenerate triangle into a constant; the values are the same either way)
    fill_t f(fill_t::lowertri_t{.lower = parse_with_ss<scalar_t>(write_with_ss(d) + "|" + lower),
                                .upper = parse_with_ss<scalar_t>(write_with_ss(d) + "|" + upper),
                                .nrow = nrow,
                                .ncol = ncol,
                                .start = start});
    dbuffer_t r = reference_fill(f);
    std::memcpy(out, r.raw(), r.size());
    return 0;
    GUARD_END
}

// Builds one of the reference's named scalarops and returns its text form.
// name: identity add mul div neg min max is_min is_max is_equal sub exp sigmoid log sqrt
//       inverse inverse_sqrt square relu silu rcp relu_deriv conjugate project_real
//       project_imag complex; "scale:<v>", "increment:<v>", "power:<n>", "convert:<dst>"
//       (dtype = src), "silu_mul" (C2's fused op), "exp_sub", "softmax_v3_sum:<c>",
//       "softmax_v3_norm:<c>".
int ref_scalarop_make(char const* name_, int dtype, char* buf, int buf_len)
{
    GUARD_BEGIN
    string     name(name_);
    dtype_t    d = dtype_of(dtype);
    scalarop_t op;
    auto       arg = [&](string const& pre) { return name.substr(pre.size()); };
    auto       starts = [&](string const& pre) { return name.rfind(pre, 0) == 0; };
    if (name == "identity") op = scalarop_t::make_identity(d);
    else if (name == "add") op = scalarop_t::make_add(d);
    else if (name == "mul") op = scalarop_t::make_mul(d);
    else if (name == "div") op = scalarop_t::make_div(d);
    else if (name == "neg") op = scalarop_t::make_neg(d);
    else if (name == "min") op = scalarop_t::make_min(d);
    else if (name == "max") op = scalarop_t::make_max(d);
    else if (name == "is_min") op = scalarop_t::make_is_min(d);
    else if (name == "is_max") op = scalarop_t::make_is_max(d);
    else if (name == "is_equal") op = scalarop_t::make_is_equal(d);
    else if (name == "sub") op = scalarop_t::make_sub(d);
    else if (name == "exp") op = scalarop_t::make_exp(d);
    else if (name == "sigmoid") op = scalarop_t::make_sigmoid(d);
    else if (name == "log") op = scalarop_t::make_log(d);
    else if (name == "sqrt") op = scalarop_t::make_sqrt(d);
    else if (name == "inverse") op = scalarop_t::make_inverse(d);
    else if (name == "inverse_sqrt") op = scalarop_t::make_inverse_sqrt(d);
    else if (name == "square") op = scalarop_t::make_square(d);
    else if (name == "relu") op = scalarop_t::make_relu(d);
    else if (name == "silu") op = scalarop_t::make_silu(d);
    else if (name == "rcp") op = scalarop_t::make_rcp(d);
    else if (name == "relu_deriv") op = scalarop_t::make_relu_deriv(d);
    else if (name == "conjugate") op = scalarop_t::make_conjugate(d);
    else if (name == "project_real") op = scalarop_t::make_project_real(d);
    else if (name == "project_imag") op = scalarop_t::make_project_imag(d);
    else if (name == "complex") op = scalarop_t::make_complex(d);
    else if (starts("scale:")) op = scalarop_t::make_scale(scalar_t(d, arg("scale:")));
    else if (starts("increment:")) op = scalarop_t::make_increment(scalar_t(d, arg("increment:")));
    else if (starts("power:")) op = scalarop_t::make_power(std::stoi(arg("power:")), d);
    else if (starts("convert:"))
        op = scalarop_t::make_convert_dtype(d, parse_with_ss<dtype_t>(arg("convert:")));
    else if (name == "silu_mul")
        op = scalarop_t::combine(scalarop_t::make_mul(d),
                                 {scalarop_t::make_silu(d), scalarop_t::make_identity(d)});
    else if (name == "exp_sub")
        op = scalarop_t::combine(scalarop_t::make_exp(d), {scalarop_t::make_sub(d)});
    else if (starts("softmax_v3_sum:")) {
        scalarop_t sc = scalarop_t::make_scale(scalar_t(d, arg("softmax_v3_sum:")));
        op = scalarop_t::combine(scalarop_t::make_exp(d),
                                 {scalarop_t::combine(sc, {scalarop_t::make_sub(d)})});
    } else if (starts("softmax_v3_norm:")) {
        scalarop_t sc = scalarop_t::make_scale(scalar_t(d, arg("softmax_v3_norm:")));
        scalarop_t ex = scalarop_t::combine(scalarop_t::make_exp(d),
                                            {scalarop_t::combine(sc, {scalarop_t::make_sub(d)})});
        op = scalarop_t::combine(scalarop_t::make_div(d), {ex, scalarop_t::make_identity(d)});
    } else
        throw std::runtime_error("unknown scalarop name " + name);
    string s = write_with_ss(op);
    if ((int)s.size() + 1 > buf_len) {
        throw std::runtime_error("buffer too small");
    }
    std::memcpy(buf, s.c_str(), s.size() + 1);
    return 0;
    GUARD_END
}

// "text|cppstr|simplified text|out dtype|num inputs"
int ref_scalarop_info(char const* text, char* buf, int buf_len)
{
    GUARD_BEGIN
    scalarop_t        op = parse_with_ss<scalarop_t>(string(text));
    std::stringstream ss;
    ss << op << "|" << op.to_cppstr() << "|" << op.simplify() << "|" << op.out_dtype() << "|"
       << op.num_inputs();
    string s = ss.str();
    if ((int)s.size() + 1 > buf_len) {
        throw std::runtime_error("buffer too small");
    }
    std::memcpy(buf, s.c_str(), s.size() + 1);
    return 0;
    GUARD_END
}

// Evaluates join over n elements; inns[i] is a dense array of the hole's dtype.
int ref_scalarop_eval(char const* text, uint64_t n, void* out, void const* const* inns)
{
    GUARD_BEGIN
    scalarop_t        op = parse_with_ss<scalarop_t>(string(text));
    int               k = op.num_inputs();
    vector<dbuffer_t> ins;
    for (int i = 0; i != k; ++i) {
        dtype_t d = op.inn_dtype(i).value();
        ins.emplace_back(d, make_buffer_reference(const_cast<void*>(inns[i]), n * dtype_size(d)));
    }
    dbuffer_t o(op.out_dtype(), make_buffer_reference(out, n * dtype_size(op.out_dtype())));
    vector<scalar_t> xs(k);
    for (uint64_t e = 0; e != n; ++e) {
        for (int i = 0; i != k; ++i) {
            xs[i] = ins[i].get(e);
        }
        o.set(e, op.eval(xs));
    }
    return 0;
    GUARD_END
}

} // extern "C"
