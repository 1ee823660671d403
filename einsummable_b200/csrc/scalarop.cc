#include "scalarop.h"

#include <cctype>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <limits>

namespace es {

namespace {

struct cursor_t {
    std::string const& s;
    size_t             i = 0;

    char peek() const { return i < s.size() ? s[i] : '\0'; }
    char get() { return i < s.size() ? s[i++] : '\0'; }
    bool eat(char const* lit)
    {
        size_t n = std::strlen(lit);
        if (s.compare(i, n, lit) == 0) {
            i += n;
            return true;
        }
        return false;
    }
    void expect(char const* lit)
    {
        if (!eat(lit)) {
            fail(ES_BAD_DESCRIPTOR,
                 "scalarop parse: expected '" + std::string(lit) + "' at offset " +
                     std::to_string(i) + " of '" + s + "'");
        }
    }
};

int parse_dtype(cursor_t& c)
{
    if (c.eat("f16")) return ES_F16;
    if (c.eat("f32")) return ES_F32;
    if (c.eat("f64")) return ES_F64;
    if (c.eat("c64")) return ES_C64;
    fail(ES_BAD_DESCRIPTOR, "scalarop parse: bad dtype at offset " + std::to_string(c.i));
}

double parse_number(cursor_t& c)
{
    char const* begin = c.s.c_str() + c.i;
    char*       end = nullptr;
    double      v = std::strtod(begin, &end);
    if (end == begin) {
        fail(ES_BAD_DESCRIPTOR, "scalarop parse: bad number at offset " + std::to_string(c.i));
    }
    c.i += size_t(end - begin);
    return v;
}

// "dtype|value" with INF / NINF / NAN tokens and "(re,im)" for c64
void parse_scalar(cursor_t& c, node_t& n)
{
    n.dtype = parse_dtype(c);
    c.expect("|");
    double const inf = std::numeric_limits<double>::infinity();
    if (c.eat("INF")) {
        n.value_re = inf;
    } else if (c.eat("NINF")) {
        n.value_re = -inf;
    } else if (c.eat("NAN")) {
        n.value_re = std::numeric_limits<double>::quiet_NaN();
    } else if (n.dtype == ES_C64) {
        c.expect("(");
        n.value_re = parse_number(c);
        c.expect(",");
        n.value_im = parse_number(c);
        c.expect(")");
    } else {
        n.value_re = parse_number(c);
    }
}

compare_t parse_compare(cursor_t& c)
{
    if (c.eat("<=")) return compare_t::le;
    if (c.eat(">=")) return compare_t::ge;
    if (c.eat("==")) return compare_t::eq;
    if (c.eat("<")) return compare_t::lt;
    if (c.eat(">")) return compare_t::gt;
    fail(ES_BAD_DESCRIPTOR, "scalarop parse: bad compare");
}

int num_children(op_kind_t k)
{
    switch (k) {
        case op_kind_t::constant:
        case op_kind_t::hole:
        case op_kind_t::variable: return 0;
        case op_kind_t::add:
        case op_kind_t::mul:
        case op_kind_t::cplex: return 2;
        case op_kind_t::ite: return 4;
        default: return 1;
    }
}

// The reference's typing rules: op_t::_type_* (src/einsummable/scalarop.cc:762-905).
int type_of(node_t const& n)
{
    auto const& c = n.children;
    auto        bad = [&](char const* what) -> int {
        fail(ES_BAD_DESCRIPTOR, std::string("scalarop type failure in ") + what);
    };
    switch (n.kind) {
        case op_kind_t::add:
        case op_kind_t::mul:
            if (c[0].dtype != c[1].dtype) bad("add/mul");
            return c[0].dtype;
        case op_kind_t::exp:
        case op_kind_t::log:
        case op_kind_t::power:
            if (c[0].dtype == ES_C64) bad("exp/log/power of complex");
            return c[0].dtype;
        case op_kind_t::ite:
            if (c[0].dtype != c[1].dtype || c[0].dtype == ES_C64 || c[2].dtype != c[3].dtype)
                bad("ite");
            return c[2].dtype;
        case op_kind_t::convert:
            if (c[0].dtype == ES_C64 || n.dtype == ES_C64 || c[0].dtype == n.dtype) bad("convert");
            return n.dtype;
        case op_kind_t::conj:
            if (c[0].dtype != ES_C64) bad("conj");
            return ES_C64;
        case op_kind_t::real:
        case op_kind_t::imag:
            if (c[0].dtype != ES_C64) bad("real/imag");
            return ES_F32;
        case op_kind_t::cplex:
            if (c[0].dtype != ES_F32 || c[1].dtype != ES_F32) bad("complex");
            return ES_C64;
        default: return n.dtype;
    }
}

node_t parse_node(cursor_t& c, int depth)
{
    if (depth > 256) {
        fail(ES_BAD_DESCRIPTOR, "scalarop parse: tree too deep");
    }
    node_t n;
    n.dtype = ES_F32;
    char p = c.peek();
    if (p == 'c') {
        if (c.eat("constant{")) {
            n.kind = op_kind_t::constant;
            parse_scalar(c, n);
            c.expect("}");
        } else if (c.eat("conj")) {
            n.kind = op_kind_t::conj;
        } else if (c.eat("complex")) {
            n.kind = op_kind_t::cplex;
        } else {
            fail(ES_BAD_DESCRIPTOR, "scalarop parse: bad token at c");
        }
    } else if (p == 'v') {
        c.expect("variable{");
        n.kind = op_kind_t::variable;
        while (std::isalnum((unsigned char)c.peek()) || c.peek() == '_') {
            n.name.push_back(c.get());
        }
        c.expect("|");
        n.dtype = parse_dtype(c);
        c.expect("}");
    } else if (p == 'h') {
        c.expect("hole|");
        n.kind = op_kind_t::hole;
        n.dtype = parse_dtype(c);
        c.expect("@");
        double v = parse_number(c);
        n.arg = int(v);
        if (n.arg < 0 || n.arg >= ES_MAX_INNS || double(n.arg) != v) {
            fail(ES_BAD_DESCRIPTOR, "scalarop parse: bad hole index");
        }
    } else if (p == '+') {
        c.get();
        n.kind = op_kind_t::add;
    } else if (p == '*') {
        c.get();
        n.kind = op_kind_t::mul;
    } else if (p == 'e') {
        c.expect("exp");
        n.kind = op_kind_t::exp;
    } else if (p == 'l') {
        c.expect("log");
        n.kind = op_kind_t::log;
    } else if (p == 'p') {
        c.expect("power{");
        n.kind = op_kind_t::power;
        n.to_the = parse_number(c);
        c.expect("}");
    } else if (p == 'i') {
        if (c.eat("ite_")) {
            n.kind = op_kind_t::ite;
            n.compare = parse_compare(c);
        } else if (c.eat("imag")) {
            n.kind = op_kind_t::imag;
        } else {
            fail(ES_BAD_DESCRIPTOR, "scalarop parse: bad token at i");
        }
    } else if (p == 't') {
        c.expect("to_");
        n.kind = op_kind_t::convert;
        n.dtype = parse_dtype(c);
    } else if (p == 'r') {
        c.expect("real");
        n.kind = op_kind_t::real;
    } else {
        fail(ES_BAD_DESCRIPTOR,
             "scalarop parse: unexpected character at offset " + std::to_string(c.i));
    }

    int nc = num_children(n.kind);
    if (nc > 0) {
        c.expect("[");
        for (int i = 0; i != nc; ++i) {
            if (i) c.expect(",");
            n.children.push_back(parse_node(c, depth + 1));
        }
        c.expect("]");
        n.dtype = type_of(n);
    }
    return n;
}

void collect_holes(node_t const& n, std::map<int, int>& holes)
{
    if (n.kind == op_kind_t::hole) {
        auto it = holes.find(n.arg);
        if (it != holes.end() && it->second != n.dtype) {
            fail(ES_BAD_DESCRIPTOR, "scalarop: one hole used with two dtypes");
        }
        holes[n.arg] = n.dtype;
    }
    if (n.kind == op_kind_t::variable) {
        fail(ES_BAD_DESCRIPTOR,
             "scalarop: unresolved variable '" + n.name +
                 "' (replace_scalar_variables must run before build)");
    }
    for (auto const& ch : n.children) {
        collect_holes(ch, holes);
    }
}

char const* compare_str(compare_t c)
{
    switch (c) {
        case compare_t::lt: return "<";
        case compare_t::gt: return ">";
        case compare_t::eq: return "==";
        case compare_t::le: return "<=";
        case compare_t::ge: return ">=";
    }
    return "?";
}

std::string fmt_g(double v)
{
    char buf[64];
    std::snprintf(buf, sizeof buf, "%g", v);
    return buf;
}

std::string scalar_str(int dtype, double re, double im)
{
    std::string s = std::string(dtype_name(dtype)) + "|";
    if (dtype == ES_C64) {
        return s + "(" + fmt_g(re) + "," + fmt_g(im) + ")";
    }
    if (std::isnan(re)) return s + "NAN";
    if (std::isinf(re)) return s + (re > 0 ? "INF" : "NINF");
    return s + fmt_g(re);
}

void write_node(node_t const& n, std::string& out)
{
    switch (n.kind) {
        case op_kind_t::constant:
            out += "constant{" + scalar_str(n.dtype, n.value_re, n.value_im) + "}";
            break;
        case op_kind_t::hole:
            out += std::string("hole|") + dtype_name(n.dtype) + "@" + std::to_string(n.arg);
            break;
        case op_kind_t::variable:
            out += "variable{" + n.name + "|" + dtype_name(n.dtype) + "}";
            break;
        case op_kind_t::add: out += "+"; break;
        case op_kind_t::mul: out += "*"; break;
        case op_kind_t::exp: out += "exp"; break;
        case op_kind_t::log: out += "log"; break;
        case op_kind_t::power: out += "power{" + fmt_g(n.to_the) + "}"; break;
        case op_kind_t::ite: out += std::string("ite_") + compare_str(n.compare); break;
        case op_kind_t::convert: out += std::string("to_") + dtype_name(n.dtype); break;
        case op_kind_t::conj: out += "conj"; break;
        case op_kind_t::real: out += "real"; break;
        case op_kind_t::imag: out += "imag"; break;
        case op_kind_t::cplex: out += "complex"; break;
    }
    if (!n.children.empty()) {
        out += "[";
        for (size_t i = 0; i != n.children.size(); ++i) {
            if (i) out += ",";
            write_node(n.children[i], out);
        }
        out += "]";
    }
}

bool is_hole(node_t const& n, int arg)
{
    return n.kind == op_kind_t::hole && n.arg == arg;
}

std::string emit_node(node_t const& n, std::vector<std::string> const& names)
{
    auto ch = [&](int i) { return emit_node(n.children[i], names); };
    bool half = n.dtype == ES_F16;
    switch (n.kind) {
        case op_kind_t::constant: return literal(n.dtype, n.value_re, n.value_im);
        case op_kind_t::hole: return names.at(n.arg);
        case op_kind_t::variable: fail(ES_BAD_DESCRIPTOR, "unresolved variable in emit");
        case op_kind_t::add:
            if (n.dtype == ES_C64) return "cf_add(" + ch(0) + "," + ch(1) + ")";
            return "(" + ch(0) + "+" + ch(1) + ")";
        case op_kind_t::mul:
            if (n.dtype == ES_C64) return "cf_mul(" + ch(0) + "," + ch(1) + ")";
            return "(" + ch(0) + "*" + ch(1) + ")";
        case op_kind_t::exp:
            if (n.dtype == ES_F64) return "exp(" + ch(0) + ")";
            return std::string(half ? "__expf(" : "expf(") + ch(0) + ")";
        case op_kind_t::log:
            if (n.dtype == ES_F64) return "log(" + ch(0) + ")";
            return std::string(half ? "__logf(" : "logf(") + ch(0) + ")";
        case op_kind_t::power: {
            double      p = n.to_the;
            std::string x = ch(0);
            bool        f64 = n.dtype == ES_F64;
            std::string one = f64 ? "1.0" : "1.0f";
            if (p == 1.0) return x;
            if (p == 2.0) return "es_sq(" + x + ")";
            if (p == 3.0) return "es_cube(" + x + ")";
            if (p == -1.0) {
                if (half) return "es_rcp_approx(" + x + ")";
                return "(" + one + "/" + x + ")";
            }
            if (p == -2.0) return "(" + one + "/es_sq(" + x + "))";
            if (p == 0.5) return std::string(f64 ? "sqrt(" : "sqrtf(") + x + ")";
            if (p == -0.5) {
                if (half) return "rsqrtf(" + x + ")";
                return "(" + one + std::string(f64 ? "/sqrt(" : "/sqrtf(") + x + "))";
            }
            // general exponent: the reference evaluates pow(x, T(p)) in the node dtype
            if (f64) return "pow(" + x + "," + literal(ES_F64, p) + ")";
            return "powf(" + x + "," + literal(n.dtype, p) + ")";
        }
        case op_kind_t::ite:
            return "((" + ch(0) + compare_str(n.compare) + ch(1) + ")?" + ch(2) + ":" + ch(3) + ")";
        case op_kind_t::convert: {
            int src = n.children[0].dtype;
            std::string x = ch(0);
            if (n.dtype == ES_F16) {
                // value is kept in a float but must carry f16 rounding from here on
                return src == ES_F64 ? "es_rt_h((float)(" + x + "))" : "es_rt_h(" + x + ")";
            }
            if (n.dtype == ES_F32) return src == ES_F64 ? "((float)(" + x + "))" : x;
            return "((double)(" + x + "))";
        }
        case op_kind_t::conj: return "cf_conj(" + ch(0) + ")";
        case op_kind_t::real: return "(" + ch(0) + ").re";
        case op_kind_t::imag: return "(" + ch(0) + ").im";
        case op_kind_t::cplex: return "cf_make(" + ch(0) + "," + ch(1) + ")";
    }
    fail(ES_BAD_DESCRIPTOR, "emit: unknown node kind");
}

} // namespace

uint16_t f16_bits(double v)
{
    // round-to-nearest-even double -> binary16
    if (std::isnan(v)) return 0x7e00;
    uint16_t sign = std::signbit(v) ? 0x8000 : 0;
    double   a = std::fabs(v);
    if (std::isinf(a)) return sign | 0x7c00;
    if (a == 0.0) return sign;
    int    e;
    double m = std::frexp(a, &e); // a = m * 2^e, m in [0.5, 1)
    // normal half: exponent range e-1 in [-14, 15]
    int he = e - 1;
    if (he < -14) {
        // subnormal: value = k * 2^-24
        double k = std::nearbyint(a * 16777216.0);
        if (k >= 1024.0) return sign | 0x0400;
        return sign | uint16_t(k);
    }
    double frac = std::nearbyint((m * 2.0 - 1.0) * 1024.0); // 10-bit mantissa, RNE via nearbyint
    if (frac >= 1024.0) {
        frac = 0.0;
        he += 1;
    }
    if (he > 15) return sign | 0x7c00;
    return sign | uint16_t((he + 15) << 10) | uint16_t(frac);
}

float round_to_f16(double v)
{
    uint16_t h = f16_bits(v);
    int      s = h >> 15;
    int      e = (h >> 10) & 31;
    int      m = h & 1023;
    double   r;
    if (e == 31) {
        r = m ? std::numeric_limits<double>::quiet_NaN() : std::numeric_limits<double>::infinity();
    } else if (e == 0) {
        r = std::ldexp(double(m), -24);
    } else {
        r = std::ldexp(double(m + 1024), e - 25);
    }
    return float(s ? -r : r);
}

char const* compute_type(int dtype)
{
    switch (dtype) {
        case ES_F16:
        case ES_F32: return "float";
        case ES_F64: return "double";
        case ES_C64: return "cf";
    }
    return "?";
}

char const* storage_type(int dtype)
{
    switch (dtype) {
        case ES_F16: return "u16";
        case ES_F32: return "float";
        case ES_F64: return "double";
        case ES_C64: return "cf";
    }
    return "?";
}

static std::string f32_literal(float f)
{
    uint32_t bits;
    std::memcpy(&bits, &f, 4);
    char buf[64];
    std::snprintf(buf, sizeof buf, "__uint_as_float(0x%08xu)", bits);
    return buf;
}

std::string literal(int dtype, double re, double im)
{
    char buf[96];
    switch (dtype) {
        case ES_F16: return f32_literal(round_to_f16(re));
        case ES_F32: return f32_literal(float(re));
        case ES_F64: {
            uint64_t bits;
            std::memcpy(&bits, &re, 8);
            std::snprintf(buf, sizeof buf, "__longlong_as_double(0x%016llxll)",
                          (unsigned long long)bits);
            return buf;
        }
        case ES_C64:
            return "cf_make(" + f32_literal(float(re)) + "," + f32_literal(float(im)) + ")";
    }
    fail(ES_BAD_DESCRIPTOR, "literal: bad dtype");
}

scalarop_t scalarop_t::parse(std::string const& text)
{
    cursor_t   c{text};
    scalarop_t op;
    op.root = parse_node(c, 0);
    if (c.i != text.size()) {
        fail(ES_BAD_DESCRIPTOR, "scalarop parse: trailing characters in '" + text + "'");
    }
    collect_holes(op.root, op.hole_dtypes);
    return op;
}

int scalarop_t::num_inputs() const
{
    return hole_dtypes.empty() ? 0 : hole_dtypes.rbegin()->first + 1;
}

bool scalarop_t::uses_all_inputs(int n) const
{
    if ((int)hole_dtypes.size() != n) return false;
    for (int i = 0; i != n; ++i) {
        if (!hole_dtypes.count(i)) return false;
    }
    return true;
}

bool scalarop_t::is_mul() const
{
    return root.kind == op_kind_t::mul && is_hole(root.children[0], 0) &&
           is_hole(root.children[1], 1);
}

bool scalarop_t::is_identity() const
{
    return is_hole(root, 0);
}

std::string scalarop_t::str() const
{
    std::string s;
    write_node(root, s);
    return s;
}

std::string scalarop_t::emit(std::vector<std::string> const& names) const
{
    return emit_node(root, names);
}

} // namespace es
