// Typed expression trees for the join of an einsummable.
//
// Parses the reference's text form of a scalarop_t (operator<< / operator>>,
// src/einsummable/scalarop.cc:2878-3011) into a tree whose node dtypes follow
// the reference's typing rules (op_t::type_of, src/einsummable/scalarop.cc:762-905),
// and emits each tree as a CUDA C++ expression for the kernel generator.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "common.h"

namespace es {

enum class op_kind_t {
    constant, hole, variable, add, mul, exp, log, power, ite, convert, conj, real, imag, cplex
};

enum class compare_t { lt, gt, eq, le, ge };

struct node_t {
    op_kind_t           kind;
    int                 dtype;      // es_dtype_t of this node's value
    std::vector<node_t> children;
    // payloads
    double      value_re = 0.0;     // constant (real part)
    double      value_im = 0.0;     // constant (imag part, c64 only)
    int         arg = -1;           // hole
    std::string name;               // variable
    double      to_the = 0.0;       // power
    compare_t   compare = compare_t::lt;
};

struct scalarop_t {
    node_t             root;
    std::map<int, int> hole_dtypes; // arg -> dtype

    static scalarop_t parse(std::string const& text);

    int out_dtype() const { return root.dtype; }
    int num_inputs() const;         // max hole + 1
    bool uses_all_inputs(int n) const;

    // exactly *[hole@0, hole@1] (scalarop_t::is_mul, src/einsummable/scalarop.cc)
    bool is_mul() const;
    // exactly hole@0
    bool is_identity() const;

    // Text form, identical to the reference's operator<< for trees this parser accepts.
    std::string str() const;

    // CUDA expression in the node's compute type; arg k is written as names[k].
    std::string emit(std::vector<std::string> const& names) const;
};

// Compute type used in generated code for a dtype: f16 and f32 -> "float",
// f64 -> "double", c64 -> "cf".
char const* compute_type(int dtype);
// Storage type in generated code: "u16", "float", "double", "cf".
char const* storage_type(int dtype);

// Literal of the compute type holding `re` (+ i*im) rounded to `dtype`.
std::string literal(int dtype, double re, double im = 0.0);

// Round a double to the nearest f16 and return it as a float value.
float round_to_f16(double v);
uint16_t f16_bits(double v);

} // namespace es
