#include "einsum.h"

#include <algorithm>
#include <set>

namespace es {

einsum_t einsum_t::from_desc(es_einsummable_desc_t const* d)
{
    if (!d) fail(ES_BAD_ARGUMENT, "null einsummable descriptor");
    if (d->join_rank < 1 || d->join_rank > ES_MAX_RANK)
        fail(ES_BAD_DESCRIPTOR, "join_rank out of range");
    if (d->n_inn < 1 || d->n_inn > ES_MAX_INNS) fail(ES_BAD_DESCRIPTOR, "n_inn out of range");
    if (d->out_rank < 1 || d->out_rank > d->join_rank)
        fail(ES_BAD_DESCRIPTOR, "out_rank out of range");
    if (!d->join) fail(ES_BAD_DESCRIPTOR, "null join text");
    if (d->castable < -1 || d->castable > 3) fail(ES_BAD_DESCRIPTOR, "bad castable code");

    einsum_t e;
    e.join_shape.assign(d->join_shape, d->join_shape + d->join_rank);
    for (uint64_t s : e.join_shape) {
        // einsummable_t's constructor rejects zero extents (src/einsummable/einsummable.cc:79-83)
        if (s == 0) fail(ES_BAD_DESCRIPTOR, "einsummable: cannot have zero join size");
    }
    std::vector<bool> seen(d->join_rank, false);
    for (int k = 0; k != d->n_inn; ++k) {
        int r = d->inn_rank[k];
        if (r < 1 || r > d->join_rank) fail(ES_BAD_DESCRIPTOR, "input rank out of range");
        std::vector<int> modes(d->inn_modes[k], d->inn_modes[k] + r);
        std::set<int>    uniq(modes.begin(), modes.end());
        if ((int)uniq.size() != r) fail(ES_BAD_DESCRIPTOR, "input repeats a mode");
        for (int m : modes) {
            if (m < 0 || m >= d->join_rank) fail(ES_BAD_DESCRIPTOR, "input mode out of range");
            seen[m] = true;
        }
        e.inns.push_back(modes);
    }
    for (int m = d->out_rank; m != d->join_rank; ++m) {
        if (!seen[m]) fail(ES_BAD_DESCRIPTOR, "aggregated mode appears in no input");
    }
    e.out_rank = d->out_rank;
    e.castable = d->castable;
    e.join = scalarop_t::parse(d->join);
    if (e.has_aggregation() && e.castable == ES_CASTABLE_NONE) {
        // src/einsummable/einsummable.cc:39-41
        fail(ES_BAD_DESCRIPTOR, "Must have castable when aggregating.");
    }
    if (!e.join.uses_all_inputs(d->n_inn)) {
        // src/einsummable/einsummable.cc:43-49
        fail(ES_BAD_DESCRIPTOR, "einsummable inns do not match the holes of its join");
    }
    if (e.out_dtype() == ES_C64 &&
        (e.castable == ES_CASTABLE_MIN || e.castable == ES_CASTABLE_MAX)) {
        fail(ES_BAD_DESCRIPTOR, "min/max castable is not defined for complex");
    }
    return e;
}

einsum_t einsum_t::merge_adjacent_dims() const
{
    int r = join_rank();
    // terms = inputs + the output (modes 0..out_rank-1)
    std::vector<std::vector<int>> terms = inns;
    {
        std::vector<int> o(out_rank);
        for (int i = 0; i != out_rank; ++i) o[i] = i;
        terms.push_back(o);
    }
    // mode i and i+1 fuse iff in every term both are absent or i is directly followed by i+1
    auto fusable = [&](int i) {
        for (auto const& t : terms) {
            auto a = std::find(t.begin(), t.end(), i);
            auto b = std::find(t.begin(), t.end(), i + 1);
            bool ha = a != t.end(), hb = b != t.end();
            if (ha != hb) return false;
            if (ha && (a + 1) != b) return false;
        }
        return true;
    };
    std::vector<int> group_of(r);
    std::vector<int> group_begin;
    for (int i = 0; i != r; ++i) {
        if (i == 0 || !fusable(i - 1)) group_begin.push_back(i);
        group_of[i] = (int)group_begin.size() - 1;
    }
    if ((int)group_begin.size() == r) return *this;

    einsum_t m;
    m.castable = castable;
    m.join = join;
    m.join_shape.assign(group_begin.size(), 1);
    for (int i = 0; i != r; ++i) m.join_shape[group_of[i]] *= join_shape[i];
    auto remap = [&](std::vector<int> const& t) {
        std::vector<int> out;
        for (int mode : t) {
            int g = group_of[mode];
            if (group_begin[g] == mode) out.push_back(g);
        }
        return out;
    };
    for (auto const& t : inns) m.inns.push_back(remap(t));
    m.out_rank = (int)remap(terms.back()).size();
    return m;
}

std::string einsum_t::str() const
{
    std::string s;
    for (size_t k = 0; k != inns.size(); ++k) {
        if (k) s += ",";
        for (int m : inns[k]) s.push_back(char('a' + m));
    }
    s += "->";
    for (int m = 0; m != out_rank; ++m) s.push_back(char('a' + m));
    return s;
}

bool einsum_t::has_broadcast() const
{
    std::set<int> normal;
    for (auto const& t : inns)
        for (int m : t)
            if (m < out_rank) normal.insert(m);
    return (int)normal.size() != out_rank;
}

bool einsum_t::is_contraction() const
{
    return inns.size() == 2 && has_aggregation() && !has_broadcast() &&
           castable == ES_CASTABLE_ADD && join.is_mul();
}

uint64_t einsum_t::algorithmic_bytes() const
{
    uint64_t b = out_nelem() * dtype_size(out_dtype());
    for (int k = 0; k != (int)inns.size(); ++k) b += inn_nelem(k) * dtype_size(inn_dtype(k));
    return b;
}

bool einsum_t::is_straight_elementwise() const
{
    if (has_aggregation()) return false;
    for (auto const& t : inns) {
        if ((int)t.size() != join_rank()) return false;
        for (int i = 0; i != join_rank(); ++i)
            if (t[i] != i) return false;
    }
    return true;
}

bool einsum_t::is_permutation() const
{
    return inns.size() == 1 && !has_aggregation() && !has_broadcast() && join.is_identity();
}

uint64_t einsum_t::out_nelem() const
{
    uint64_t n = 1;
    for (int i = 0; i != out_rank; ++i) n *= join_shape[i];
    return n;
}

uint64_t einsum_t::inn_nelem(int k) const
{
    uint64_t n = 1;
    for (int m : inns[k]) n *= join_shape[m];
    return n;
}

uint64_t einsum_t::join_nelem() const
{
    uint64_t n = 1;
    for (uint64_t s : join_shape) n *= s;
    return n;
}

std::vector<uint64_t> einsum_t::inn_strides(int k) const
{
    std::vector<uint64_t> st(join_rank(), 0);
    uint64_t              s = 1;
    auto const&           t = inns[k];
    for (int i = (int)t.size() - 1; i >= 0; --i) {
        st[t[i]] = s;
        s *= join_shape[t[i]];
    }
    return st;
}

std::vector<uint64_t> einsum_t::out_strides() const
{
    std::vector<uint64_t> st(join_rank(), 0);
    uint64_t              s = 1;
    for (int i = out_rank - 1; i >= 0; --i) {
        st[i] = s;
        s *= join_shape[i];
    }
    return st;
}

std::string einsum_t::describe() const
{
    std::string s = str() + "|";
    for (size_t i = 0; i != join_shape.size(); ++i)
        s += (i ? "," : "") + std::to_string(join_shape[i]);
    s += "|" + std::to_string(out_rank) + "|";
    for (size_t k = 0; k != inns.size(); ++k) {
        if (k) s += ";";
        for (size_t j = 0; j != inns[k].size(); ++j)
            s += (j ? "," : "") + std::to_string(inns[k][j]);
    }
    return s;
}

std::string einsum_t::key() const
{
    return describe() + "|" + std::to_string(castable) + "|" + join.str();
}

} // namespace es
