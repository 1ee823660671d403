// Fusion across node boundaries of a memgraph: an elementwise apply node is folded into the nodes
// that read its result, so the intermediate tensor never makes its round trip through device memory.
//
// The reference keeps such chains as separate nodes (softmax = 5 nodes, src/einsummable/gwriter.cc:830-855;
// RMSNorm = 8 nodes, llama/modules.cc:126-195); the es_b200 library compiles any scalarop tree into one
// kernel, so folding a producer A into its reader B is a substitution of A's join for one of B's holes
// plus a composition of the index maps.  The result is again a memgraph_t (the folded node stays in the
// list as an alloc node, which launches nothing, so ids keep indexing the list), valid both for in-order
// and for dependency-ordered execution: a reader that now reads A's inputs takes over A's dependencies,
// and every later node that writes into memory A read -- the memgraph reuses freed memory, and the del
// that freed it only knew A as a reader -- is made to depend on the readers.  gpu_program_t,
// gpu_exchange_program_t and es_exchange::make_units take the folded graph as they take any other.
//
// A is folded into B when
//   * A is an elementwise einsummable (no aggregation), B an einsummable that is not a plain contraction
//     (those run on the tensor cores with the join x0 * x1),
//   * every reader of A's result qualifies (A is then folded into each of them), reads it in one input
//     slot, and the result is neither saved nor read by a move, a copy or an evict,
//   * A and B iterate over the same number of points, and B reads A's result with exactly the shape and
//     dtype A wrote it in (a taskgraph node may view the same bytes under another shape or dtype,
//     src/einsummable/taskgraph.cc:765-793: such readers are left alone),
//   * nothing between A and its last reader in node order writes memory A reads, and no reader does,
//   * the folded node has at most 8 inputs (ES_MAX_INNS of es_b200.h).
//
// The same rules, in the same order, as einsummable_b200/fuse.py (fuse_elementwise_chains), which works on
// the memgraph as data; the two are compared node by node in the tests.
//
// Header-only; include from a file that sees the reference's src/ tree.
#pragma once
#if __has_include("../../einsummable/memgraph.h")
#include "../../einsummable/memgraph.h"
#else
#include "src/einsummable/memgraph.h"
#endif

#include <algorithm>
#include <map>
#include <optional>
#include <set>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace es_fuse {

constexpr int MAX_INNS = 8;

namespace detail {

using region_t = std::pair<uint64_t, uint64_t>; // offset, size

inline bool overlap(region_t const& a, region_t const& b)
{
    return a.first < b.first + b.second && b.first < a.first + a.second;
}

inline region_t region(mem_t const& m)
{
    return {m.offset, m.size};
}

// what a node writes in location `loc`'s memory
inline std::optional<region_t> written_region(memgraph_t::op_t const& op, int loc)
{
    if (op.is_apply()) {
        auto const& a = op.get_apply();
        if (a.loc != loc) return std::nullopt;
        return region(a.mems[0]);
    }
    if (op.is_constant()) {
        auto const& c = op.get_constant();
        if (c.loc != loc) return std::nullopt;
        return region_t{c.offset, c.get_size()};
    }
    if (op.is_move()) { // the destination pulls the bytes at the move's place in its own order
        auto const& m = op.get_move();
        if (m.get_dst_loc() != loc) return std::nullopt;
        return region_t{std::get<1>(m.dst), m.size};
    }
    if (op.is_copy()) {
        auto const& c = op.get_copy();
        if (c.loc != loc) return std::nullopt;
        return region_t{c.dst_offset, c.size};
    }
    if (op.is_load()) {
        auto const& l = op.get_load();
        if (l.dst.loc != loc) return std::nullopt;
        return region_t{l.dst.offset, l.dst.size};
    }
    return std::nullopt;
}

inline bool elementwise(einsummable_t const& e)
{
    return e.out_rank == int(e.join_shape.size());
}

// one "hole|<dtype>@<slot>" of a join's text form
struct hole_t {
    size_t      begin, end;
    std::string dtype;
    int         slot;
};

inline std::vector<hole_t> holes_of(std::string const& text)
{
    std::vector<hole_t> out;
    size_t              pos = 0;
    while ((pos = text.find("hole|", pos)) != std::string::npos) {
        size_t at = text.find('@', pos);
        if (at == std::string::npos) break;
        size_t end = at + 1;
        while (end < text.size() && text[end] >= '0' && text[end] <= '9') ++end;
        out.push_back({pos, end, text.substr(pos + 5, at - pos - 5), std::stoi(text.substr(at + 1, end - at - 1))});
        pos = end;
    }
    return out;
}

// a contraction the tensor-core kernel serves as it stands: x0 * x1 summed over the aggregated modes
inline bool plain_contraction(einsummable_t const& e)
{
    if (!e.castable || e.castable.value() != castable_t::add || e.inns.size() != 2 || elementwise(e)) return false;
    std::string text = write_with_ss(e.join);
    auto        holes = holes_of(text);
    if (holes.size() != 2 || holes[0].slot != 0 || holes[1].slot != 1) return false;
    return text == "*[hole|" + holes[0].dtype + "@0,hole|" + holes[1].dtype + "@1]";
}

inline uint64_t product(std::vector<uint64_t> const& v)
{
    uint64_t r = 1;
    for (uint64_t x : v) r *= x;
    return r;
}

// b with its input `slot` replaced by the expression a
inline einsummable_t compose(einsummable_t const& a, einsummable_t const& b, int slot)
{
    int const   shift = int(a.inns.size()) - 1;
    std::string a_text = write_with_ss(a.join), b_text = write_with_ss(b.join);
    std::string a_new;
    {
        size_t pos = 0;
        for (hole_t const& h : holes_of(a_text)) {
            a_new += a_text.substr(pos, h.begin - pos) + "hole|" + h.dtype + "@" + std::to_string(h.slot + slot);
            pos = h.end;
        }
        a_new += a_text.substr(pos);
    }
    std::string text;
    size_t      pos = 0;
    for (hole_t const& h : holes_of(b_text)) {
        text += b_text.substr(pos, h.begin - pos);
        if (h.slot == slot) text += a_new;
        else text += "hole|" + h.dtype + "@" + std::to_string(h.slot < slot ? h.slot : h.slot + shift);
        pos = h.end;
    }
    text += b_text.substr(pos);
    std::vector<int> const&       via = b.inns[slot]; // a's mode m is b's mode via[m]
    std::vector<std::vector<int>> inns(b.inns.begin(), b.inns.begin() + slot);
    for (auto const& inn : a.inns) {
        std::vector<int> mapped;
        for (int m : inn) mapped.push_back(via[m]);
        inns.push_back(mapped);
    }
    inns.insert(inns.end(), b.inns.begin() + slot + 1, b.inns.end());
    return einsummable_t(b.join_shape, inns, b.out_rank, parse_with_ss<scalarop_t>(text), b.castable);
}

} // namespace detail

struct folded_t {
    memgraph_t       memgraph;
    std::vector<int> folded; // ids of the nodes folded away, in node order
};

// `saved`: the regions that hold the graph's saved results (the save_to_data of memgraph_t::make);
// a node that writes into one of them is never folded away.
inline folded_t fold_elementwise(memgraph_t const& graph, std::vector<memloc_t> const& saved)
{
    using namespace detail;
    folded_t out{graph, {}};
    auto&    nodes = out.memgraph.nodes;
    int const n = int(nodes.size());
    std::vector<char> alive(n, 1);
    for (int ia = 0; ia != n; ++ia) {
        if (!nodes[ia].op.is_einsummable()) continue;
        memgraph_t::apply_t const a = nodes[ia].op.get_apply();
        einsummable_t const&      ea = a.get_einsummable();
        if (!elementwise(ea)) continue;
        region_t const a_out = region(a.mems[0]);
        int const      loc = a.loc;
        bool           is_saved = false;
        for (memloc_t const& s : saved) is_saved = is_saved || (s.loc == loc && overlap(a_out, {s.offset, s.size}));
        if (is_saved) continue;
        // readers of the result: apply nodes after A that depend on it and read exactly its region
        std::vector<int> readers;
        bool             shipped = false;
        for (int ib = ia + 1; ib != n && !shipped; ++ib) {
            if (!alive[ib] || !nodes[ib].inns.count(ia)) continue;
            auto const& op = nodes[ib].op;
            if (op.is_move() || op.is_copy() || op.is_evict()) {
                shipped = true; // another location, a copy or the storage reads the materialised tensor
            } else if (op.is_apply() && op.get_apply().loc == loc) {
                auto const& mems = op.get_apply().mems;
                for (size_t k = 1; k < mems.size(); ++k) {
                    if (region(mems[k]) == a_out) {
                        readers.push_back(ib);
                        break;
                    }
                }
            }
        }
        if (shipped || readers.empty()) continue;
        std::vector<region_t> a_reads;
        uint64_t              in_bytes = 0;
        for (size_t k = 1; k < a.mems.size(); ++k) {
            a_reads.push_back(region(a.mems[k]));
            in_bytes += a.mems[k].size;
        }
        // with R readers the producer is evaluated R times instead of once: R * in(A) bytes against
        // in(A) + (R + 1) * out(A) before
        uint64_t const n_r = readers.size();
        if ((n_r - 1) * in_bytes > (n_r + 1) * a_out.second) continue;
        std::vector<std::pair<int, int>> plans; // reader, slot
        for (int ib : readers) {
            auto const& op = nodes[ib].op;
            if (!op.is_einsummable()) break;
            memgraph_t::apply_t const& b = op.get_apply();
            einsummable_t const&       eb = b.get_einsummable();
            if (plain_contraction(eb)) break;
            std::vector<int> slots;
            for (size_t k = 1; k < b.mems.size(); ++k)
                if (region(b.mems[k]) == a_out) slots.push_back(int(k) - 1);
            if (slots.size() != 1 || product(ea.join_shape) != product(eb.join_shape)) break;
            std::vector<int> const& via = eb.inns[slots[0]];
            bool                    same_shape = int(via.size()) == ea.out_rank;
            for (int m = 0; same_shape && m != ea.out_rank; ++m) same_shape = ea.join_shape[m] == eb.join_shape[via[m]];
            if (!same_shape) break; // the reader views the bytes under another shape
            if (eb.inn_dtype(slots[0]) != ea.out_dtype()) break; // ... or another dtype
            if (int(eb.inns.size()) - 1 + int(ea.inns.size()) > MAX_INNS) break;
            bool clobbers = false;
            for (region_t const& r : a_reads) clobbers = clobbers || overlap(region(b.mems[0]), r);
            if (clobbers) break;
            plans.push_back({ib, slots[0]});
        }
        if (plans.size() != readers.size()) continue;
        bool hazard = false;
        for (int ic = ia + 1; ic < readers.back() && !hazard; ++ic) {
            if (!alive[ic]) continue;
            auto w = written_region(nodes[ic].op, loc);
            if (!w) continue;
            for (region_t const& r : a_reads) hazard = hazard || overlap(*w, r);
        }
        if (hazard) continue;
        std::set<int> const a_inns = nodes[ia].inns;
        for (auto const& [ib, slot] : plans) {
            memgraph_t::apply_t b = nodes[ib].op.get_apply();
            einsummable_t       e = compose(ea, b.get_einsummable(), slot);
            std::vector<mem_t>  mems(b.mems.begin(), b.mems.begin() + 1 + slot);
            mems.insert(mems.end(), a.mems.begin() + 1, a.mems.end());
            mems.insert(mems.end(), b.mems.begin() + 2 + slot, b.mems.end());
            b.mems = mems;
            b.op = e;
            nodes[ib].op = memgraph_t::op_t(b);
            nodes[ib].inns.erase(ia);
            nodes[ib].inns.insert(a_inns.begin(), a_inns.end());
        }
        // later writers into memory A read must now also wait for the readers
        for (int ic = readers.back() + 1; ic != n; ++ic) {
            if (!alive[ic]) continue;
            auto w = written_region(nodes[ic].op, loc);
            if (!w) continue;
            bool hits = false;
            for (region_t const& r : a_reads) hits = hits || overlap(*w, r);
            if (hits)
                for (int ib : readers) nodes[ic].inns.insert(ib);
        }
        alive[ia] = 0;
        out.folded.push_back(ia);
        // the folded node stays as a node that launches nothing
        nodes[ia].op = memgraph_t::op_t(memgraph_t::alloc_t{loc, a_out.first, a_out.second});
    }
    // the edges the other way round
    for (auto& node : nodes) node.outs.clear();
    for (int id = 0; id != n; ++id)
        for (int i : nodes[id].inns) nodes[i].outs.insert(id);
    return out;
}

// ---- the attention chain --------------------------------------------------------------------------------
//
// softmax(Q K^T + mask) V is five apply nodes in the reference's graphs (src/einsummable/gwriter.cc:830-855,
// llama/modules.cc:285-383) -- after fold_elementwise: the scores contraction, the row maximum of
// scores + mask, the row sum of the exponentials, the normalised probabilities in f16, the contraction
// with V.  fold_attention replaces every such chain by ONE node for the library's attention kernel
// (es_b200_launch_attention / es_b200_program_add_attention).  A memgraph_t has no such op, so the result
// is a memgraph_t plus a map: the chain's last node keeps its place and its einsummable but now lists the
// memories [out, Q, K, V, mask] (five memories on a two-input einsummable: whoever executes it without
// looking at the map fails on the input count instead of computing something else), the map gives its
// descriptor; the other four nodes become alloc nodes.  The conditions are those of the fold above: the
// four intermediate results have no other reader and are neither saved nor shipped, nothing between the
// first and the last node writes memory the chain now reads later; later writers into that memory are
// made to wait for the new node.  The same rules as fuse.py: fuse_attention.

struct attention_t {
    uint32_t batch = 0, heads = 0, rows = 0, keys = 0, head_dim = 0;
    int32_t  skip_known = 0; // the mask is a lower-triangular fill (0 / -inf) starting at skip_from:
    int32_t  skip_from = 0;  // the kernel computes it and leaves out the key blocks above the diagonal
    int64_t  q_stride[3] = {0, 0, 0}, k_stride[3] = {0, 0, 0}, v_stride[3] = {0, 0, 0}, out_stride[3] = {0, 0, 0};
    int64_t  mask_stride = 0;

    // what the kernel serves: head dim a multiple of 8 up to 128, strides multiples of 8
    bool eligible() const
    {
        if (head_dim % 8 || head_dim > 128 || batch > 65535 || heads > 65535) return false;
        for (int i = 0; i != 3; ++i)
            if (q_stride[i] % 8 || k_stride[i] % 8 || v_stride[i] % 8 || out_stride[i] % 8) return false;
        return true;
    }
};

struct attention_node_t {
    attention_t desc;
    int         loc = 0;
    mem_t       out, q, k, v, mask;
};

struct attention_folded_t {
    memgraph_t                      memgraph;
    std::map<int, attention_node_t> attention; // by node id
};

namespace detail {

inline std::string normal_join(std::string const& text)
{
    return write_with_ss(parse_with_ss<scalarop_t>(text));
}

inline std::vector<int64_t> row_major_strides(std::vector<uint64_t> const& shape)
{
    std::vector<int64_t> st(shape.size(), 1);
    for (int i = int(shape.size()) - 2; i >= 0; --i) st[i] = st[i + 1] * int64_t(shape[i + 1]);
    return st;
}

inline std::vector<int> sorted_modes(std::vector<int> v)
{
    std::sort(v.begin(), v.end());
    return v;
}

struct chain_t {
    int              idx[5]; // scores, max, sum, probabilities, output
    attention_node_t node;
};

struct chain_matcher_t {
    std::vector<memgraph_t::node_t> const& nodes;
    std::vector<char> const&               alive;
    std::vector<memloc_t> const&           saved;
    std::map<int, attention_node_t> const& done; // the nodes that already stand for a whole chain
    std::string const x16 = normal_join("*[hole|f16@0,hole|f16@1]");
    std::string const x = "to_f32[+[hole|f16@0,hole|f16@1]]";
    std::string const e = "exp[+[" + x + ",*[constant{f32|-1},hole|f32@2]]]";
    std::string const j_max = normal_join(x);
    std::string const j_sum = normal_join(e);
    std::string const j_norm = normal_join("to_f16[*[" + e + ",power{-1}[hole|f32@3]]]");

    // the apply nodes that read node ix's result, if they are exactly `want` many, read it as written,
    // and nothing ships or saves it
    std::optional<std::vector<int>> sole_readers(int ix, size_t want) const
    {
        auto const& a = nodes[ix].op.get_apply();
        region_t    out = region(a.mems[0]);
        for (memloc_t const& s : saved)
            if (s.loc == a.loc && overlap(out, {s.offset, s.size})) return std::nullopt;
        std::vector<int> got;
        for (int ib = ix + 1; ib != int(nodes.size()); ++ib) {
            if (!alive[ib] || !nodes[ib].inns.count(ix)) continue;
            auto const& op = nodes[ib].op;
            if (op.is_move() || op.is_copy() || op.is_evict()) return std::nullopt;
            if (op.is_apply()) {
                auto const& b = op.get_apply();
                bool        reads = false;
                for (size_t k = 1; k < b.mems.size(); ++k) reads = reads || region(b.mems[k]) == out;
                if (b.loc != a.loc || !b.is_einsummable() || done.count(ib) || !reads) return std::nullopt;
                got.push_back(ib);
            }
        }
        if (got.size() != want) return std::nullopt;
        return got;
    }

    std::optional<chain_t> match(int i_s) const
    {
        auto const&          s = nodes[i_s].op.get_apply();
        einsummable_t const& es = s.get_einsummable();
        if (es.join_shape.size() != 5 || es.out_rank != 4 || !plain_contraction(es) || write_with_ss(es.join) != x16)
            return std::nullopt;
        uint64_t const b = es.join_shape[0], h = es.join_shape[1], rows = es.join_shape[2], keys = es.join_shape[3],
                       d = es.join_shape[4];
        int q_slot = -1, k_slot = -1;
        for (int slot = 0; slot != int(es.inns.size()); ++slot) {
            auto const& modes = es.inns[slot];
            if (sorted_modes(modes) == std::vector<int>{0, 1, 2, 4} && modes.back() == 4) q_slot = slot;
            else if (sorted_modes(modes) == std::vector<int>{0, 1, 3, 4} && modes.back() == 4) k_slot = slot;
        }
        if (q_slot < 0 || k_slot < 0) return std::nullopt;
        auto strides = [&](einsummable_t const& e, std::vector<int> const& modes, int row_mode, int64_t* out3) {
            std::vector<uint64_t> shape;
            for (int m : modes) shape.push_back(e.join_shape[m]);
            auto st = row_major_strides(shape);
            for (size_t i = 0; i != modes.size(); ++i) {
                if (modes[i] == 0) out3[0] = st[i];
                if (modes[i] == 1) out3[1] = st[i];
                if (modes[i] == row_mode) out3[2] = st[i];
            }
        };
        auto r_s = sole_readers(i_s, 3);
        if (!r_s) return std::nullopt;
        int const   i_m = (*r_s)[0], i_l = (*r_s)[1], i_p = (*r_s)[2];
        auto const &m = nodes[i_m].op.get_apply(), &l = nodes[i_l].op.get_apply(), &pn = nodes[i_p].op.get_apply();
        einsummable_t const &em = m.get_einsummable(), &el = l.get_einsummable(), &ep = pn.get_einsummable();
        region_t const        s_out = region(s.mems[0]);
        std::vector<uint64_t> shape4{b, h, rows, keys};
        using vv = std::vector<std::vector<int>>;
        std::vector<int> const full{0, 1, 2, 3};
        auto                   max_c = [](einsummable_t const& e, castable_t c) { return e.castable && e.castable.value() == c; };
        if (!(max_c(em, castable_t::max) && em.out_rank == 3 && em.join_shape == shape4 && em.inns == vv{full, {2, 3}} &&
              write_with_ss(em.join) == j_max && m.mems.size() == 3 && region(m.mems[1]) == s_out))
            return std::nullopt;
        region_t const mask = region(m.mems[2]), m_out = region(m.mems[0]);
        if (!(max_c(el, castable_t::add) && el.out_rank == 3 && el.join_shape == shape4 &&
              el.inns == vv{full, {2, 3}, {0, 1, 2}} && write_with_ss(el.join) == j_sum && l.mems.size() == 4 &&
              region(l.mems[1]) == s_out && region(l.mems[2]) == mask && region(l.mems[3]) == m_out))
            return std::nullopt;
        region_t const l_out = region(l.mems[0]);
        if (!(ep.out_rank == 4 && ep.join_shape == shape4 && ep.inns == vv{full, {2, 3}, {0, 1, 2}, {0, 1, 2}} &&
              write_with_ss(ep.join) == j_norm && pn.mems.size() == 5 && region(pn.mems[1]) == s_out &&
              region(pn.mems[2]) == mask && region(pn.mems[3]) == m_out && region(pn.mems[4]) == l_out))
            return std::nullopt;
        auto r_m = sole_readers(i_m, 2), r_l = sole_readers(i_l, 1);
        if (!r_m || *r_m != std::vector<int>{i_l, i_p} || !r_l || *r_l != std::vector<int>{i_p}) return std::nullopt;
        auto r_p = sole_readers(i_p, 1);
        if (!r_p) return std::nullopt;
        int const            i_o = (*r_p)[0];
        auto const&          o = nodes[i_o].op.get_apply();
        einsummable_t const& eo = o.get_einsummable();
        if (!(plain_contraction(eo) && write_with_ss(eo.join) == x16 && eo.out_rank == 4 &&
              eo.join_shape == std::vector<uint64_t>{b, h, rows, d, keys}))
            return std::nullopt;
        region_t const p_out = region(pn.mems[0]);
        int            v_slot = -1;
        bool           has_p = false;
        for (int slot = 0; slot != int(eo.inns.size()); ++slot) {
            auto const& modes = eo.inns[slot];
            if (modes == std::vector<int>{0, 1, 2, 4}) {
                if (region(o.mems[1 + slot]) != p_out) return std::nullopt;
                has_p = true;
            } else if (sorted_modes(modes) == std::vector<int>{0, 1, 3, 4} && modes.back() == 3) {
                v_slot = slot;
            }
        }
        if (v_slot < 0 || eo.inns.size() != 2 || !has_p) return std::nullopt;
        chain_t c;
        c.idx[0] = i_s, c.idx[1] = i_m, c.idx[2] = i_l, c.idx[3] = i_p, c.idx[4] = i_o;
        attention_t& a = c.node.desc;
        a.batch = uint32_t(b), a.heads = uint32_t(h), a.rows = uint32_t(rows), a.keys = uint32_t(keys), a.head_dim = uint32_t(d);
        strides(es, es.inns[q_slot], 2, a.q_stride);
        strides(es, es.inns[k_slot], 3, a.k_stride);
        strides(eo, eo.inns[v_slot], 4, a.v_stride);
        auto ost = row_major_strides({b, h, rows, d});
        for (int i = 0; i != 3; ++i) a.out_stride[i] = ost[i];
        a.mask_stride = int64_t(keys);
        c.node.loc = s.loc;
        c.node.out = o.mems[0];
        c.node.q = s.mems[1 + q_slot];
        c.node.k = s.mems[1 + k_slot];
        c.node.v = o.mems[1 + v_slot];
        c.node.mask = m.mems[2];
        return c;
    }
};

// If the f16 [rows, cols] tensor in `reg` of location `loc`, as the node at `before` reads it, is a
// lower-triangular fill -- 0 where column <= row - start, -inf elsewhere -- its start.  Looks through
// what the compilers put between the fill and its readers: copies of row blocks (touches without a
// castable) and moves of whole tensors.
inline std::optional<int64_t> lowertri_start(std::vector<memgraph_t::node_t> const& nodes, std::vector<char> const& alive,
                                             int loc, region_t reg, int before, uint64_t rows, uint64_t cols, int depth = 0)
{
    if (depth > 4 || reg.second != rows * cols * 2) return std::nullopt;
    std::vector<std::pair<uint64_t, uint64_t>> covered;
    std::optional<int64_t>                     start;
    for (int ic = before - 1; ic >= 0; --ic) {
        if (!alive[ic]) continue;
        auto const& op = nodes[ic].op;
        auto        w = written_region(op, loc);
        if (!w || !overlap(*w, reg)) continue;
        if (op.is_constant()) {
            auto const& c = op.get_constant();
            if (!covered.empty() || *w != reg || !c.fill.is_lowertri()) return std::nullopt;
            auto const& f = c.fill.get_lowertri();
            int64_t     bound = int64_t(1) << 30;
            if (f.lower.dtype != dtype_t::f16 || f.nrow != rows || f.ncol != cols || f.upper.data[0] != 0 ||
                f.upper.data[1] != 252 || f.lower.data[0] != 0 || f.lower.data[1] != 0 || f.start >= bound || f.start <= -bound)
                return std::nullopt;
            return f.start;
        }
        if (op.is_move()) {
            auto const& m = op.get_move();
            if (!covered.empty() || *w != reg) return std::nullopt;
            return lowertri_start(nodes, alive, m.get_src_loc(), {std::get<1>(m.src), m.size}, ic, rows, cols, depth + 1);
        }
        if (op.is_touch()) {
            auto const&    a = op.get_apply();
            touch_t const& t = a.get_touch();
            if (*w != reg || t.dtype != dtype_t::f16 || t.castable || t.selection.size() != 2) return std::nullopt;
            auto const &r = t.selection[0], &c = t.selection[1];
            if (r.d_out != rows || c.d_inn != cols || c.d_out != cols || c.offset_inn != 0 || c.offset_out != 0 || c.size != cols)
                return std::nullopt;
            for (auto const& [lo, hi] : covered)
                if (r.offset_out < hi && lo < r.offset_out + r.size) return std::nullopt; // an older lifetime shows through
            auto sub = lowertri_start(nodes, alive, loc, region(a.mems[1]), ic, r.d_inn, cols, depth + 1);
            if (!sub) return std::nullopt;
            int64_t here = *sub + int64_t(r.offset_out) - int64_t(r.offset_inn); // row i of the block is row i - oo + oi of the source
            if (start && *start != here) return std::nullopt;
            start = here;
            covered.push_back({r.offset_out, r.offset_out + r.size});
            uint64_t total = 0;
            for (auto const& [lo, hi] : covered) total += hi - lo;
            if (total == rows) return start;
            continue;
        }
        return std::nullopt;
    }
    return std::nullopt;
}

} // namespace detail

// `graph`: a memgraph after fold_elementwise (the patterns are those of the folded chain).
inline attention_folded_t fold_attention(memgraph_t const& graph, std::vector<memloc_t> const& saved)
{
    using namespace detail;
    attention_folded_t out{graph, {}};
    auto&              nodes = out.memgraph.nodes;
    int const          n = int(nodes.size());
    std::vector<char>  alive(n, 1);
    chain_matcher_t    matcher{nodes, alive, saved, out.attention};
    for (int i_s = 0; i_s != n; ++i_s) {
        if (!alive[i_s] || !nodes[i_s].op.is_einsummable() || out.attention.count(i_s)) continue;
        auto got = matcher.match(i_s);
        if (!got) continue;
        chain_t&          c = *got;
        attention_node_t& a = c.node;
        if (!a.desc.eligible() || a.out.offset % 16 || a.q.offset % 16 || a.k.offset % 16 || a.v.offset % 16 || a.mask.offset % 16)
            continue;
        int const      i_o = c.idx[4];
        region_t const reads[4] = {region(a.q), region(a.k), region(a.v), region(a.mask)};
        bool           bad = false;
        for (region_t const& r : reads) bad = bad || overlap(region(a.out), r);
        // Q and K are now read where the last node stands instead of the first, the mask instead of
        // where the max node stood (V is read where it always was)
        for (int ic = i_s + 1; ic < i_o && !bad; ++ic) {
            if (!alive[ic] || std::find(c.idx, c.idx + 5, ic) != c.idx + 5) continue;
            auto w = written_region(nodes[ic].op, a.loc);
            if (!w) continue;
            bad = overlap(*w, reads[0]) || overlap(*w, reads[1]) || (ic > c.idx[1] && overlap(*w, reads[3]));
        }
        if (bad) continue;
        auto tri = lowertri_start(nodes, alive, a.loc, reads[3], c.idx[1], a.desc.rows, a.desc.keys);
        if (tri) {
            a.desc.skip_known = 1;
            a.desc.skip_from = int32_t(*tri);
        }
        std::set<int> deps;
        for (int i : c.idx) deps.insert(nodes[i].inns.begin(), nodes[i].inns.end());
        for (int i : c.idx) deps.erase(i);
        memgraph_t::apply_t o = nodes[i_o].op.get_apply();
        o.mems = {a.out, a.q, a.k, a.v, a.mask};
        o.group = -1;
        nodes[i_o].op = memgraph_t::op_t(o);
        nodes[i_o].inns = deps;
        for (int ic = i_o + 1; ic != n; ++ic) {
            if (!alive[ic]) continue;
            auto w = written_region(nodes[ic].op, a.loc);
            if (!w) continue;
            bool hits = false;
            for (region_t const& r : reads) hits = hits || overlap(*w, r);
            if (hits) nodes[ic].inns.insert(i_o);
        }
        for (int k = 0; k != 4; ++k) {
            int         i = c.idx[k];
            auto const& ap = nodes[i].op.get_apply();
            mem_t       m = ap.mems[0];
            int         loc = ap.loc;
            alive[i] = 0;
            nodes[i].op = memgraph_t::op_t(memgraph_t::alloc_t{loc, m.offset, m.size});
        }
        out.attention[i_o] = a;
    }
    for (auto& node : nodes) node.outs.clear();
    for (int id = 0; id != n; ++id)
        for (int i : nodes[id].inns) nodes[i].outs.insert(id);
    return out;
}

} // namespace es_fuse
