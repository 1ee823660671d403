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
//   * the folded node has at most 8 inputs (ES_B200_MAX_INNS).
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

} // namespace es_fuse
