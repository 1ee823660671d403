// The launchable units of one location of a memgraph when every location is driven by its own process
// (one process per GPU), with the units each depends on -- what a host needs to fill a program of the
// es_b200 library's executor (es_b200_program_add_*) including the exchange ops between processes:
//
//   per move between two locations: a `signal` on the source rank (stores the run number into the
//   destination's ready flag when the producers are done), on the destination rank an `await` (waits
//   for the flag) followed by a `pull` (copies the bytes over and acknowledges) or, when exactly one
//   touch reads the moved block, that touch as an `rtouch` reading the peer's memory in place, and on
//   the source rank a `wait` for the acknowledgement in front of whatever reuses the source region.
//
// The reference needs none of this: gpu_mg_server_t drives all GPUs of a box from one process and a
// move is one cudaMemcpyAsync behind a stream callback (src/engine/gpu/exec_graph.cc:406-467,
// src/engine/exec_state.cc:110-219).  Dependencies are the memgraph's own edges looked through the
// nodes that launch nothing (inputmem, inputsto, partialize, alloc, del: src/einsummable/memgraph.h:189-309);
// the touches of a partial-sum group are chained in node order, the first being the copy
// (src/engine/gpu/exec_graph.cc:167-172,368-378).  make_units gives the units in memgraph order, which
// all ranks share: along it every dependency, also across ranks, points forward, so one in-order lane
// for the ops that wait for a peer cannot dead-lock.  order_units gives them in the order in which a
// simulation of all ranks served them (what the data is expected to be ready for first comes first).
//
// Header-only; include from a file that sees the reference's src/ tree (as gpu_kernel_manager.h does
// when placed in src/engine/gpu/, or with the tree's root on the include path).
#pragma once
#if __has_include("../../einsummable/memgraph.h")
#include "../../einsummable/memgraph.h"
#else
#include "src/einsummable/memgraph.h"
#endif

#include "gpu_fuse.h"

#include <algorithm>
#include <map>
#include <queue>
#include <set>
#include <sstream>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

namespace es_exchange {

// the nodes of a graph that stand for a whole attention chain (es_fuse::fold_attention), by node id;
// every function below takes it as an optional argument
using attention_map_t = std::map<int, es_fuse::attention_node_t>;

struct unit_t {
    std::string      kind;       // einsummable attention touch rtouch constant copy evict load signal await pull wait
                                 // and, with group_sum: rsum ack
    int              node = -1;  // memgraph node (compute units)
    std::vector<int> moves;      // memgraph move nodes (exchange units; rtouch: the move it consumes)
    std::vector<int> deps;       // indices of earlier units of this rank
    bool             first = true; // touch / rtouch: the group's first member runs as a copy
    std::vector<int> nodes;      // rsum: the touches it stands for (node = the first of them)
};

// incoming moves of one run share an await (and a pull) only when their sources are expected to be
// ready within this many microseconds of each other
constexpr double AWAIT_SPREAD_US = 12.0;

namespace detail {

using node_t = memgraph_t::node_t;

inline bool bookkeeping(memgraph_t::op_t const& op)
{
    return op.is_inputmem() || op.is_inputsto() || op.is_partialize() || op.is_alloc() || op.is_del();
}

inline bool cross(memgraph_t::op_t const& op)
{
    return op.is_move() && op.get_move().get_src_loc() != op.get_move().get_dst_loc();
}

// the locations a node belongs to
inline std::vector<int> sides(memgraph_t::op_t const& op)
{
    if (op.is_move()) return {op.get_move().get_src_loc(), op.get_move().get_dst_loc()};
    if (op.is_inputmem()) return {op.get_inputmem().loc};
    if (op.is_inputsto()) return {op.get_inputsto().storage_loc};
    if (op.is_constant()) return {op.get_constant().loc};
    if (op.is_apply()) return {op.get_apply().loc};
    if (op.is_copy()) return {op.get_copy().loc};
    if (op.is_evict()) return {op.get_evict().src.loc};
    if (op.is_load()) return {op.get_load().dst.loc};
    if (op.is_partialize()) return {op.get_partialize().loc};
    if (op.is_alloc()) return {op.get_alloc().loc};
    return {op.get_del().loc};
}

// latency + work (+ extra) in microseconds of a node for the readiness estimate: launch latency plus the
// algorithmic bytes / flops at round B200 rates; returned apart so that they are added in a fixed order
struct cost_t {
    double lat, work, extra;
};
inline cost_t attention_cost_us(es_fuse::attention_t const& a)
{
    double flops = 4.0 * double(a.batch) * double(a.heads) * double(a.rows) * double(a.keys) * double(a.head_dim) *
                   (a.skip_known ? 0.6 : 1.0);
    return {5.0, flops / 0.6e9, 0.0};
}

inline cost_t cost_us(memgraph_t const& mg, int id, attention_map_t const* attention = nullptr)
{
    auto const& op = mg.nodes[id].op;
    if (attention && attention->count(id)) return attention_cost_us(attention->at(id).desc);
    if (op.is_apply()) {
        auto const& a = op.get_apply();
        if (a.is_einsummable()) {
            einsummable_t const& e = a.get_einsummable();
            double nbytes = 0;
            for (auto const& m : a.mems) nbytes += double(m.size);
            std::string join = write_with_ss(e.join);
            bool contraction = e.inns.size() == 2 && e.castable && e.castable.value() == castable_t::add &&
                               e.out_rank < int(e.join_shape.size()) && join.rfind("*[hole", 0) == 0;
            if (contraction) {
                double flops = 2.0;
                for (uint64_t d : e.join_shape) flops *= double(d);
                return {5.0, std::max(flops / 1.25e9, nbytes / 5.0e6), 0.0};
            }
            return {2.5, nbytes / 5.5e6, 0.0};
        }
        return {2.5, double(a.mems[1].size) * 2 / 4.5e6, 0.0}; // a touch, as a copy
    }
    if (op.is_constant()) return {2.5, 0.5, 0.0};
    if (op.is_move()) {
        auto const& m = op.get_move();
        if (m.get_src_loc() != m.get_dst_loc()) return {6.0, double(m.size) / 0.65e6, 5.0}; // pull; signal and flag
        return {2.5, 2 * double(m.size) / 4.5e6, 0.0};
    }
    if (op.is_copy()) return {2.5, 2 * double(op.get_copy().size) / 4.5e6, 0.0};
    if (op.is_evict()) return {4.0, double(op.get_evict().src.size) / 0.05e6, 0.0};
    if (op.is_load()) return {4.0, double(op.get_load().dst.size) / 0.05e6, 0.0};
    return {0.0, 0.0, 0.0};
}

} // namespace detail

// Run number of every move node: a run is a stretch of move nodes adjacent in the memgraph's order
// (nodes that launch nothing aside) that do not depend on one another.  A function of the graph alone.
inline std::map<int, int> move_runs(memgraph_t const& mg)
{
    using namespace detail;
    std::vector<std::set<int>> moved_from(mg.nodes.size());
    std::map<int, int>         runs;
    std::set<int>              members;
    int                        run_id = 0;
    for (int id = 0; id != int(mg.nodes.size()); ++id) {
        auto const&   node = mg.nodes[id];
        std::set<int> acc;
        for (int i : node.inns) {
            auto const& dep = mg.nodes[i].op;
            if (dep.is_move()) acc.insert(i);
            else if (bookkeeping(dep)) acc.insert(moved_from[i].begin(), moved_from[i].end());
        }
        moved_from[id] = acc;
        if (bookkeeping(node.op)) continue;
        bool hits = false;
        for (int m : acc) hits = hits || members.count(m);
        if (!node.op.is_move() || hits) {
            ++run_id;
            members.clear();
        }
        if (node.op.is_move()) {
            members.insert(id);
            runs[id] = run_id;
        }
    }
    return runs;
}

// Earliest finish time of every node if nothing ever waited for a free GPU or link.
inline std::vector<double> node_levels(memgraph_t const& mg, attention_map_t const* attention = nullptr)
{
    using namespace detail;
    std::vector<double> level(mg.nodes.size(), 0.0);
    for (int id = 0; id != int(mg.nodes.size()); ++id) {
        double start = 0.0;
        for (int i : mg.nodes[id].inns) start = std::max(start, level[i]);
        if (bookkeeping(mg.nodes[id].op)) {
            level[id] = start;
        } else {
            cost_t c = cost_us(mg, id, attention);
            level[id] = start + c.lat + c.work + c.extra;
        }
    }
    return level;
}

// group_sum: the remote adds of a partial-sum group -- whole dense blocks that arrive from several peers and
// are added into the same tensor one after the other -- become ONE unit `rsum` (an elementwise kernel
// out = out + r1 + ... + rk over the peers' memory) followed by an `ack` unit that acknowledges the k moves,
// instead of k dependent remote touches.
inline std::vector<unit_t> make_units(memgraph_t const& mg, int rank, attention_map_t const* attention = nullptr,
                                      bool group_sum = false)
{
    using namespace detail;
    int const                  n = int(mg.nodes.size());
    std::map<int, int>         runs = move_runs(mg);
    std::map<int, std::vector<int>> run_members;
    for (auto const& [id, r] : runs) run_members[r].push_back(id);
    std::vector<double> levels = node_levels(mg, attention);
    auto ready_level = [&](int m) {
        double v = 0.0;
        for (int i : mg.nodes[m].inns) v = std::max(v, levels[i]);
        return v;
    };
    // real nodes a bookkeeping node stands for
    std::vector<std::set<int>> closure(n);
    for (int id = 0; id != n; ++id) {
        if (!bookkeeping(mg.nodes[id].op)) continue;
        for (int i : mg.nodes[id].inns) {
            if (bookkeeping(mg.nodes[i].op)) closure[id].insert(closure[i].begin(), closure[i].end());
            else closure[id].insert(i);
        }
    }
    // incoming moves read by exactly one touch: the touch reads them in place
    std::map<int, int> remote_touch, touch_move;
    {
        std::map<int, std::vector<int>> users;
        for (int id = 0; id != n; ++id) {
            if (bookkeeping(mg.nodes[id].op)) continue;
            for (int i : mg.nodes[id].inns)
                if (cross(mg.nodes[i].op)) users[i].push_back(id);
        }
        for (auto const& [m, us] : users) {
            auto const& mv = mg.nodes[m].op.get_move();
            if (us.size() != 1 || mv.get_dst_loc() != rank) continue;
            auto const& t = mg.nodes[us[0]].op;
            if (!t.is_apply() || !t.get_apply().is_touch() || t.get_apply().loc != mv.get_dst_loc()) continue;
            auto const& a = t.get_apply();
            if (a.mems[1].offset != std::get<1>(mv.dst) || a.mems[1].size != mv.size) continue;
            int n_cross = 0;
            for (int i : mg.nodes[us[0]].inns) n_cross += cross(mg.nodes[i].op) ? 1 : 0;
            if (n_cross != 1) continue;
            remote_touch[m] = us[0];
            touch_move[us[0]] = m;
        }
    }
    // group_sum: fused_tail[touch] = (group, the touches summed together); never the group's first member
    // (that one is the copy); the others commute, so the remote ones may be added where the last of them stands
    std::map<int, std::pair<int, std::vector<int>>> fused_tail;
    std::map<int, std::set<int>>                    pending_tail;
    if (group_sum) {
        std::map<int, std::vector<int>> members_of;
        for (int id = 0; id != n; ++id) {
            auto const& op = mg.nodes[id].op;
            if (op.is_touch() && op.get_apply().group >= 0 && op.get_apply().loc == rank)
                members_of[op.get_apply().group].push_back(id);
        }
        auto dense_add = [&](int tid) {
            touch_t const& t = mg.nodes[tid].op.get_apply().get_touch();
            if (!touch_move.count(tid) || !t.castable || t.castable.value() != castable_t::add) return false;
            if (t.dtype != dtype_t::f16 && t.dtype != dtype_t::f32) return false;
            for (auto const& d : t.selection)
                if (d.d_inn != d.d_out || d.d_inn != d.size || d.offset_inn != 0 || d.offset_out != 0) return false;
            return true;
        };
        for (auto const& [group, ms] : members_of) {
            std::vector<int> tail;
            for (size_t i = 1; i < ms.size(); ++i)
                if (dense_add(ms[i])) tail.push_back(ms[i]);
            if (tail.size() >= 2 && tail.size() <= 7)
                for (int tid : tail) fused_tail[tid] = {group, tail};
        }
    }
    std::vector<unit_t> units;
    std::map<int, int>  unit_of, signal_of, waited, group_last;
    auto raw_deps = [&](int id, int side) { // side < 0: all
        std::set<int> acc;
        for (int i : mg.nodes[id].inns) {
            auto const& dep = mg.nodes[i].op;
            if (side >= 0) {
                std::vector<int> s = sides(dep);
                if (std::find(s.begin(), s.end(), side) == s.end()) continue;
            }
            if (bookkeeping(dep)) acc.insert(closure[i].begin(), closure[i].end());
            else acc.insert(i);
        }
        return acc;
    };
    auto resolve = [&](std::set<int> const& raw) {
        std::set<int>    deps;
        std::vector<int> tokens;
        for (int r : raw) {
            auto const& dep = mg.nodes[r].op;
            if (cross(dep)) {
                auto const& mv = dep.get_move();
                if (mv.get_dst_loc() == rank) {
                    deps.insert(unit_of.at(r));
                } else if (mv.get_src_loc() == rank) {
                    auto it = waited.find(r);
                    if (it != waited.end()) deps.insert(it->second);
                    else tokens.push_back(r);
                }
            } else {
                auto it = unit_of.find(r);
                if (it != unit_of.end()) deps.insert(it->second);
            }
        }
        if (!tokens.empty()) {
            unit_t        w;
            std::set<int> sig;
            for (int t : tokens) {
                auto it = signal_of.find(t);
                if (it != signal_of.end()) sig.insert(it->second);
            }
            w.kind = "wait";
            w.moves = tokens;
            w.deps.assign(sig.begin(), sig.end());
            units.push_back(w);
            for (int t : tokens) waited[t] = int(units.size()) - 1;
            deps.insert(int(units.size()) - 1);
        }
        return std::vector<int>(deps.begin(), deps.end());
    };
    auto emit = [&](unit_t u) {
        units.push_back(std::move(u));
        return int(units.size()) - 1;
    };
    for (int id = 0; id != n; ++id) {
        auto const& op = mg.nodes[id].op;
        if (bookkeeping(op)) continue;
        if (cross(op)) {
            auto const&             mv = op.get_move();
            std::vector<int> const& run = run_members[runs.at(id)];
            if (mv.get_dst_loc() == rank && !unit_of.count(id)) {
                std::vector<int> all;
                for (int m : run)
                    if (cross(mg.nodes[m].op) && mg.nodes[m].op.get_move().get_dst_loc() == rank) all.push_back(m);
                std::stable_sort(all.begin(), all.end(), [&](int a, int b) {
                    double la = ready_level(a), lb = ready_level(b);
                    return la < lb || (la == lb && a < b);
                });
                std::vector<std::vector<int>> clusters(1, std::vector<int>(1, all[0]));
                for (size_t k = 1; k < all.size(); ++k) {
                    if (ready_level(all[k]) - ready_level(clusters.back()[0]) > AWAIT_SPREAD_US) clusters.emplace_back();
                    clusters.back().push_back(all[k]);
                }
                for (auto members : clusters) {
                    std::sort(members.begin(), members.end());
                    unit_t aw;
                    aw.kind = "await";
                    aw.moves = members;
                    int const        ai = emit(aw);
                    std::vector<int> copied;
                    for (int m : members) {
                        unit_of[m] = ai;
                        if (!remote_touch.count(m)) copied.push_back(m);
                    }
                    if (!copied.empty()) {
                        std::set<int> raw;
                        for (int m : copied) {
                            std::set<int> r = raw_deps(m, rank);
                            raw.insert(r.begin(), r.end());
                        }
                        std::vector<int> deps = resolve(raw);
                        deps.push_back(ai);
                        std::sort(deps.begin(), deps.end());
                        deps.erase(std::unique(deps.begin(), deps.end()), deps.end());
                        unit_t pl;
                        pl.kind = "pull";
                        pl.moves = copied;
                        pl.deps = deps;
                        int const pi = emit(pl);
                        for (int m : copied) unit_of[m] = pi;
                    }
                }
            }
            if (mv.get_src_loc() == rank && !signal_of.count(id)) {
                // outgoing members of the run with the same producers share a signal; groups in the
                // order of their (sorted) dependency lists' first appearance
                std::vector<std::pair<std::vector<int>, std::vector<int>>> by_deps;
                for (int m : run) {
                    if (!cross(mg.nodes[m].op) || mg.nodes[m].op.get_move().get_src_loc() != rank) continue;
                    std::vector<int> deps = resolve(raw_deps(m, rank));
                    auto it = std::find_if(by_deps.begin(), by_deps.end(), [&](auto const& g) { return g.first == deps; });
                    if (it == by_deps.end()) by_deps.push_back({deps, {m}});
                    else it->second.push_back(m);
                }
                for (auto const& [deps, ms] : by_deps) {
                    unit_t sg;
                    sg.kind = "signal";
                    sg.moves = ms;
                    sg.deps = deps;
                    int const si = emit(sg);
                    for (int m : ms) signal_of[m] = si;
                }
            }
            continue;
        }
        std::vector<int> s = sides(op);
        if (op.is_move()) {
            if (s[0] != rank || s[1] != rank) continue;
        } else if (s[0] != rank) {
            continue;
        }
        std::vector<int> deps = resolve(raw_deps(id, -1));
        unit_t           u;
        u.node = id;
        if (op.is_apply() && op.get_apply().is_touch()) {
            int const group = op.get_apply().group;
            if (group >= 0) {
                auto it = group_last.find(group);
                u.first = it == group_last.end();
                if (!u.first) {
                    deps.push_back(it->second);
                    std::sort(deps.begin(), deps.end());
                    deps.erase(std::unique(deps.begin(), deps.end()), deps.end());
                }
            }
            auto ft = fused_tail.find(id);
            if (ft != fused_tail.end()) {
                auto const& [key, tail] = ft->second;
                std::set<int>& acc = pending_tail[key];
                acc.insert(deps.begin(), deps.end());
                if (id != tail.back()) continue; // emitted with the last member of the tail
                unit_t r;
                r.kind = "rsum";
                r.nodes = tail;
                r.node = tail[0];
                for (int t : tail) r.moves.push_back(touch_move.at(t));
                r.deps.assign(acc.begin(), acc.end());
                int const ri = emit(r);
                for (int t : tail) unit_of[t] = ri;
                unit_t a;
                a.kind = "ack";
                a.moves = r.moves;
                a.deps = {ri};
                emit(a);
                group_last[key] = ri;
                continue;
            }
            auto tm = touch_move.find(id);
            if (tm != touch_move.end()) {
                u.kind = "rtouch";
                u.moves = {tm->second};
            } else {
                u.kind = "touch";
            }
            u.deps = deps;
            int const ui = emit(u);
            if (group >= 0) group_last[group] = ui;
            unit_of[id] = ui;
            continue;
        }
        if (op.is_apply()) u.kind = (attention && attention->count(id)) ? "attention" : "einsummable";
        else if (op.is_constant()) u.kind = "constant";
        else if (op.is_move() || op.is_copy()) u.kind = "copy";
        else if (op.is_evict()) u.kind = "evict";
        else if (op.is_load()) u.kind = "load";
        else throw std::runtime_error("es_exchange::make_units: unknown memgraph node kind");
        u.deps = deps;
        unit_of[id] = emit(u);
    }
    // sources nobody on this rank reused: the run ends by collecting their acknowledgements
    std::vector<int> rest;
    std::set<int>    sig;
    for (int id = 0; id != n; ++id) {
        if (cross(mg.nodes[id].op) && mg.nodes[id].op.get_move().get_src_loc() == rank && !waited.count(id)) {
            rest.push_back(id);
            auto it = signal_of.find(id);
            if (it != signal_of.end()) sig.insert(it->second);
        }
    }
    if (!rest.empty()) {
        unit_t w;
        w.kind = "wait";
        w.moves = rest;
        w.deps.assign(sig.begin(), sig.end());
        units.push_back(w);
    }
    return units;
}

// ---- the order of a rank's units: by simulated service --------------------------------------------------
//
// make_units gives memgraph order.  That order is valid but serves the exchange ops, which share one
// in-order lane, by node number instead of by when their data is expected.  order_units simulates all
// ranks under a simple machine model (each rank's GPU, incoming link and PCIe link do one unit's work at
// a time; launch latencies overlap; a flag takes about 2 us to cross NVLink) and returns the rank's
// units in the order in which the simulation served them, dependencies renumbered.  Every rank
// simulates all ranks and gets the same answer, and along every dependency, also across ranks, the
// place in the order of service increases, so the reordered lanes cannot dead-lock either.

namespace detail {

enum server_t { SERVER_NONE = 0, SERVER_GPU = 1, SERVER_LINK = 2, SERVER_PCIE = 3 };

struct unit_cost_t {
    double lat, work;
    int    server;
};

inline unit_cost_t unit_cost_us(memgraph_t const& mg, unit_t const& u, attention_map_t const* attention = nullptr)
{
    std::string const& k = u.kind;
    if (k == "attention") {
        cost_t c = attention_cost_us(attention->at(u.node).desc);
        return {c.lat, c.work, SERVER_GPU};
    }
    if (k == "einsummable") {
        cost_t c = cost_us(mg, u.node);
        return {c.lat, c.work, SERVER_GPU};
    }
    if (k == "touch") {
        double bytes = double(mg.nodes[u.node].op.get_apply().mems[1].size * uint64_t(u.first ? 2 : 3));
        return {2.5, bytes / 4.5e6, SERVER_GPU};
    }
    if (k == "rtouch") return {6.0, double(mg.nodes[u.node].op.get_apply().mems[1].size) / 0.65e6, SERVER_LINK};
    if (k == "rsum") {
        uint64_t size = 0;
        for (int t : u.nodes) size += mg.nodes[t].op.get_apply().mems[1].size;
        return {6.0, double(size) / 0.65e6, SERVER_LINK};
    }
    if (k == "await" || k == "signal" || k == "ack") return {3.0, 0.0, SERVER_NONE};
    if (k == "constant") return {2.5, 0.5, SERVER_GPU};
    if (k == "copy") {
        auto const& op = mg.nodes[u.node].op;
        uint64_t    size = op.is_move() ? op.get_move().size : op.get_copy().size;
        return {2.5, double(2 * size) / 4.5e6, SERVER_GPU};
    }
    if (k == "evict") return {4.0, double(mg.nodes[u.node].op.get_evict().src.size) / 0.05e6, SERVER_PCIE};
    if (k == "load") return {4.0, double(mg.nodes[u.node].op.get_load().dst.size) / 0.05e6, SERVER_PCIE};
    if (k == "pull") {
        uint64_t size = 0;
        for (int m : u.moves) size += mg.nodes[m].op.get_move().size;
        return {6.0, double(size) / 0.65e6, SERVER_LINK};
    }
    if (k == "wait") return {2.0, 0.0, SERVER_NONE};
    throw std::runtime_error("es_exchange: no cost for a unit of kind " + k);
}

} // namespace detail

struct service_t {
    double ready = 0.0, finish = 0.0;
    int    place = -1; // in the order of service over all ranks
};

// Ready time, finish time and place in the order of service of every unit of every rank.
inline std::vector<std::vector<service_t>> simulate(memgraph_t const& mg, std::vector<std::vector<unit_t>> const& units_by_rank,
                                                    attention_map_t const* attention = nullptr)
{
    using namespace detail;
    using key_t = std::pair<int, int>; // rank, index
    int const                        world = int(units_by_rank.size());
    std::map<int, key_t>             sig_of, pull_of;
    for (int r = 0; r != world; ++r) {
        for (int i = 0; i != int(units_by_rank[r].size()); ++i) {
            unit_t const& u = units_by_rank[r][i];
            if (u.kind == "signal") {
                for (int m : u.moves) sig_of[m] = {r, i};
            } else if (u.kind == "pull" || u.kind == "rtouch" || u.kind == "ack") {
                for (int m : u.moves) pull_of[m] = {r, i};
            }
        }
    }
    std::vector<std::vector<std::vector<key_t>>> preds(world), succs(world);
    std::vector<std::vector<unit_cost_t>>        cost(world);
    size_t                                       total = 0;
    for (int r = 0; r != world; ++r) {
        preds[r].resize(units_by_rank[r].size());
        succs[r].resize(units_by_rank[r].size());
        cost[r].resize(units_by_rank[r].size());
        total += units_by_rank[r].size();
    }
    for (int r = 0; r != world; ++r) {
        for (int i = 0; i != int(units_by_rank[r].size()); ++i) {
            unit_t const& u = units_by_rank[r][i];
            auto&         p = preds[r][i];
            for (int d : u.deps) p.push_back({r, d});
            if (u.kind == "await") {
                for (int m : u.moves) p.push_back(sig_of.at(m));
            } else if (u.kind == "wait") {
                for (int m : u.moves) p.push_back(pull_of.at(m));
            }
            cost[r][i] = unit_cost_us(mg, u, attention);
        }
    }
    for (int r = 0; r != world; ++r)
        for (int i = 0; i != int(preds[r].size()); ++i)
            for (key_t q : preds[r][i]) succs[q.first][q.second].push_back({r, i});
    // the bottom level of a unit: its own time plus the longest chain of work that hangs on it; among
    // units that become ready at the same moment the one with the largest goes first
    std::vector<std::vector<int>> left(world);
    std::vector<key_t>            order, stack;
    for (int r = 0; r != world; ++r) {
        left[r].resize(preds[r].size());
        for (int i = 0; i != int(preds[r].size()); ++i) {
            left[r][i] = int(preds[r][i].size());
            if (left[r][i] == 0) stack.push_back({r, i});
        }
    }
    while (!stack.empty()) {
        key_t k = stack.back();
        stack.pop_back();
        order.push_back(k);
        for (key_t c : succs[k.first][k.second])
            if (--left[c.first][c.second] == 0) stack.push_back(c);
    }
    if (order.size() != total) throw std::runtime_error("es_exchange: the units of the ranks wait for one another in a cycle");
    std::vector<std::vector<double>> bottom(world);
    for (int r = 0; r != world; ++r) bottom[r].assign(preds[r].size(), 0.0);
    for (auto it = order.rbegin(); it != order.rend(); ++it) {
        double below = 0.0;
        for (key_t c : succs[it->first][it->second]) below = std::max(below, bottom[c.first][c.second]);
        unit_cost_t const& c = cost[it->first][it->second];
        bottom[it->first][it->second] = c.lat + c.work + below;
    }
    // first come first served; ties by bottom level, then by rank and index
    using item_t = std::tuple<double, double, int, int>;
    std::priority_queue<item_t, std::vector<item_t>, std::greater<item_t>> heap;
    std::vector<std::vector<service_t>>                                    times(world);
    std::vector<std::vector<double>>                                       ready_at(world);
    for (int r = 0; r != world; ++r) {
        times[r].resize(preds[r].size());
        ready_at[r].assign(preds[r].size(), 0.0);
        for (int i = 0; i != int(preds[r].size()); ++i) {
            left[r][i] = int(preds[r][i].size());
            if (left[r][i] == 0) heap.push({0.0, -bottom[r][i], r, i});
        }
    }
    std::map<std::pair<int, int>, double> free_at; // (rank, server) -> when its current work ends
    int                                   served = 0;
    while (!heap.empty()) {
        auto [t, nb, r, i] = heap.top();
        (void)nb;
        heap.pop();
        unit_cost_t const& c = cost[r][i];
        double             begin = t + c.lat;
        if (c.server != SERVER_NONE && c.work > 0) {
            auto it = free_at.find({r, c.server});
            if (it != free_at.end()) begin = std::max(begin, it->second);
            free_at[{r, c.server}] = begin + c.work;
        }
        double fin = begin + c.work;
        times[r][i].ready = t;
        times[r][i].finish = fin;
        times[r][i].place = served++;
        for (key_t s : succs[r][i]) {
            double& ra = ready_at[s.first][s.second];
            ra = std::max(ra, fin + (s.first != r ? 2.0 : 0.0));
            if (--left[s.first][s.second] == 0) heap.push({ra, -bottom[s.first][s.second], s.first, s.second});
        }
    }
    return times;
}

// The units of `rank` in the order of simulated service (the closing wait stays last), dependencies
// renumbered; `service`, when given, receives each returned unit's simulated ready and finish time.
inline std::vector<unit_t> order_units(memgraph_t const& mg, int world, int rank, std::vector<service_t>* service = nullptr,
                                       attention_map_t const* attention = nullptr, bool group_sum = false)
{
    std::vector<std::vector<unit_t>> all;
    for (int r = 0; r != world; ++r) all.push_back(make_units(mg, r, attention, group_sum));
    auto                       times = simulate(mg, all, attention);
    std::vector<unit_t> const& units = all[rank];
    int const                  n = int(units.size());
    int const                  closing = (n && units[n - 1].kind == "wait") ? n - 1 : -1;
    std::vector<int>           order(n);
    for (int i = 0; i != n; ++i) order[i] = i;
    std::sort(order.begin(), order.end(), [&](int a, int b) {
        if ((a == closing) != (b == closing)) return b == closing;
        return times[rank][a].place < times[rank][b].place;
    });
    std::vector<int> new_index(n);
    for (int i = 0; i != n; ++i) new_index[order[i]] = i;
    std::vector<unit_t> out;
    if (service) service->clear();
    for (int old : order) {
        unit_t u = units[old];
        for (int& d : u.deps) d = new_index[d];
        std::sort(u.deps.begin(), u.deps.end());
        for (int d : u.deps)
            if (d >= int(out.size())) throw std::runtime_error("es_exchange: the simulated order breaks a dependency");
        out.push_back(u);
        if (service) service->push_back(times[rank][old]);
    }
    return out;
}

// The units as JSON, for comparing plans across implementations.
inline std::string units_json(std::vector<unit_t> const& units)
{
    std::ostringstream out;
    auto vec = [&](std::vector<int> const& v) {
        out << "[";
        for (size_t i = 0; i != v.size(); ++i) out << (i ? "," : "") << v[i];
        out << "]";
    };
    out << "[";
    for (size_t i = 0; i != units.size(); ++i) {
        auto const& u = units[i];
        out << (i ? "," : "") << "{\"kind\":\"" << u.kind << "\",\"node\":" << u.node << ",\"first\":" << (u.first ? "true" : "false")
            << ",\"moves\":";
        vec(u.moves);
        out << ",\"deps\":";
        vec(u.deps);
        out << ",\"nodes\":";
        vec(u.nodes);
        out << "}";
    }
    out << "]";
    return out.str();
}

} // namespace es_exchange
