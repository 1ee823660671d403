// Test infrastructure, not product code.
//
// Produces the reference's own partitioned graphs for the graph-level configs and
// runs the reference's own memgraph interpreter on them:
//   * config 1: build_matmul_even_splits (exps/GPU_correctness.cc:207-223) +
//     alocate01 (src/autoplace/alocate.h:20-23)
//   * configs 4: builder_t::make_first_token (llama/builder.cc:3-77) +
//     autoplace01(make_default01) (src/autoplace/autoplace.h:40-66)
//   * config 5: transformer_t forward, the log-softmax loss and graph_writer_t::backprop as
//     llama/gpu_train.cc:154-322 builds them (without LoRA), plus the vanilla update
//     w - lr * g of src/misc/update.cc:13-30 with the learning rate as a constant
//   then taskgraph_t::make (src/einsummable/taskgraph.h:15-19) and
//   memgraph_t::make_without_evict with gpu_alignment_settings
//   (src/einsummable/memgraph.h:117-147).
// ref_graph_write_json dumps the memgraph (every node with its dependencies,
// offsets, einsummable / touch / fill payload and group) plus where each block of
// every input and saved tensor lives; ref_graph_run interprets the memgraph on
// caller buffers with the reference's own per-op functions (see there).  The JSON
// files are the fixtures the product's memgraph runner is tested and benchmarked on.
#include "src/einsummable/reference.h"
#include "src/einsummable/memgraph.h"
#include "src/einsummable/taskgraph.h"
#include "src/autoplace/autoplace.h"
#include "src/autoplace/alocate.h"
#include "llama/builder.h"
#include "llama/modules.h"
#include "src/misc/update.h"

#include <fstream>

#include "../einsummable_b200/host/gpu_exchange_plan.h"
#include "../einsummable_b200/host/gpu_fuse.h"

namespace {

struct built_graph_t {
    graph_t                  graph;
    vector<placement_t>      placements;
    map<int, vtensor_t<int>> inn_tids, save_tids;
    taskgraph_t              taskgraph;
    map<int, mem_t>          inn_mem, save_mem;
    memgraph_t               memgraph;
    // with storage (evict / load): where every input / saved block lives, memory or storage
    bool                       has_storage = false;
    map<int, memstoloc_t>      inn_msl, save_msl;
    vector<map<int, buffer_t>> sto;   // storage contents around ref_graph_run_storage
    map<int, string>         names; // graph id -> name (weights etc.)
    map<string, scalar_t>    vars;  // scalar variables of the updater, substituted where a node is used
    // after ref_graph_fold_attention: the nodes that stand for a whole attention chain
    std::map<int, es_fuse::attention_node_t> attention;
    // hand-made graphs (ref_graph_build_fold_case): regions to treat as saved results
    std::vector<memloc_t> extra_saved;
};

vector<built_graph_t*> g_graphs;
thread_local string    g_gerr;

int finish(built_graph_t* b)
{
    auto [inn_tids, save_tids, tg] = taskgraph_t::make(b->graph, b->placements);
    b->inn_tids = inn_tids;
    b->save_tids = save_tids;
    b->taskgraph = tg;
    auto [inn_mem, save_mem, mg] =
        memgraph_t::make_without_evict(b->taskgraph, {}, allocator_settings_t::gpu_alignment_settings());
    b->inn_mem = inn_mem;
    b->save_mem = save_mem;
    b->memgraph = mg;
    g_graphs.push_back(b);
    return int(g_graphs.size()) - 1;
}

// The same with a memory limit per location: memgraph_t::make (src/einsummable/memgraph.h:158-164)
// evicts to and loads from one storage per location when the tensors do not fit
// (as exps/reference.cc:89-211 test_make_memgraph_with_evict sets it up).
int finish_with_storage(built_graph_t* b, uint64_t mem_limit)
{
    auto [inn_tids, save_tids, tg] = taskgraph_t::make(b->graph, b->placements);
    b->inn_tids = inn_tids;
    b->save_tids = save_tids;
    b->taskgraph = tg;
    int              nlocs = tg.num_locs();
    vector<int>      which_storage(nlocs);
    vector<uint64_t> mem_sizes(nlocs, mem_limit);
    std::iota(which_storage.begin(), which_storage.end(), 0);
    auto [inn_msl, save_msl, mg] = memgraph_t::make(b->taskgraph, which_storage, mem_sizes, {},
                                                    allocator_settings_t::gpu_alignment_settings());
    b->has_storage = true;
    b->inn_msl = inn_msl;
    b->save_msl = save_msl;
    b->memgraph = mg;
    b->sto.resize(nlocs);
    g_graphs.push_back(b);
    return int(g_graphs.size()) - 1;
}

string jstr(string const& s)
{
    string o = "\"";
    for (char c : s) {
        if (c == '"' || c == '\\') {
            o.push_back('\\');
        }
        o.push_back(c);
    }
    return o + "\"";
}

template <typename T> string jvec(vector<T> const& v)
{
    std::stringstream ss;
    ss << "[";
    for (size_t i = 0; i != v.size(); ++i) {
        ss << (i ? "," : "") << v[i];
    }
    ss << "]";
    return ss.str();
}

string castable_json(optional<castable_t> const& c)
{
    if (!c) {
        return "null";
    }
    switch (c.value()) {
        case castable_t::add: return "\"add\"";
        case castable_t::mul: return "\"mul\"";
        case castable_t::min: return "\"min\"";
        case castable_t::max: return "\"max\"";
    }
    return "null";
}

string scalar_json(scalar_t const& s)
{
    // the 8 raw payload bytes as an integer list (exact for every dtype, incl. -inf)
    vector<int> b(8, 0);
    for (int i = 0; i != int(dtype_size(s.dtype)); ++i) {
        b[i] = s.data[i]; // bytes past the dtype's size are not part of the value
    }
    // "text": the form the protobuf messages carry (fill_t::to_proto, src/einsummable/fill.cc:97-118)
    return "{\"dtype\":" + jstr(write_with_ss(s.dtype)) + ",\"raw\":" + jvec(b) + ",\"text\":" + jstr(write_with_ss(s)) + "}";
}

void tensor_json(std::ostream& out, built_graph_t const& b, int gid, vtensor_t<int> const& tids,
                 map<int, mem_t> const& mems)
{
    auto const& node = b.graph.nodes[gid];
    auto const& part = b.placements[gid].partition;
    out << "{\"gid\":" << gid << ",\"dtype\":" << jstr(write_with_ss(node.op.out_dtype()))
        << ",\"shape\":" << jvec(node.op.out_shape()) << ",\"name\":"
        << jstr(b.names.count(gid) ? b.names.at(gid) : string("")) << ",\"partdims\":[";
    for (size_t d = 0; d != part.partdims.size(); ++d) {
        out << (d ? "," : "") << jvec(part.partdims[d].sizes());
    }
    out << "],\"blocks\":[";
    auto const& vec = tids.get();
    for (size_t i = 0; i != vec.size(); ++i) {
        int          tid = vec[i];
        if (b.has_storage) {
            memstoloc_t const& msl = (&mems == &b.inn_mem ? b.inn_msl : b.save_msl).at(tid);
            uint64_t           size = b.taskgraph.nodes[tid].op.out_size();
            if (msl.is_memloc()) {
                auto const& m = msl.get_memloc();
                out << (i ? "," : "") << "{\"loc\":" << m.loc << ",\"offset\":" << m.offset << ",\"size\":" << m.size << "}";
            } else {
                auto const& st = msl.get_stoloc();
                out << (i ? "," : "") << "{\"loc\":" << b.taskgraph.out_loc(tid) << ",\"sto_loc\":" << st.loc
                    << ",\"sto_id\":" << st.id << ",\"size\":" << size << "}";
            }
            continue;
        }
        mem_t const& m = mems.at(tid);
        out << (i ? "," : "") << "{\"loc\":" << b.taskgraph.out_loc(tid) << ",\"offset\":" << m.offset
            << ",\"size\":" << m.size << "}";
    }
    out << "]}";
}

} // namespace

// for oracle/ref_engine_run.cc, which hands the memgraph to the reference's own GPU engine
memgraph_t const& ref_graph_memgraph(int h)
{
    return g_graphs.at(h)->memgraph;
}

// the regions that hold the saved results of a built graph (what the fold passes must leave in place)
std::vector<memloc_t> saved_regions(built_graph_t const& b)
{
    std::vector<memloc_t> saved;
    if (b.has_storage) {
        for (auto const& [tid, msl] : b.save_msl)
            if (msl.is_memloc()) saved.push_back(msl.get_memloc());
    } else {
        for (auto const& [tid, m] : b.save_mem) saved.push_back(memloc_t{m.offset, m.size, b.taskgraph.out_loc(tid)});
    }
    saved.insert(saved.end(), b.extra_saved.begin(), b.extra_saved.end());
    return saved;
}
std::vector<memloc_t> ref_graph_saved(int h)
{
    return saved_regions(*g_graphs.at(h));
}

extern "C" {

char const* ref_graph_last_error()
{
    return g_gerr.c_str();
}

#define G_BEGIN try {
#define G_END                                                                                      \
    }                                                                                              \
    catch (std::exception const& e)                                                                \
    {                                                                                              \
        g_gerr = e.what();                                                                         \
        return -1;                                                                                 \
    }

// config 1: ij,jk->ik, n x n, every dim split n_split ways, blocks placed on nlocs locations
int ref_graph_build_c1(uint64_t n, int n_split, int nlocs, int dtype_code)
{
    G_BEGIN
    dtype_t     dtype = dtype_code == 0 ? dtype_t::f16 : dtype_t::f32;
    partdim_t   pd = partdim_t::split(n, n_split);
    partition_t part2({pd, pd});
    partition_t part3({pd, pd, pd});
    graph_constructor_t g;
    int lhs = g.insert_input(part2, dtype);
    int rhs = g.insert_input(part2, dtype);
    int join = g.insert_einsummable(part3, einsummable_t::from_matmul(n, n, n, dtype), {lhs, rhs});
    int out = g.insert_formation(part2, join, true);
    auto* b = new built_graph_t();
    b->graph = g.graph;
    vector<partition_t> parts = vector_from_each_member(g.get_placements(), partition_t, partition);
    b->placements = alocate01(b->graph, parts, nlocs, 100);
    b->names[lhs] = "lhs";
    b->names[rhs] = "rhs";
    b->names[out] = "out";
    return finish(b);
    G_END
}

// config 4: one (or more) LLaMA transformer layers, first-token graph
int ref_graph_build_llama(uint64_t dim,
                          uint64_t n_heads,
                          uint64_t multiple_of,
                          uint64_t vocab_size,
                          int      n_layers,
                          uint64_t batch,
                          uint64_t seqlen,
                          int      nlocs,
                          int      dtype_code)
{
    G_BEGIN
    set_default_dtype(dtype_code == 0 ? dtype_t::f16 : dtype_t::f32);
    model_args_t args = model_args_t::llama_7B(batch);
    args.dim = dim;
    args.n_heads = n_heads;
    args.multiple_of = multiple_of;
    args.vocab_size = vocab_size;
    args.n_layers = n_layers;
    args.max_seq_len = seqlen; // unused freqs_cis blocks would make memgraph_t::make_ throw
    builder_t builder = builder_t::make_first_token(args, seqlen);
    auto*     b = new built_graph_t();
    b->graph = builder.graph;
    b->placements = autoplace01(b->graph, autoplace_config_t::make_default01(nlocs, 1));
    for (auto const& [name, gid] : builder.weights) {
        b->names[gid] = name;
    }
    b->names[builder.freqs_cis] = "freqs_cis";
    b->names[builder.embeddings] = "embeddings";
    if (builder.mask) {
        b->names[builder.mask.value()] = "mask";
    }
    b->names[builder.scores] = "scores";
    return finish(b);
    G_END
}

// config 4 with the autoplacer's knobs exposed (autoplace_config_t, src/autoplace/autoplace.h:6-66):
// flops_per_byte_moved (default 1000), search space 0 contraction / 1 all / 2 all_range (default),
// max_branching (default 2), discount_input_factor (default 1)
int ref_graph_build_llama_cfg(uint64_t dim, uint64_t n_heads, uint64_t multiple_of, uint64_t vocab_size, int n_layers,
                              uint64_t batch, uint64_t seqlen, int nlocs, int dtype_code, uint64_t fpbm, int space,
                              int branching, uint64_t discount)
{
    G_BEGIN
    set_default_dtype(dtype_code == 0 ? dtype_t::f16 : dtype_t::f32);
    model_args_t args = model_args_t::llama_7B(batch);
    args.dim = dim;
    args.n_heads = n_heads;
    args.multiple_of = multiple_of;
    args.vocab_size = vocab_size;
    args.n_layers = n_layers;
    args.max_seq_len = seqlen;
    builder_t builder = builder_t::make_first_token(args, seqlen);
    auto*     b = new built_graph_t();
    b->graph = builder.graph;
    parts_space_t sp = space == 0 ? parts_space_t::contraction : (space == 1 ? parts_space_t::all : parts_space_t::all_range);
    vector<partition_t> parts = apart01(b->graph, nlocs, branching, discount, sp);
    b->placements = alocate01(b->graph, parts, nlocs, fpbm);
    for (auto const& [name, gid] : builder.weights) {
        b->names[gid] = name;
    }
    b->names[builder.freqs_cis] = "freqs_cis";
    b->names[builder.embeddings] = "embeddings";
    if (builder.mask) {
        b->names[builder.mask.value()] = "mask";
    }
    b->names[builder.scores] = "scores";
    return finish(b);
    G_END
}

// Config 4's graph under a hand-written tensor-parallel placement instead of autoplace01 -- the kind of
// placement llama/first_token.cc:240-343 offers beside "auto" (its "data" / "dim" / "seq" partitioners feed
// apart03; this one needs a different split in different parts of the layer, which apart03's forward
// propagation cannot express, so every node's partition is set here):
//   * the residual stream ([batch, seq, heads, head_dim] and its row statistics) is split over the sequence;
//   * wq / wk / wv are split over their output heads, everything between them and wo (RoPE, scores,
//     softmax, P V) over heads, wo over its input heads with the partial sums added into the
//     sequence-split residual stream;
//   * w1 / w3 over the hidden dim, the SwiGLU product over the hidden dim, w2 over its hidden (contracted)
//     dim with the partial sums added into the residual stream;
//   * the vocabulary projection over the vocabulary; what is left (the last token's rows: the final norm
//     of one row per batch entry) on the last location, where those rows already are.
// Block k of the one split dim lives on location k, so every weight block is used where it lives.
// The reference's taskgraph compiler does the rest (refinement touches, moves, partial-sum groups).
int ref_graph_build_llama_tp(uint64_t dim, uint64_t n_heads, uint64_t multiple_of, uint64_t vocab_size, int n_layers,
                             uint64_t batch, uint64_t seqlen, int nlocs, int dtype_code)
{
    G_BEGIN
    set_default_dtype(dtype_code == 0 ? dtype_t::f16 : dtype_t::f32);
    model_args_t args = model_args_t::llama_7B(batch);
    args.dim = dim;
    args.n_heads = n_heads;
    args.multiple_of = multiple_of;
    args.vocab_size = vocab_size;
    args.n_layers = n_layers;
    args.max_seq_len = seqlen;
    builder_t builder = builder_t::make_first_token(args, seqlen);
    auto*     b = new built_graph_t();
    b->graph = builder.graph;
    graph_t const& graph = b->graph;
    enum region_t { NONE = 0, ROW, HEAD, HID, VOC, TAIL };
    enum role_t { R_NONE = 0, R_QKV, R_WO, R_W13, R_W2, R_VOCAB };
    map<int, role_t> weight_role;
    for (auto const& [name, gid] : builder.weights) {
        auto ends = [&](char const* suffix) {
            string sfx(suffix);
            return name.size() >= sfx.size() && name.compare(name.size() - sfx.size(), sfx.size(), sfx) == 0;
        };
        if (ends("wq.weight") || ends("wk.weight") || ends("wv.weight")) weight_role[gid] = R_QKV;
        else if (ends("wo.weight")) weight_role[gid] = R_WO;
        else if (ends("w1.weight") || ends("w3.weight")) weight_role[gid] = R_W13;
        else if (ends("w2.weight")) weight_role[gid] = R_W2;
        else if (ends("output.weight")) weight_role[gid] = R_VOCAB;
    }
    uint64_t const hidden = [&] {
        for (auto const& [name, gid] : builder.weights)
            if (weight_role.count(gid) && weight_role[gid] == R_W2) return graph.nodes[gid].op.out_shape().back();
        return uint64_t(0);
    }();
    int const n = nlocs;
    vector<region_t>          region(graph.nodes.size(), NONE);
    vector<role_t>            role(graph.nodes.size(), R_NONE);
    vector<vector<partdim_t>> pds(graph.nodes.size());
    auto singletons = [](vector<uint64_t> const& shape) {
        vector<partdim_t> ret;
        for (uint64_t d : shape) ret.push_back(partdim_t::singleton(d));
        return ret;
    };
    // the partition of a shape in a region: one dim split n ways, chosen by what the dim is
    auto split_by_region = [&](vector<uint64_t> const& shape, region_t r) {
        vector<partdim_t> ret = singletons(shape);
        int               which = -1;
        if (r == ROW) {
            if (shape.size() >= 2 && shape[0] == batch && shape[1] == seqlen) which = 1;
        } else if (r == HEAD) {
            for (int i = 0; i != int(shape.size()); ++i)
                if (shape[i] == n_heads) { which = i; break; }
        } else if (r == HID) {
            for (int i = 0; i != int(shape.size()); ++i)
                if (shape[i] == hidden) { which = i; break; }
        } else if (r == VOC) {
            for (int i = 0; i != int(shape.size()); ++i)
                if (shape[i] == vocab_size) { which = i; break; }
        }
        if (which >= 0 && shape[which] % uint64_t(n) == 0) ret[which] = partdim_t::split(shape[which], n);
        return ret;
    };
    for (int gid : graph.get_order()) {
        auto const&      node = graph.nodes[gid];
        vector<uint64_t> out_shape = node.op.out_shape();
        if (node.op.is_input()) {
            auto it = weight_role.find(gid);
            pds[gid] = singletons(out_shape);
            if (it != weight_role.end()) {
                int which = (it->second == R_QKV || it->second == R_W13 || it->second == R_VOCAB) ? 0 : 2;
                pds[gid][which] = partdim_t::split(out_shape[which], n);
            } else if (gid == builder.embeddings) {
                region[gid] = ROW;
                pds[gid] = split_by_region(out_shape, ROW);
            }
            continue;
        }
        if (node.op.is_fill()) {
            pds[gid] = singletons(out_shape);
            continue;
        }
        // what the inputs say
        region_t r = NONE;
        for (int inn : node.inns)
            if (region[inn] != NONE) r = region[inn];
        if (node.op.is_einsummable()) {
            einsummable_t const& e = node.op.get_einsummable();
            role_t               w = R_NONE;
            int                  w_slot = -1;
            for (int k = 0; k != int(node.inns.size()); ++k) {
                int  src = node.inns[k];
                auto it = weight_role.find(src);
                if (it != weight_role.end() && e.has_aggregation()) { w = it->second; w_slot = k; }
            }
            vector<partdim_t> join = singletons(e.join_shape);
            if (w != R_NONE) {
                // a projection: split the join mode that the weight's split dim maps to
                int wdim = (w == R_QKV || w == R_W13 || w == R_VOCAB) ? 0 : 2;
                int mode = e.inns[w_slot][wdim];
                join[mode] = partdim_t::split(e.join_shape[mode], n);
                role[gid] = w;
                region[gid] = w == R_QKV ? HEAD : (w == R_W13 ? HID : (w == R_VOCAB ? VOC : ROW));
            } else {
                region[gid] = r;
                // follow the first input that is split; modes it lacks stay whole
                for (int k = 0; k != int(node.inns.size()); ++k) {
                    auto const& ipd = pds[node.inns[k]];
                    bool        any = false;
                    for (int i = 0; i != int(ipd.size()); ++i)
                        if (ipd[i].num_parts() > 1) any = true;
                    if (!any || region[node.inns[k]] != r) continue;
                    for (int i = 0; i != int(ipd.size()); ++i) join[e.inns[k][i]] = ipd[i];
                    break;
                }
            }
            pds[gid] = join;
            continue;
        }
        if (node.op.is_formation()) {
            int inn = node.inns[0];
            if (role[inn] == R_WO || role[inn] == R_W2) {
                region[gid] = ROW; // the partial sums land in the sequence-split residual stream
                pds[gid] = split_by_region(out_shape, ROW);
            } else {
                region[gid] = region[inn];
                pds[gid] = vector<partdim_t>(pds[inn].begin(), pds[inn].begin() + out_shape.size());
            }
            continue;
        }
        // complexer / squeezer / select: by region and shape
        region[gid] = r;
        pds[gid] = split_by_region(out_shape, r);
        if (r == ROW && !(out_shape.size() >= 2 && out_shape[0] == batch && out_shape[1] == seqlen)) region[gid] = TAIL;
    }
    for (int gid = 0; gid != int(graph.nodes.size()); ++gid) {
        partition_t    part(pds[gid]);
        vtensor_t<int> locs(part.block_shape());
        if (part.num_parts() == n)
            for (int i = 0; i != n; ++i) locs.get()[i] = i;
        else if (part.num_parts() == 1)
            locs.get()[0] = region[gid] == TAIL ? n - 1 : 0;
        else
            throw std::runtime_error("tensor-parallel placement: node " + std::to_string(gid) + " has " +
                                     std::to_string(part.num_parts()) + " blocks");
        b->placements.emplace_back(part, locs);
    }
    for (auto const& [name, gid] : builder.weights) {
        b->names[gid] = name;
    }
    b->names[builder.freqs_cis] = "freqs_cis";
    b->names[builder.embeddings] = "embeddings";
    if (builder.mask) {
        b->names[builder.mask.value()] = "mask";
    }
    b->names[builder.scores] = "scores";
    return finish(b);
    G_END
}

// The exchange units of one rank as the C++ planner (einsummable_b200/host/gpu_exchange_plan.h) makes them
// from the built memgraph, as JSON: compared in the tests with what the Python planner makes of the
// JSON form of the same memgraph.
int ref_graph_exchange_units(int h, int rank, char const* path)
{
    G_BEGIN
    built_graph_t* b = g_graphs.at(h);
    std::ofstream  out(path);
    out << es_exchange::units_json(es_exchange::make_units(b->memgraph, rank, b->attention.empty() ? nullptr : &b->attention)) << "\n";
    return 0;
    G_END
}

// The same in the order of simulated service (es_exchange::order_units), each unit with its simulated
// ready and finish time: compared with the Python runner's order_units_by_simulation.
int ref_graph_exchange_units_ordered(int h, int rank, char const* path)
{
    G_BEGIN
    built_graph_t*                      b = g_graphs.at(h);
    std::vector<es_exchange::service_t> service;
    auto units = es_exchange::order_units(b->memgraph, b->memgraph.num_compute_locs, rank, &service,
                                          b->attention.empty() ? nullptr : &b->attention);
    std::ofstream out(path);
    out.precision(17);
    out << "{\"units\":" << es_exchange::units_json(units) << ",\"ready_us\":[";
    for (size_t i = 0; i != service.size(); ++i) out << (i ? "," : "") << service[i].ready;
    out << "],\"finish_us\":[";
    for (size_t i = 0; i != service.size(); ++i) out << (i ? "," : "") << service[i].finish;
    out << "]}\n";
    return 0;
    G_END
}

// The units of one rank, in the order of simulated service, with the remote adds of every partial-sum group
// summed by one unit (make_units' group_sum): compared with the Python planner's group_sum=True.
int ref_graph_exchange_units_group_sum(int h, int rank, char const* path)
{
    G_BEGIN
    built_graph_t*                      b = g_graphs.at(h);
    std::vector<es_exchange::service_t> service;
    auto units = es_exchange::order_units(b->memgraph, b->memgraph.num_compute_locs, rank, &service,
                                          b->attention.empty() ? nullptr : &b->attention, true);
    std::ofstream out(path);
    out << "{\"units\":" << es_exchange::units_json(units) << "}\n";
    return 0;
    G_END
}

// Hand-made one-location memgraphs around one elementwise producer A (exp, f32, 64 elements, reads region 0,
// writes region 1; regions are 256 bytes apart) and its reader B (x + y over regions 1 and 4, into region 2), for
// the conditions under which the fold must refuse:
//   0 nothing in the way (A folds into B)          1 a fill between A and B writes the memory A reads
//   2 B reads A's bytes under another shape         3 A's result is a saved result
//   4 a copy node reads A's result                  5 two readers (A folds into both)
//   6 B writes into the memory A reads              7 as 0, and a later fill into the memory A reads, which
//                                                     depended on A alone, must afterwards depend on B
int ref_graph_build_fold_case(int which)
{
    G_BEGIN
    uint64_t const n = 64, sz = n * 4;
    auto           mem = [&](int region) { return mem_t{uint64_t(region) * sz, sz}; };
    memgraph_t     mg(1, 1, vector<int>{0});
    auto           input = [&](int region) { return mg.insert(memgraph_t::op_t(memgraph_t::inputmem_t{0, region * sz, sz}), {}); };
    auto           apply = [&](einsummable_t const& e, vector<int> regions, set<int> deps) {
        vector<mem_t> mems;
        for (int r : regions) mems.push_back(mem(r));
        return mg.insert(memgraph_t::op_t(memgraph_t::apply_t{0, mems, e, -1}), deps);
    };
    auto fill = [&](int region, set<int> deps) {
        fill_t f(fill_t::constant_t{scalar_t(float(1.5)), {n}});
        return mg.insert(memgraph_t::op_t(memgraph_t::constant_t{0, region * sz, f}), deps);
    };
    einsummable_t e_exp({n}, {{0}}, 1, scalarop_t::make_exp(dtype_t::f32));
    einsummable_t e_exp2({8, 8}, {{0, 1}}, 2, scalarop_t::make_exp(dtype_t::f32));
    einsummable_t e_add({n}, {{0}, {0}}, 1, scalarop_t::make_add(dtype_t::f32));
    einsummable_t e_mul({n}, {{0}, {0}}, 1, scalarop_t::make_mul(dtype_t::f32));
    built_graph_t* b = new built_graph_t();
    int            x = input(0), y = input(4);
    int            a = apply(which == 2 ? e_exp2 : e_exp, {1, 0}, {x});
    if (which == 1) {
        int f = fill(0, {a});
        apply(e_add, {2, 1, 4}, {a, y, f});
    } else if (which == 4) {
        apply(e_add, {2, 1, 4}, {a, y});
        mg.insert(memgraph_t::op_t(memgraph_t::copy_t{0, sz, 1 * sz, 3 * sz}), {a});
    } else if (which == 5) {
        apply(e_add, {2, 1, 4}, {a, y});
        apply(e_mul, {3, 4, 1}, {a, y});
    } else if (which == 6) {
        apply(e_add, {0, 1, 4}, {a, y});
    } else if (which == 7) {
        apply(e_add, {2, 1, 4}, {a, y});
        fill(0, {a});
    } else {
        apply(e_add, {2, 1, 4}, {a, y});
    }
    if (which == 3) b->extra_saved.push_back(memloc_t{1 * sz, sz, 0});
    b->memgraph = mg;
    g_graphs.push_back(b);
    return int(g_graphs.size()) - 1;
    G_END
}

// A new handle whose memgraph is the C++ fold of handle h's (einsummable_b200/host/gpu_fuse.h): the
// folded graph is again a memgraph_t, so ref_graph_write_json / ref_graph_run / ref_graph_exchange_units
// take it like any other.  Returns the handle; *n_folded receives the number of nodes folded away.
int ref_graph_fold_elementwise(int h, int* n_folded)
{
    G_BEGIN
    built_graph_t const&  b = *g_graphs.at(h);
    std::vector<memloc_t> saved = saved_regions(b);
    es_fuse::folded_t f = es_fuse::fold_elementwise(b.memgraph, saved);
    built_graph_t*    nb = new built_graph_t(b);
    nb->memgraph = f.memgraph;
    if (n_folded) *n_folded = int(f.folded.size());
    g_graphs.push_back(nb);
    return int(g_graphs.size()) - 1;
    G_END
}

// The attention chains of handle h's memgraph (which has been through ref_graph_fold_elementwise) as the
// C++ pass finds them (es_fuse::fold_attention): a new handle whose memgraph has every chain replaced by one
// node, and, written to `path` as JSON, that node's descriptor and memories by node id.
int ref_graph_fold_attention(int h, char const* path)
{
    G_BEGIN
    built_graph_t const&  b = *g_graphs.at(h);
    std::vector<memloc_t> saved = saved_regions(b);
    es_fuse::attention_folded_t f = es_fuse::fold_attention(b.memgraph, saved);
    std::ofstream               out(path);
    auto v3 = [&](int64_t const* v) { out << "[" << v[0] << "," << v[1] << "," << v[2] << "]"; };
    auto mem = [&](mem_t const& m) { out << "[" << m.offset << "," << m.size << "]"; };
    out << "{";
    bool first = true;
    for (auto const& [id, a] : f.attention) {
        auto const& d = a.desc;
        out << (first ? "" : ",") << "\"" << id << "\":{\"loc\":" << a.loc << ",\"attention\":{\"batch\":" << d.batch
            << ",\"heads\":" << d.heads << ",\"rows\":" << d.rows << ",\"keys\":" << d.keys << ",\"head_dim\":" << d.head_dim
            << ",\"skip_known\":" << d.skip_known << ",\"skip_from\":" << d.skip_from << ",\"q_stride\":";
        v3(d.q_stride);
        out << ",\"k_stride\":";
        v3(d.k_stride);
        out << ",\"v_stride\":";
        v3(d.v_stride);
        out << ",\"out_stride\":";
        v3(d.out_stride);
        out << ",\"mask_stride\":" << d.mask_stride << "},\"mems\":[";
        mem(a.out), out << ",", mem(a.q), out << ",", mem(a.k), out << ",", mem(a.v), out << ",", mem(a.mask);
        out << "]}";
        first = false;
    }
    out << "}\n";
    built_graph_t* nb = new built_graph_t(b);
    nb->memgraph = f.memgraph;
    nb->attention = f.attention;
    g_graphs.push_back(nb);
    return int(g_graphs.size()) - 1;
    G_END
}

// config 5: forward + backward + vanilla weight update of n_layers LLaMA layers
int ref_graph_build_llama_train(uint64_t dim,
                                uint64_t n_heads,
                                uint64_t multiple_of,
                                uint64_t vocab_size,
                                int      n_layers,
                                uint64_t batch,
                                uint64_t seqlen,
                                int      nlocs,
                                int      dtype_code,
                                double   learning_rate,
                                int      save_grads,
                                int      updater,
                                int      lora_rank)
{
    G_BEGIN
    dtype_t dtype = dtype_code == 0 ? dtype_t::f16 : dtype_t::f32;
    set_default_dtype(dtype);
    model_args_t args = model_args_t::llama_7B(batch);
    args.dim = dim;
    args.n_heads = n_heads;
    args.multiple_of = multiple_of;
    args.vocab_size = vocab_size;
    args.n_layers = n_layers;
    args.max_seq_len = seqlen;
    auto* b = new built_graph_t();
    {
        graph_writer_t writer;
        // lora_rank > 0: the reference trainer's set-up (llama/gpu_train.cc:164,236-252): only the
        // low-rank adapters are trained, the base weights are inputs that are saved as they are
        transformer_t  model(&writer, args, 0, lora_rank > 0 ? optional<int>(lora_rank) : std::nullopt);
        tensor_t       embeddings = writer.input(full_shape_t(
            {full_dim_t::singleton(args.batch_size), full_dim_t::singleton(seqlen), args.full_dim()}));
        tensor_t predictions = model.forward(embeddings);
        tensor_t labels = writer.input(vector<uint64_t>{args.batch_size, args.vocab_size}, dtype);
        tensor_t loss;
        {
            tensor_t v = predictions;
            tensor_t c = writer.reduction("bv->b", castable_t::max, v);
            v = writer.ew("bv,b->bv", scalarop_t::make_sub(dtype), v, c);
            tensor_t ev = writer.ew(scalarop_t::make_exp(dtype), v);
            tensor_t evsubset = writer.contraction("bv,bv->b", ev, labels);
            tensor_t evsum = writer.reduction("bv->b", castable_t::add, ev);
            tensor_t lll = writer.ew("b,b->b", scalarop_t::make_div(dtype), evsubset, evsum);
            lll = writer.ew(scalarop_t::make_log(dtype), lll);
            loss = lll.scale(scalar_t(dtype, write_with_ss(1.0 / double(args.batch_size))));
        }
        loss.save_inplace();
        vector<tensor_t> ws;
        vector<string>   wnames;
        for (auto [name, tensor] : model.weight_map()) {
            b->names[tensor.get_id()] = name;
            if (lora_rank > 0 && name.find("lora") == string::npos) {
                continue; // a frozen base weight
            }
            ws.push_back(tensor);
            wnames.push_back(name);
        }
        vector<tensor_t> grads = writer.backprop(loss, ws);
        b->names[embeddings.get_id()] = "embeddings";
        b->names[labels.get_id()] = "labels";
        b->names[loss.get_id()] = "loss";
        b->names[model.full_freqs_cis.get_id()] = "freqs_cis";
        vector<int> weight_ids = vector_from_each_method(ws, int, get_id);
        vector<int> grad_ids = vector_from_each_method(grads, int, get_id);
        b->graph = writer.get_graph();
        if (updater == 1) {
            // the reference trainer's AdamW (src/misc/update.cc:100-189) with f32 as its minimum
            // precision, its state tensors m and v as extra inputs, and the scalar variables of
            // iteration 1 (update_vars, :74-98) substituted wherever a node is written or interpreted
            updater_desc_t          desc{dtype, updater_desc_t::adamw_t{.min_precision = dtype_t::f32}};
            vector<tuple<int, int>> old_news;
            auto inits = update_weights(desc, b->graph, old_news, weight_ids, grad_ids);
            b->vars["beta1"] = scalar_t(dtype, "0.9");
            b->vars["beta2"] = scalar_t(dtype, "0.999");
            b->vars["eta"] = scalar_t(dtype, write_with_ss(learning_rate));
            update_vars(desc, 1, b->vars);
            map<int, string> wname;
            for (size_t i = 0; i != weight_ids.size(); ++i) wname[weight_ids[i]] = wnames[i];
            int n_state = 0;
            for (auto const& [old_id, new_id] : old_news) {
                b->graph.nodes[new_id].op.set_save(true);
                if (wname.count(old_id)) {
                    b->names[new_id] = "new." + wname.at(old_id);
                } else {
                    // m and v come in pairs per weight, in the order update_weights created them
                    string which = (n_state % 2 == 0) ? "m." : "v.";
                    b->names[old_id] = which + wnames[n_state / 2];
                    b->names[new_id] = "new." + which + wnames[n_state / 2];
                    ++n_state;
                }
            }
            if (save_grads) {
                for (size_t i = 0; i != weight_ids.size(); ++i) {
                    b->graph.nodes[grad_ids[i]].op.set_save(true);
                    b->names[grad_ids[i]] = "grad." + wnames[i];
                }
            }
        } else {
        scalarop_t update = scalarop_t::combine(
            scalarop_t::make_sub(dtype),
            {scalarop_t::make_identity(dtype),
             scalarop_t::make_scale(scalar_t(dtype, write_with_ss(learning_rate)))});
        for (size_t i = 0; i != weight_ids.size(); ++i) {
            vector<uint64_t> shape = b->graph.out_shape(weight_ids[i]);
            int              rank = shape.size();
            einsummable_t    e(shape, vector<vector<int>>(2, vector_iota<int>(rank)), rank, update);
            int              id = b->graph.insert_einsummable(e, {weight_ids[i], grad_ids[i]});
            b->graph.nodes[id].op.set_save(true);
            b->names[id] = "new." + wnames[i];
            if (save_grads) {
                b->graph.nodes[grad_ids[i]].op.set_save(true);
                b->names[grad_ids[i]] = "grad." + wnames[i];
            }
        }
        }
    }
    b->placements = autoplace01(b->graph, autoplace_config_t::make_default01(nlocs, 1));
    return finish(b);
    G_END
}

// config 1 with a memory limit per location: the memgraph evicts to / loads from storage
int ref_graph_build_c1_evict(uint64_t n, int n_split, int nlocs, int dtype_code, uint64_t mem_limit)
{
    G_BEGIN
    dtype_t     dtype = dtype_code == 0 ? dtype_t::f16 : dtype_t::f32;
    partdim_t   pd = partdim_t::split(n, n_split);
    partition_t part2({pd, pd});
    partition_t part3({pd, pd, pd});
    graph_constructor_t g;
    int lhs = g.insert_input(part2, dtype);
    int rhs = g.insert_input(part2, dtype);
    int join = g.insert_einsummable(part3, einsummable_t::from_matmul(n, n, n, dtype), {lhs, rhs});
    int out = g.insert_formation(part2, join, true);
    auto* b = new built_graph_t();
    b->graph = g.graph;
    vector<partition_t> parts = vector_from_each_member(g.get_placements(), partition_t, partition);
    b->placements = alocate01(b->graph, parts, nlocs, 100);
    b->names[lhs] = "lhs";
    b->names[rhs] = "rhs";
    b->names[out] = "out";
    return finish_with_storage(b, mem_limit);
    G_END
}

// Storage contents of a graph built with a memory limit: written before, read after
// ref_graph_run_storage, which is the reference's own reference_compute_memgraph with storage
// (src/einsummable/reference.cc:191-307).
int ref_graph_sto_write(int h, int sto_loc, int sto_id, void const* data, uint64_t size)
{
    G_BEGIN
    built_graph_t& b = *g_graphs.at(h);
    buffer_t       buf = make_buffer(size);
    std::copy((uint8_t const*)data, (uint8_t const*)data + size, buf->data);
    b.sto.at(sto_loc)[sto_id] = buf;
    return 0;
    G_END
}

int ref_graph_sto_read(int h, int sto_loc, int sto_id, void* data, uint64_t size)
{
    G_BEGIN
    built_graph_t& b = *g_graphs.at(h);
    buffer_t       buf = b.sto.at(sto_loc).at(sto_id);
    if (buf->size != size) throw std::runtime_error("storage block has another size");
    std::copy(buf->data, buf->data + size, (uint8_t*)data);
    return 0;
    G_END
}

int ref_graph_run_storage(int h, void** loc_buffers)
{
    G_BEGIN
    built_graph_t&   b = *g_graphs.at(h);
    vector<buffer_t> locs;
    auto             sizes = b.memgraph.mem_sizes();
    for (size_t i = 0; i != sizes.size(); ++i) {
        locs.push_back(make_buffer_reference((uint8_t*)loc_buffers[i], sizes[i]));
    }
    reference_compute_memgraph(b.memgraph, locs, b.sto);
    return 0;
    G_END
}

int ref_graph_num_locs(int h)
{
    return g_graphs.at(h)->memgraph.num_compute_locs;
}

int ref_graph_mem_sizes(int h, uint64_t* out)
{
    G_BEGIN
    auto sizes = g_graphs.at(h)->memgraph.mem_sizes();
    for (size_t i = 0; i != sizes.size(); ++i) {
        out[i] = sizes[i];
    }
    return int(sizes.size());
    G_END
}

int ref_graph_write_json(int h, char const* path)
{
    G_BEGIN
    built_graph_t const& b = *g_graphs.at(h);
    memgraph_t const&    mg = b.memgraph;
    std::ofstream        out(path);
    out << "{\"num_locs\":" << mg.num_compute_locs << ",\"num_storage_locs\":" << mg.num_storage_locs
        << ",\"storage_locs\":" << jvec(mg.storage_locs) << ",\"mem_sizes\":" << jvec(mg.mem_sizes());
    // statistics of the taskgraph
    {
        int      n_apply = 0, n_move = 0, n_partialize = 0;
        uint64_t move_bytes = 0;
        double   flops = 0;
        for (auto const& node : b.taskgraph.nodes) {
            if (node.op.is_apply()) {
                n_apply++;
                auto const& e = node.op.get_apply().einsummable;
                if (e.is_contraction()) {
                    flops += 2.0 * double(product(e.join_shape));
                }
            } else if (node.op.is_move()) {
                n_move++;
                move_bytes += node.op.get_move().size;
            } else if (node.op.is_partialize()) {
                n_partialize++;
            }
        }
        out << ",\"taskgraph\":{\"nodes\":" << b.taskgraph.nodes.size() << ",\"apply\":" << n_apply
            << ",\"move\":" << n_move << ",\"move_bytes\":" << move_bytes
            << ",\"partialize\":" << n_partialize << ",\"contraction_flops\":" << flops << "}";
    }
    out << ",\"inputs\":[";
    {
        bool first = true;
        for (auto const& [gid, tids] : b.inn_tids) {
            out << (first ? "" : ",");
            first = false;
            tensor_json(out, b, gid, tids, b.inn_mem);
        }
    }
    out << "],\"outputs\":[";
    {
        bool first = true;
        for (auto const& [gid, tids] : b.save_tids) {
            out << (first ? "" : ",");
            first = false;
            tensor_json(out, b, gid, tids, b.save_mem);
        }
    }
    out << "],\"nodes\":[";
    for (int id = 0; id != int(mg.nodes.size()); ++id) {
        auto const& node = mg.nodes[id];
        auto const& op = node.op;
        out << (id ? "," : "") << "\n{\"id\":" << id << ",\"inns\":"
            << jvec(vector<int>(node.inns.begin(), node.inns.end()));
        if (op.is_inputmem()) {
            auto const& x = op.get_inputmem();
            out << ",\"kind\":\"inputmem\",\"loc\":" << x.loc << ",\"offset\":" << x.offset
                << ",\"size\":" << x.size;
        } else if (op.is_constant()) {
            auto const& x = op.get_constant();
            out << ",\"kind\":\"constant\",\"loc\":" << x.loc << ",\"offset\":" << x.offset;
            if (x.fill.is_constant()) {
                auto const& c = x.fill.get_constant();
                out << ",\"fill\":{\"type\":\"constant\",\"value\":" << scalar_json(c.value)
                    << ",\"nelem\":" << product(c.shape) << "}";
            } else {
                auto const& l = x.fill.get_lowertri();
                out << ",\"fill\":{\"type\":\"lowertri\",\"lower\":" << scalar_json(l.lower)
                    << ",\"upper\":" << scalar_json(l.upper) << ",\"nrow\":" << l.nrow
                    << ",\"ncol\":" << l.ncol << ",\"start\":" << l.start << "}";
            }
        } else if (op.is_apply()) {
            auto const& a = op.get_apply();
            out << ",\"kind\":\"apply\",\"loc\":" << a.loc << ",\"group\":" << a.group << ",\"mems\":[";
            for (size_t i = 0; i != a.mems.size(); ++i) {
                out << (i ? "," : "") << "[" << a.mems[i].offset << "," << a.mems[i].size << "]";
            }
            out << "]";
            if (a.is_einsummable()) {
                einsummable_t const e = a.get_einsummable().replace_scalar_variables(b.vars);
                out << ",\"einsummable\":{\"join_shape\":" << jvec(e.join_shape) << ",\"inns\":[";
                for (size_t i = 0; i != e.inns.size(); ++i) {
                    out << (i ? "," : "") << jvec(e.inns[i]);
                }
                out << "],\"out_rank\":" << e.out_rank << ",\"join\":" << jstr(write_with_ss(e.join))
                    << ",\"castable\":" << castable_json(e.castable) << "}";
            } else {
                auto const& t = a.get_touch();
                out << ",\"touch\":{\"dtype\":" << jstr(write_with_ss(t.dtype))
                    << ",\"castable\":" << castable_json(t.castable) << ",\"selection\":[";
                for (size_t i = 0; i != t.selection.size(); ++i) {
                    auto const& s = t.selection[i];
                    out << (i ? "," : "") << "[" << s.d_inn << "," << s.d_out << "," << s.offset_inn
                        << "," << s.offset_out << "," << s.size << "]";
                }
                out << "]}";
            }
        } else if (op.is_move()) {
            auto const& m = op.get_move();
            out << ",\"kind\":\"move\",\"src_loc\":" << std::get<0>(m.src)
                << ",\"src_offset\":" << std::get<1>(m.src) << ",\"dst_loc\":" << std::get<0>(m.dst)
                << ",\"dst_offset\":" << std::get<1>(m.dst) << ",\"size\":" << m.size;
        } else if (op.is_copy()) {
            auto const& c = op.get_copy();
            out << ",\"kind\":\"copy\",\"loc\":" << c.loc << ",\"size\":" << c.size
                << ",\"src_offset\":" << c.src_offset << ",\"dst_offset\":" << c.dst_offset;
        } else if (op.is_partialize()) {
            auto const& x = op.get_partialize();
            out << ",\"kind\":\"partialize\",\"loc\":" << x.loc << ",\"offset\":" << x.offset << ",\"size\":" << x.size;
        } else if (op.is_alloc()) {
            auto const& x = op.get_alloc();
            out << ",\"kind\":\"alloc\",\"loc\":" << x.loc << ",\"offset\":" << x.offset << ",\"size\":" << x.size;
        } else if (op.is_del()) {
            auto const& x = op.get_del();
            out << ",\"kind\":\"del\",\"loc\":" << x.loc << ",\"offset\":" << x.offset << ",\"size\":" << x.size;
        } else if (op.is_inputsto()) {
            auto const& x = op.get_inputsto();
            out << ",\"kind\":\"inputsto\",\"loc\":" << x.storage_loc << ",\"storage_loc\":" << x.storage_loc
                << ",\"storage_id\":" << x.storage_id << ",\"size\":" << x.size;
        } else if (op.is_evict()) {
            auto const& x = op.get_evict();
            out << ",\"kind\":\"evict\",\"loc\":" << x.src.loc << ",\"offset\":" << x.src.offset << ",\"size\":" << x.src.size
                << ",\"storage_loc\":" << x.dst.loc << ",\"storage_id\":" << x.dst.id;
        } else if (op.is_load()) {
            auto const& x = op.get_load();
            out << ",\"kind\":\"load\",\"loc\":" << x.dst.loc << ",\"offset\":" << x.dst.offset << ",\"size\":" << x.dst.size
                << ",\"storage_loc\":" << x.src.loc << ",\"storage_id\":" << x.src.id;
        } else {
            throw std::runtime_error("unknown memgraph node kind");
        }
        out << "}";
    }
    out << "\n]}\n";
    return 0;
    G_END
}

// The memgraph executed op by op with the reference's own per-op interpreter
// functions, in get_order() order, with the first-touch-of-a-group-is-a-copy rule
// -- the loop of reference_compute_memgraph (src/einsummable/reference.cc:191-307)
// extended by the one case it lacks: constant (fill) nodes, which a LLaMA
// memgraph contains (the causal mask) and which reference_compute_memgraph
// rejects ("should not happen").  Fills use the reference's reference_fill.
int ref_graph_run(int h, void** loc_buffers)
{
    G_BEGIN
    built_graph_t const& b = *g_graphs.at(h);
    memgraph_t const&    mg = b.memgraph;
    auto                 at = [&](int loc, uint64_t offset) {
        return reinterpret_cast<uint8_t*>(loc_buffers[loc]) + offset;
    };
    set<int> groups_touched;
    for (int const& id : mg.get_order()) {
        auto const& op = mg.nodes[id].op;
        if (op.is_constant()) {
            auto const& c = op.get_constant();
            dbuffer_t   v = reference_fill(c.fill);
            std::copy((uint8_t*)v.raw(), (uint8_t*)v.raw() + v.size(), at(c.loc, c.offset));
        } else if (op.is_apply()) {
            auto const& apply = op.get_apply();
            auto        buf = [&](int i, dtype_t d) {
                return dbuffer_t(d, make_buffer_reference(at(apply.loc, apply.mems[i].offset), apply.mems[i].size));
            };
            if (apply.is_einsummable()) {
                einsummable_t const e = apply.get_einsummable().replace_scalar_variables(b.vars);
                vector<dbuffer_t> inns;
                for (int i = 1; i != apply.mems.size(); ++i) {
                    inns.push_back(buf(i, e.inn_dtype(i - 1)));
                }
                reference_einsummable_inplace(e, buf(0, e.out_dtype()), inns);
            } else {
                touch_t touch = apply.get_touch();
                if (apply.group < 0) {
                    touch.castable.reset();
                } else if (groups_touched.count(apply.group) == 0) {
                    touch.castable.reset();
                    groups_touched.insert(apply.group);
                }
                reference_touch(touch, buf(0, touch.dtype), buf(1, touch.dtype));
            }
        } else if (op.is_move()) {
            auto const& m = op.get_move();
            uint8_t*    src = at(std::get<0>(m.src), std::get<1>(m.src));
            std::copy(src, src + m.size, at(std::get<0>(m.dst), std::get<1>(m.dst)));
        } else if (op.is_copy()) {
            auto const& c = op.get_copy();
            std::copy(at(c.loc, c.src_offset), at(c.loc, c.src_offset) + c.size, at(c.loc, c.dst_offset));
        } else if (op.is_inputmem() || op.is_partialize() || op.is_alloc() || op.is_del()) {
            // nothing to do
        } else {
            throw std::runtime_error("ref_graph_run: storage nodes are not expected here");
        }
    }
    return 0;
    G_END
}

} // extern "C"
