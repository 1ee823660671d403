// gpu_program_t over the es_b200 C ABI; see gpu_program.h.
#include "gpu_program.h"

#include <cstring>

namespace {

void check(int status, char const* what)
{
    if (status != ES_OK) {
        throw std::runtime_error(string(what) + ": es_b200 status " + std::to_string(status) + ": " +
                                 es_b200_last_error());
    }
}

void scalar_bytes(scalar_t const& s, unsigned char out[8])
{
    std::memset(out, 0, 8);
    std::memcpy(out, s.data, dtype_size(s.dtype));
}

void* host_block(storage_blocks_t const* storage, stoloc_t const& at, char const* who)
{
    if (!storage) {
        throw std::runtime_error(string(who) + ": the memgraph has evict / load nodes but no storage blocks were given");
    }
    auto iter = storage->find({at.loc, at.id});
    if (iter == storage->end()) {
        throw std::runtime_error(string(who) + ": no host block for storage id " + std::to_string(at.id) +
                                 " of storage location " + std::to_string(at.loc));
    }
    return iter->second;
}

es_attention_t attention_descriptor(es_fuse::attention_t const& d)
{
    es_attention_t a;
    std::memset(&a, 0, sizeof(a));
    a.batch = d.batch, a.heads = d.heads, a.rows = d.rows, a.keys = d.keys, a.head_dim = d.head_dim;
    a.skip_known = d.skip_known, a.skip_from = d.skip_from;
    for (int i = 0; i != 3; ++i) {
        a.q_stride[i] = d.q_stride[i], a.k_stride[i] = d.k_stride[i];
        a.v_stride[i] = d.v_stride[i], a.out_stride[i] = d.out_stride[i];
    }
    a.mask_stride = d.mask_stride;
    return a;
}

} // namespace

gpu_program_t::gpu_program_t(memgraph_t const&            memgraph,
                             int                          loc,
                             kernel_manager_t&            km,
                             void*                        mem,
                             map<string, scalar_t> const& scalar_vars,
                             int                          max_lanes,
                             es_exchange::attention_map_t const* attention,
                             storage_blocks_t const*      storage)
    : prog(nullptr), workspace(nullptr), n_ops(0)
{
    check(es_b200_program_create(km.c_handle(), &prog), "es_b200_program_create");
    auto at = [&](uint64_t offset) { return static_cast<void*>(static_cast<char*>(mem) + offset); };

    int const n = int(memgraph.nodes.size());
    // op index of every node that launches something here; for the others (inputmem, inputsto,
    // partialize, alloc, del: they carry "this memory is free again" but launch nothing) the ops
    // they stand for
    vector<int>         op_of(n, -1);
    vector<vector<int>> stands_for(n);
    map<int, int>       group_last; // touches of a group are chained; the first one is the copy
                                    // (src/engine/gpu/exec_graph.cc:167-172,368-378)
    for (int mid = 0; mid != n; ++mid) {
        auto const& node = memgraph.nodes[mid];
        auto const& op = node.op;
        if (!memgraph.is_local_to(mid, loc)) {
            continue;
        }
        vector<int> deps;
        for (int inn : node.inns) {
            if (op_of[inn] >= 0) {
                deps.push_back(op_of[inn]);
            } else {
                deps.insert(deps.end(), stands_for[inn].begin(), stands_for[inn].end());
            }
        }
        std::sort(deps.begin(), deps.end());
        deps.erase(std::unique(deps.begin(), deps.end()), deps.end());

        int index = -1;
        if (op.is_inputmem() || op.is_inputsto() || op.is_partialize() || op.is_alloc() || op.is_del()) {
            stands_for[mid] = deps;
            continue;
        } else if (attention && attention->count(mid)) {
            es_fuse::attention_node_t const& a = attention->at(mid);
            es_attention_t                   d = attention_descriptor(a.desc);
            check(es_b200_program_add_attention(prog, &d, at(a.out.offset), at(a.q.offset), at(a.k.offset),
                                                at(a.v.offset), at(a.mask.offset), deps.data(), int(deps.size()), &index),
                  "es_b200_program_add_attention");
        } else if (op.is_apply()) {
            auto const& apply = op.get_apply();
            if (apply.is_einsummable()) {
                einsummable_t e =
                    apply.get_einsummable().replace_scalar_variables(scalar_vars).merge_adjacent_dims();
                if (!km.build(e)) {
                    throw std::runtime_error("gpu_program_t: could not build " + write_with_ss(e));
                }
                vector<void const*> inns;
                for (size_t i = 1; i != apply.mems.size(); ++i) {
                    inns.push_back(at(apply.mems[i].offset));
                }
                check(es_b200_program_add_einsummable(prog, km.kernel_id(e), at(apply.mems[0].offset), inns.data(),
                                                      int(inns.size()), deps.data(), int(deps.size()), &index),
                      "es_b200_program_add_einsummable");
            } else {
                touch_t const& touch = apply.get_touch();
                int            castable = touch.castable ? int(touch.castable.value()) : ES_CASTABLE_NONE;
                if (apply.group >= 0) {
                    auto iter = group_last.find(apply.group);
                    if (iter == group_last.end()) {
                        castable = ES_CASTABLE_NONE;
                    } else {
                        deps.push_back(iter->second);
                    }
                } else {
                    castable = ES_CASTABLE_NONE;
                }
                vector<es_touchdim_t> dims;
                for (auto const& d : touch.selection) {
                    dims.push_back(es_touchdim_t{d.d_inn, d.d_out, d.offset_inn, d.offset_out, d.size});
                }
                check(es_b200_program_add_touch(prog, dims.data(), int(dims.size()), castable, int(touch.dtype),
                                                at(apply.mems[0].offset), at(apply.mems[1].offset), deps.data(),
                                                int(deps.size()), &index),
                      "es_b200_program_add_touch");
                if (apply.group >= 0) {
                    group_last[apply.group] = index;
                }
            }
        } else if (op.is_constant()) {
            auto const&   c = op.get_constant();
            unsigned char a[8], b[8];
            if (c.fill.is_constant()) {
                auto const& f = c.fill.get_constant();
                scalar_bytes(f.value, a);
                check(es_b200_program_add_fill_constant(prog, int(f.value.dtype), a, product(f.shape), at(c.offset),
                                                        deps.data(), int(deps.size()), &index),
                      "es_b200_program_add_fill_constant");
            } else {
                auto const& f = c.fill.get_lowertri();
                scalar_bytes(f.lower, a);
                scalar_bytes(f.upper, b);
                check(es_b200_program_add_fill_lowertri(prog, int(f.lower.dtype), a, b, f.nrow, f.ncol, f.start,
                                                        at(c.offset), deps.data(), int(deps.size()), &index),
                      "es_b200_program_add_fill_lowertri");
            }
        } else if (op.is_move()) {
            auto const& m = op.get_move();
            if (m.get_src_loc() != loc || m.get_dst_loc() != loc) {
                throw std::runtime_error("gpu_program_t: a move between locations needs one program per device");
            }
            check(es_b200_program_add_copy(prog, at(std::get<1>(m.src)), at(std::get<1>(m.dst)), m.size, deps.data(),
                                           int(deps.size()), &index),
                  "es_b200_program_add_copy");
        } else if (op.is_copy()) {
            auto const& c = op.get_copy();
            check(es_b200_program_add_copy(prog, at(c.src_offset), at(c.dst_offset), c.size, deps.data(),
                                           int(deps.size()), &index),
                  "es_b200_program_add_copy");
        } else if (op.is_evict()) {
            auto const& e = op.get_evict();
            check(es_b200_program_add_evict(prog, at(e.src.offset), host_block(storage, e.dst, "gpu_program_t"), e.src.size,
                                            deps.data(), int(deps.size()), &index),
                  "es_b200_program_add_evict");
        } else if (op.is_load()) {
            auto const& l = op.get_load();
            check(es_b200_program_add_load(prog, host_block(storage, l.src, "gpu_program_t"), at(l.dst.offset), l.dst.size,
                                           deps.data(), int(deps.size()), &index),
                  "es_b200_program_add_load");
        } else {
            throw std::runtime_error("gpu_program_t: unknown memgraph node kind");
        }
        op_of[mid] = index;
        n_ops++;
    }
    uint64_t ws = 0;
    check(es_b200_program_finalize(prog, max_lanes, &ws), "es_b200_program_finalize");
    if (ws > 0) {
        if (cudaMalloc(&workspace, ws) != cudaSuccess) {
            throw std::runtime_error("gpu_program_t: could not allocate the workspace");
        }
    }
    check(es_b200_program_set_workspace(prog, workspace, ws), "es_b200_program_set_workspace");
}

gpu_program_t::~gpu_program_t()
{
    if (prog) {
        es_b200_program_destroy(prog);
    }
    if (workspace) {
        cudaFree(workspace);
    }
}

void gpu_program_t::launch(cudaStream_t stream)
{
    check(es_b200_program_launch(prog, stream), "es_b200_program_launch");
}

void gpu_program_t::instantiate()
{
    check(es_b200_program_instantiate(prog), "es_b200_program_instantiate");
}

void gpu_program_t::replay(cudaStream_t stream)
{
    check(es_b200_program_replay(prog, stream), "es_b200_program_replay");
}


// ------------------------------------------------------------------ one process per GPU
gpu_exchange_program_t::gpu_exchange_program_t(memgraph_t const&            memgraph,
                                               int                          rank,
                                               kernel_manager_t&            km,
                                               vector<void*> const&         peer_mem,
                                               vector<void*> const&         peer_flags,
                                               map<string, scalar_t> const& scalar_vars,
                                               int                          max_lanes,
                                               uint32_t                     wait_limit_ms,
                                               es_exchange::attention_map_t const* attention,
                                               bool                         group_sum,
                                               storage_blocks_t const*      storage)
    : prog(nullptr), workspace(nullptr), n_ops(0)
{
    check(es_b200_program_create(km.c_handle(), &prog), "es_b200_program_create");
    auto at = [&](int loc, uint64_t offset) { return static_cast<void*>(static_cast<char*>(peer_mem.at(loc)) + offset); };
    // cross-location moves in node order index the flag words
    map<int, int> move_index;
    for (int mid = 0; mid != int(memgraph.nodes.size()); ++mid) {
        auto const& op = memgraph.nodes[mid].op;
        if (op.is_move() && op.get_move().get_src_loc() != op.get_move().get_dst_loc()) {
            int k = int(move_index.size());
            move_index[mid] = k;
        }
    }
    int const n_moves = int(move_index.size());
    auto flag = [&](int owner, int kind, int mid) {
        return static_cast<void*>(static_cast<uint32_t*>(peer_flags.at(owner)) + kind * n_moves + move_index.at(mid));
    };
    // the rank's units in the order in which a simulation of all ranks serves them: the exchange ops share
    // one in-order lane, so what is expected to be ready first has to be asked for first
    for (es_exchange::unit_t const& u :
         es_exchange::order_units(memgraph, memgraph.num_compute_locs, rank, nullptr, attention, group_sum)) {
        int         index = -1;
        int const*  deps = u.deps.data();
        int const   n_deps = int(u.deps.size());
        if (u.kind == "einsummable") {
            auto const&   apply = memgraph.nodes[u.node].op.get_apply();
            einsummable_t e = apply.get_einsummable().replace_scalar_variables(scalar_vars).merge_adjacent_dims();
            if (!km.build(e)) {
                throw std::runtime_error("gpu_exchange_program_t: could not build " + write_with_ss(e));
            }
            vector<void const*> inns;
            for (size_t i = 1; i != apply.mems.size(); ++i) {
                inns.push_back(at(rank, apply.mems[i].offset));
            }
            check(es_b200_program_add_einsummable(prog, km.kernel_id(e), at(rank, apply.mems[0].offset), inns.data(),
                                                  int(inns.size()), deps, n_deps, &index),
                  "es_b200_program_add_einsummable");
        } else if (u.kind == "attention") {
            es_fuse::attention_node_t const& a = attention->at(u.node);
            es_attention_t                   d = attention_descriptor(a.desc);
            check(es_b200_program_add_attention(prog, &d, at(rank, a.out.offset), at(rank, a.q.offset),
                                                at(rank, a.k.offset), at(rank, a.v.offset), at(rank, a.mask.offset),
                                                deps, n_deps, &index),
                  "es_b200_program_add_attention");
        } else if (u.kind == "touch" || u.kind == "rtouch") {
            auto const&    apply = memgraph.nodes[u.node].op.get_apply();
            touch_t const& touch = apply.get_touch();
            int castable = (u.first || !touch.castable) ? ES_CASTABLE_NONE : int(touch.castable.value());
            vector<es_touchdim_t> dims;
            for (auto const& d : touch.selection) {
                dims.push_back(es_touchdim_t{d.d_inn, d.d_out, d.offset_inn, d.offset_out, d.size});
            }
            if (u.kind == "rtouch") {
                // the one reader of a moved block reads it where it is, in the source rank's memory
                auto const& mv = memgraph.nodes[u.moves[0]].op.get_move();
                check(es_b200_program_add_remote_touch(prog, dims.data(), int(dims.size()), castable, int(touch.dtype),
                                                       at(rank, apply.mems[0].offset),
                                                       at(mv.get_src_loc(), std::get<1>(mv.src)),
                                                       flag(mv.get_src_loc(), 1, u.moves[0]), deps, n_deps, &index),
                      "es_b200_program_add_remote_touch");
            } else {
                check(es_b200_program_add_touch(prog, dims.data(), int(dims.size()), castable, int(touch.dtype),
                                                at(rank, apply.mems[0].offset), at(rank, apply.mems[1].offset), deps,
                                                n_deps, &index),
                      "es_b200_program_add_touch");
            }
        } else if (u.kind == "constant") {
            auto const&   c = memgraph.nodes[u.node].op.get_constant();
            unsigned char a[8], b[8];
            if (c.fill.is_constant()) {
                auto const& f = c.fill.get_constant();
                scalar_bytes(f.value, a);
                check(es_b200_program_add_fill_constant(prog, int(f.value.dtype), a, product(f.shape), at(rank, c.offset),
                                                        deps, n_deps, &index),
                      "es_b200_program_add_fill_constant");
            } else {
                auto const& f = c.fill.get_lowertri();
                scalar_bytes(f.lower, a);
                scalar_bytes(f.upper, b);
                check(es_b200_program_add_fill_lowertri(prog, int(f.lower.dtype), a, b, f.nrow, f.ncol, f.start,
                                                        at(rank, c.offset), deps, n_deps, &index),
                      "es_b200_program_add_fill_lowertri");
            }
        } else if (u.kind == "copy") {
            auto const& op = memgraph.nodes[u.node].op;
            if (op.is_move()) {
                auto const& m = op.get_move();
                check(es_b200_program_add_copy(prog, at(rank, std::get<1>(m.src)), at(rank, std::get<1>(m.dst)), m.size, deps,
                                               n_deps, &index),
                      "es_b200_program_add_copy");
            } else {
                auto const& c = op.get_copy();
                check(es_b200_program_add_copy(prog, at(rank, c.src_offset), at(rank, c.dst_offset), c.size, deps, n_deps,
                                               &index),
                      "es_b200_program_add_copy");
            }
        } else if (u.kind == "rsum") {
            // out = out + r1 + ... + rk, the r's read where they are, in the peers' memory: one generated
            // elementwise kernel instead of k remote touches that wait for one another
            auto const&    first = memgraph.nodes[u.nodes[0]].op.get_apply();
            touch_t const& touch = first.get_touch();
            string const   dt = write_with_ss(touch.dtype);
            uint64_t const nelem = first.mems[0].size / dtype_size(touch.dtype);
            string         join = "hole|" + dt + "@0";
            for (size_t i = 1; i <= u.nodes.size(); ++i) {
                join = "+[" + join + ",hole|" + dt + "@" + std::to_string(i) + "]";
            }
            einsummable_t e({nelem}, vector<vector<int>>(u.nodes.size() + 1, vector<int>{0}), 1,
                            parse_with_ss<scalarop_t>(join));
            if (!km.build(e)) {
                throw std::runtime_error("gpu_exchange_program_t: could not build " + write_with_ss(e));
            }
            void*               out = at(rank, first.mems[0].offset);
            vector<void const*> inns{out};
            for (int m : u.moves) {
                auto const& mv = memgraph.nodes[m].op.get_move();
                inns.push_back(at(mv.get_src_loc(), std::get<1>(mv.src)));
            }
            check(es_b200_program_add_einsummable(prog, km.kernel_id(e), out, inns.data(), int(inns.size()), deps,
                                                  n_deps, &index),
                  "es_b200_program_add_einsummable");
        } else if (u.kind == "ack") {
            // the done flags of the moves an rsum consumed, in the sources' arrays
            vector<void*> flags;
            for (int m : u.moves) {
                flags.push_back(flag(memgraph.nodes[m].op.get_move().get_src_loc(), 1, m));
            }
            check(es_b200_program_add_signal(prog, flags.data(), int(flags.size()), deps, n_deps, &index),
                  "es_b200_program_add_signal");
        } else if (u.kind == "signal" || u.kind == "await" || u.kind == "wait") {
            // signal: the ready flags in the destinations' arrays; await: this rank's ready flags;
            // wait: this rank's done flags
            vector<void*> flags;
            for (int m : u.moves) {
                auto const& mv = memgraph.nodes[m].op.get_move();
                flags.push_back(u.kind == "wait" ? flag(rank, 1, m) : flag(mv.get_dst_loc(), 0, m));
            }
            if (u.kind == "signal") {
                check(es_b200_program_add_signal(prog, flags.data(), int(flags.size()), deps, n_deps, &index),
                      "es_b200_program_add_signal");
            } else {
                check(es_b200_program_add_wait(prog, flags.data(), int(flags.size()), deps, n_deps, &index),
                      "es_b200_program_add_wait");
            }
        } else if (u.kind == "pull") {
            vector<es_pull_item_t> items;
            for (int m : u.moves) {
                auto const&    mv = memgraph.nodes[m].op.get_move();
                es_pull_item_t it;
                it.src = at(mv.get_src_loc(), std::get<1>(mv.src));
                it.dst = at(rank, std::get<1>(mv.dst));
                it.bytes = mv.size;
                it.ready_flag = nullptr; // the await in front of this pull has seen the flag
                it.done_flag = flag(mv.get_src_loc(), 1, m);
                items.push_back(it);
            }
            check(es_b200_program_add_pull(prog, items.data(), int(items.size()), deps, n_deps, &index),
                  "es_b200_program_add_pull");
        } else if (u.kind == "evict") {
            auto const& e = memgraph.nodes[u.node].op.get_evict();
            check(es_b200_program_add_evict(prog, at(rank, e.src.offset), host_block(storage, e.dst, "gpu_exchange_program_t"),
                                            e.src.size, deps, n_deps, &index),
                  "es_b200_program_add_evict");
        } else if (u.kind == "load") {
            auto const& l = memgraph.nodes[u.node].op.get_load();
            check(es_b200_program_add_load(prog, host_block(storage, l.src, "gpu_exchange_program_t"), at(rank, l.dst.offset),
                                           l.dst.size, deps, n_deps, &index),
                  "es_b200_program_add_load");
        } else {
            throw std::runtime_error("gpu_exchange_program_t: unknown unit kind " + u.kind);
        }
        n_ops++;
    }
    uint64_t ws = 0;
    check(es_b200_program_finalize(prog, max_lanes, &ws), "es_b200_program_finalize");
    if (ws > 0) {
        if (cudaMalloc(&workspace, ws) != cudaSuccess) {
            throw std::runtime_error("gpu_exchange_program_t: could not allocate the workspace");
        }
    }
    check(es_b200_program_set_workspace(prog, workspace, ws), "es_b200_program_set_workspace");
    if (wait_limit_ms) {
        check(es_b200_program_set_wait_limit(prog, wait_limit_ms), "es_b200_program_set_wait_limit");
    }
}

gpu_exchange_program_t::~gpu_exchange_program_t()
{
    if (prog) {
        es_b200_program_destroy(prog);
    }
    if (workspace) {
        cudaFree(workspace);
    }
}

void gpu_exchange_program_t::launch(cudaStream_t stream)
{
    check(es_b200_program_launch(prog, stream), "es_b200_program_launch");
}

void gpu_exchange_program_t::instantiate()
{
    check(es_b200_program_instantiate(prog), "es_b200_program_instantiate");
}

void gpu_exchange_program_t::replay(cudaStream_t stream)
{
    check(es_b200_program_replay(prog, stream), "es_b200_program_replay");
}
