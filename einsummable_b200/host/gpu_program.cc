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

} // namespace

gpu_program_t::gpu_program_t(memgraph_t const&            memgraph,
                             int                          loc,
                             kernel_manager_t&            km,
                             void*                        mem,
                             map<string, scalar_t> const& scalar_vars,
                             int                          max_lanes)
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
        } else {
            throw std::runtime_error("gpu_program_t: evict / load nodes need a storage (es_b200_program_add_evict / _add_load)");
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
