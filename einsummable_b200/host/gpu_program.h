// gpu_program_t: the nodes of a memgraph that run on one GPU, compiled once into a program of the
// es_b200 library's executor and replayed without the host in the loop.
//
// An alternative to exec_graph_t::make_gpu_exec_graph + exec_state_t::event_loop
// (src/engine/gpu/exec_graph.cc:37-256, src/engine/exec_state.cc:110-219) for the part of
// gpu_mg_server_t::execute_memgraph (src/server/gpu/server.cc:96-136) that runs on one device: the same
// memgraph_t, the same kernel_manager_t, the same global buffer -- but every op is ordered behind
// exactly the ops it depends on by CUDA events (or CUDA-graph edges) instead of being launched from a
// stream callback of its predecessors.
//
// Place beside gpu_kernel_manager.{h,cc} in src/engine/gpu/.  One location per program; moves to or from
// other locations are not handled here (a box driven by one process needs one program per device and
// events between them; processes that each drive one GPU use the exchange ops of es_b200.h).
#pragma once
#include "../../base/setup.h"

#include "../../einsummable/memgraph.h"
#include "gpu_exchange_plan.h"
#include "gpu_kernel_manager.h"

// Where the tensors of a memgraph with storage live on the host: (storage location, storage id) -> a pinned
// host block of the tensor's size (e.g. from es_b200_storage_reference).  Ids are unique within a run
// (src/einsummable/memgraph.h:311-316), so with the blocks fixed in advance evict_t / load_t
// (src/engine/gpu/exec_graph.cc:469-577) are plain copies in a static schedule; an inputsto node's block holds
// its tensor before the run, a saved tensor that ended up in storage is in its block afterwards.
using storage_blocks_t = map<tuple<int, int>, void*>;

struct gpu_program_t {
    // mem: the global buffer of location `loc` (server.cc:38-43).  The kernel manager must outlive the program.
    // attention: for a graph from es_fuse::fold_attention (gpu_fuse.h), the nodes that stand for a whole
    // softmax(Q K^T + mask) V chain; each becomes one es_b200_program_add_attention op.
    gpu_program_t(memgraph_t const&                   memgraph,
                  int                                 loc,
                  kernel_manager_t&                   km,
                  void*                               mem,
                  map<string, scalar_t> const&        scalar_vars = {},
                  int                                 max_lanes = 16,
                  es_exchange::attention_map_t const* attention = nullptr,
                  storage_blocks_t const*             storage = nullptr);
    ~gpu_program_t();

    gpu_program_t(gpu_program_t const&) = delete;
    gpu_program_t& operator=(gpu_program_t const&) = delete;

    // One run, asynchronous on `stream` (which continues when every op has finished).
    void launch(cudaStream_t stream);
    // The run as one CUDA graph: instantiate() once (after one launch()), then replay().
    void instantiate();
    void replay(cudaStream_t stream);

    int num_ops() const
    {
        return n_ops;
    }

private:
    es_b200_program_t* prog;
    void*              workspace;
    int                n_ops;
};

// One rank's share of a memgraph when every location is driven by its own process (one process per GPU):
// the units of gpu_exchange_plan.h, in the order of simulated service, as a program, moves between locations as the
// library's exchange ops
// (es_b200_program_add_signal / _add_wait / _add_pull / _add_remote_touch).
//
// peer_mem[r] is location r's global buffer as THIS process can address it (peer-mapped / IPC / symmetric
// memory; peer_mem[rank] is the local buffer), and flags(r) the same for an array of 2 x n_moves zeroed 32-bit
// words that every rank places at the same offset: word k is the ready flag of cross-location move k (it lives in
// the destination's array), word n_moves + k its done flag (in the source's array), k counting the memgraph's
// cross-location moves in node order.  All ranks build their programs from the same memgraph and launch them
// the same number of times.  attention: as for gpu_program_t.  group_sum: the remote adds of a partial-sum group as one
// kernel over the peers' memory (es_exchange::make_units).
struct gpu_exchange_program_t {
    gpu_exchange_program_t(memgraph_t const&            memgraph,
                           int                          rank,
                           kernel_manager_t&            km,
                           vector<void*> const&         peer_mem,
                           vector<void*> const&         peer_flags,
                           map<string, scalar_t> const& scalar_vars = {},
                           int                          max_lanes = 16,
                           uint32_t                     wait_limit_ms = 0,
                           es_exchange::attention_map_t const* attention = nullptr,
                           bool                         group_sum = false,
                           storage_blocks_t const*      storage = nullptr);
    ~gpu_exchange_program_t();

    gpu_exchange_program_t(gpu_exchange_program_t const&) = delete;
    gpu_exchange_program_t& operator=(gpu_exchange_program_t const&) = delete;

    void launch(cudaStream_t stream);
    void instantiate();
    void replay(cudaStream_t stream);

    int num_ops() const
    {
        return n_ops;
    }

private:
    es_b200_program_t* prog;
    void*              workspace;
    int                n_ops;
};
