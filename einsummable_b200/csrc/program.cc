// The program executor: a memgraph's nodes for one GPU as a static, dependency-ordered launch
// schedule.
//
// The reference runs a memgraph through exec_state_t::event_loop (src/engine/exec_state.cc:110-219):
// every node is launched when its dependencies have called back from a CUDA stream
// (cudaStreamAddCallback, src/engine/gpu/exec_graph.cc:318-332), with at most five streams per
// device (src/server/gpu/server.h:81), so every node costs a device->host->device round trip.
// Here the same dependency graph is compiled once into "lanes" (CUDA streams) joined by events:
// an op waits for exactly the ops it depends on, nothing returns to the host between ops, and the
// whole schedule can be captured into one CUDA graph and replayed.
//
// Lanes.  Ops that spin on a flag another GPU raises (pull, wait) go to an exchange lane of
// their own (optionally a few: round robin in program order, so each of these lanes is in program
// order) and no other op is ever queued behind them.  The ranks list their exchange ops in one global order
// along which every dependency -- also those that cross ranks -- points forward; the earliest
// unfinished exchange op is therefore always at the head of its lane with everything it needs
// finished or running, and can proceed whatever the other lanes wait for.  (This relies on what
// every kernel that waits for a peer GPU relies on: kernels of different streams whose
// dependencies are met get to run beside a kernel that spins.  Every wait is bounded, so a
// platform where that failed would report an error word, not hang.  With one exchange lane this
// has held in every run; with four, launched eagerly on more streams than the device has
// hardware queues, bounded waits did run out on 8 GPUs -- hence the default of one.)  Every other op continues
// the lane of one of its dependencies when that dependency is the lane's last op, and otherwise
// takes the lane that has been idle longest.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "attention.h"
#include "common.h"
#include "exchange.h"
#include "handle.h"
#include "kernels.h"
#include "nvtx_ranges.h"
#include "pdl.h"

namespace {

using namespace es;

enum op_kind_t {
    OP_EINSUMMABLE = 0,
    OP_TOUCH = 1,
    OP_FILL_CONSTANT = 2,
    OP_FILL_LOWERTRI = 3,
    OP_COPY = 4,
    OP_SIGNAL = 5,
    OP_PULL = 6,
    OP_WAIT = 7,
    OP_TOUCH_BATCH = 8,
    OP_EVICT = 9,
    OP_LOAD = 10,
    OP_ATTENTION = 11
};

char const* const OP_NAMES[] = {"einsummable", "touch", "fill_constant", "fill_lowertri", "copy",
                                "signal",      "pull",  "wait",          "touch_batch",   "evict",
                                "load",        "attention"};

struct op_t {
    int              kind = 0;
    std::vector<int> deps;
    // schedule (finalize)
    int              lane = -1;
    std::vector<int> wait_on; // ops of other lanes whose events this op waits for
    bool             record = false;
    // payloads
    uint64_t                 kernel_id = 0;
    void*                    out = nullptr;
    std::vector<void const*> inns;
    uint64_t                 ws_need = 0;
    touch_args_t             touch;
    int                      touch_width = 0, dtype = 0;
    unsigned char            v0[8], v1[8];
    uint64_t                 nelem = 0, nrow = 0, ncol = 0;
    int64_t                  start = 0;
    void const*              src = nullptr;
    uint64_t                 bytes = 0;
    std::vector<uint32_t*>   flags;      // signal / wait
    std::vector<pull_item_t> pulls;      // pull
    std::vector<touch_args_t> batch;     // touch batch (one dtype, one width)
    es_attention_t           attn;
    uint64_t                 batch_slots = 0;
    // device-side descriptor arrays (finalize)
    uint64_t                 dev_off = 0, dev_off2 = 0;
    uint32_t                 max_ctas = 1;
    uint64_t                 work_bytes = 0;
};

} // namespace

struct es_b200_program {
    es_b200*                 h = nullptr; // null: planning only (no device)
    std::vector<op_t>        ops;
    bool                     finalized = false;
    int                      n_lanes = 0;
    bool                     has_spin = false;
    int                      exchange_lanes = 1; // lanes shared by the ops that wait for a peer
    int                      n_exchange = 0;     // how many of them the schedule uses
    bool                     pdl = true;         // programmatic dependent launch between the ops of a lane
    uint32_t                 limit_ms = 0;
    std::vector<cudaStream_t> lanes;
    std::vector<cudaEvent_t>  events; // one per op that some other lane waits for
    std::vector<int>          event_of;
    std::vector<int>          lane_last;
    cudaEvent_t               fork_ev = nullptr;
    std::vector<cudaEvent_t>  join_ev;
    char*                     dev_buf = nullptr;
    uint64_t                  dev_bytes = 0;
    uint32_t*                 epoch_dev = nullptr;
    std::vector<uint64_t>     lane_ws_off;
    uint64_t                  ws_total = 0;
    char*                     ws_base = nullptr;
    uint64_t                  ws_bytes = 0;
    cudaStream_t              capture_stream = nullptr;
    cudaGraph_t               graph = nullptr;
    cudaGraphExec_t           exec = nullptr;
    std::vector<cudaEvent_t>  t0, t1; // timing events (launch_timed)
    cudaGraph_t               graph_timed = nullptr; // the run with a time stamp before and after every op
    cudaGraphExec_t           exec_timed = nullptr;
    unsigned long long*       stamps_dev = nullptr;  // [2 * n_ops + 2]
};

namespace {

void check_program(es_b200_program* p, bool want_final)
{
    if (!p) fail(ES_BAD_ARGUMENT, "null program");
    if (want_final && !p->finalized) fail(ES_BAD_ARGUMENT, "program: finalize first");
    if (!want_final && p->finalized) fail(ES_BAD_ARGUMENT, "program: already finalized");
}

int add_op(es_b200_program* p, op_t&& op, int const* deps, int n_deps, int* index)
{
    if (n_deps < 0 || (n_deps > 0 && !deps)) fail(ES_BAD_ARGUMENT, "program: bad dependency list");
    int me = (int)p->ops.size();
    for (int i = 0; i != n_deps; ++i) {
        if (deps[i] < 0 || deps[i] >= me) fail(ES_BAD_ARGUMENT, "program: a dependency must be an earlier op");
        op.deps.push_back(deps[i]);
    }
    std::sort(op.deps.begin(), op.deps.end());
    op.deps.erase(std::unique(op.deps.begin(), op.deps.end()), op.deps.end());
    p->ops.push_back(std::move(op));
    if (index) *index = me;
    return me;
}

bool is_spin(op_t const& op)
{
    if (op.kind == OP_WAIT) return true;
    if (op.kind == OP_PULL)
        for (auto const& it : op.pulls)
            if (it.ready) return true;
    return false;
}

uint64_t round_up(uint64_t v, uint64_t a)
{
    return (v + a - 1) / a * a;
}

// Lane assignment and the cross-lane waits that are actually needed.
void schedule(es_b200_program* p, int max_lanes)
{
    auto& ops = p->ops;
    int   n = (int)ops.size();
    p->has_spin = false;
    for (auto const& op : ops) p->has_spin = p->has_spin || is_spin(op);
    int first_compute = p->has_spin ? std::max(p->exchange_lanes, 1) : 0;
    int n_lanes = std::max(max_lanes, 1) + first_compute;
    int n_spin = 0;
    p->n_exchange = first_compute;
    std::vector<int> tail(n_lanes, -1);
    // known[l][m]: the highest op index of lane m known to be complete when lane l's next op starts
    std::vector<std::vector<int>> known(n_lanes, std::vector<int>(n_lanes, -1));
    std::vector<std::vector<int>> known_after(n); // snapshot once the op has been issued
    int used = 0;
    for (int i = 0; i != n; ++i) {
        op_t& op = ops[i];
        int   lane = -1;
        if (is_spin(op)) {
            lane = n_spin++ % first_compute; // round robin, so that every exchange lane is in program order
        } else {
            int best = -1;
            for (int d : op.deps) {
                int l = ops[d].lane;
                if (l >= first_compute && tail[l] == d && d > best) {
                    best = d;
                    lane = l;
                }
            }
            if (lane < 0) {
                // the lane whose last op is oldest (an empty lane first)
                lane = first_compute;
                for (int l = first_compute; l != n_lanes; ++l)
                    if (tail[l] < tail[lane]) lane = l;
            }
        }
        op.lane = lane;
        used = std::max(used, lane + 1);
        op.wait_on.clear();
        // latest dependency per other lane; skip what this lane already knows to be complete
        std::vector<int> need(n_lanes, -1);
        for (int d : op.deps) {
            int l = ops[d].lane;
            if (l != lane) need[l] = std::max(need[l], d);
        }
        for (int l = 0; l != n_lanes; ++l) {
            if (need[l] < 0 || known[lane][l] >= need[l]) continue;
            op.wait_on.push_back(need[l]);
            ops[need[l]].record = true;
            // waiting for op d also brings everything d's lane knew when d was issued
            auto const& ka = known_after[need[l]];
            for (int m = 0; m != n_lanes; ++m) known[lane][m] = std::max(known[lane][m], ka[m]);
            known[lane][l] = std::max(known[lane][l], need[l]);
        }
        tail[lane] = i;
        known[lane][lane] = i;
        known_after[i] = known[lane];
        known_after[i][lane] = i;
    }
    p->n_lanes = std::max(used, 1);
    p->lane_last.assign(p->n_lanes, -1);
    for (int i = 0; i != n; ++i) p->lane_last[ops[i].lane] = i;
    // workspace: ops of one lane run one after the other and share the lane's slice
    p->lane_ws_off.assign(p->n_lanes, 0);
    std::vector<uint64_t> need_ws(p->n_lanes, 0);
    for (auto const& op : ops)
        if (op.kind == OP_EINSUMMABLE) need_ws[op.lane] = std::max(need_ws[op.lane], op.ws_need);
    uint64_t off = 0;
    for (int l = 0; l != p->n_lanes; ++l) {
        p->lane_ws_off[l] = off;
        off += round_up(need_ws[l], 256);
    }
    p->ws_total = off;
}

void free_device_side(es_b200_program* p)
{
    if (p->exec) cudaGraphExecDestroy(p->exec);
    if (p->graph) cudaGraphDestroy(p->graph);
    if (p->exec_timed) cudaGraphExecDestroy(p->exec_timed);
    if (p->graph_timed) cudaGraphDestroy(p->graph_timed);
    if (p->stamps_dev) cudaFree(p->stamps_dev);
    p->exec_timed = nullptr;
    p->graph_timed = nullptr;
    p->stamps_dev = nullptr;
    if (p->capture_stream) cudaStreamDestroy(p->capture_stream);
    for (auto e : p->events) cudaEventDestroy(e);
    for (auto e : p->join_ev) cudaEventDestroy(e);
    for (auto e : p->t0) cudaEventDestroy(e);
    for (auto e : p->t1) cudaEventDestroy(e);
    if (p->fork_ev) cudaEventDestroy(p->fork_ev);
    for (auto s : p->lanes) cudaStreamDestroy(s);
    if (p->dev_buf) cudaFree(p->dev_buf);
    p->exec = nullptr;
    p->graph = nullptr;
    p->capture_stream = nullptr;
    p->events.clear();
    p->join_ev.clear();
    p->t0.clear();
    p->t1.clear();
    p->fork_ev = nullptr;
    p->lanes.clear();
    p->dev_buf = nullptr;
}

// Descriptor arrays of the exchange ops and touch batches, the epoch word and the pull counters
// go into one device buffer, allocated and filled once.
void upload(es_b200_program* p)
{
    auto&             ops = p->ops;
    std::vector<char> host(256, 0); // [0,4): epoch
    auto              place = [&](void const* data, uint64_t bytes) {
        uint64_t off = round_up(host.size(), 16);
        host.resize(off + bytes, 0);
        if (data) std::memcpy(host.data() + off, data, bytes);
        return off;
    };
    for (auto& op : ops) {
        if (op.kind == OP_SIGNAL || op.kind == OP_WAIT) {
            op.dev_off = place(op.flags.data(), op.flags.size() * sizeof(uint32_t*));
        } else if (op.kind == OP_PULL) {
            op.dev_off = place(op.pulls.data(), op.pulls.size() * sizeof(pull_item_t));
            op.dev_off2 = place(nullptr, op.pulls.size() * sizeof(uint32_t));
        } else if (op.kind == OP_TOUCH_BATCH) {
            op.dev_off = place(op.batch.data(), op.batch.size() * sizeof(touch_args_t));
        } else if (op.kind == OP_TOUCH && op.touch.done) {
            op.dev_off = place(nullptr, sizeof(uint32_t));
        }
    }
    p->dev_bytes = round_up(host.size(), 256);
    host.resize(p->dev_bytes, 0);
    ES_CUDA_CHECK(cudaMalloc(&p->dev_buf, p->dev_bytes));
    ES_CUDA_CHECK(cudaMemcpy(p->dev_buf, host.data(), p->dev_bytes, cudaMemcpyHostToDevice));
    p->epoch_dev = reinterpret_cast<uint32_t*>(p->dev_buf);
    for (auto& op : ops) {
        if (op.kind == OP_TOUCH && op.touch.done) {
            op.touch.counter = reinterpret_cast<uint32_t*>(p->dev_buf + op.dev_off);
            op.touch.epoch = p->epoch_dev;
        }
    }
}

void launch_op(es_b200_program* p, op_t const& op, cudaStream_t s)
{
    es_b200* h = p->h;
    switch (op.kind) {
        case OP_EINSUMMABLE: {
            void* ws = op.ws_need ? p->ws_base + p->lane_ws_off[op.lane] : nullptr;
            launch_built(h, op.kernel_id, s, op.out, op.inns.data(), (int)op.inns.size(), ws,
                         op.ws_need ? round_up(op.ws_need, 256) : 0);
            break;
        }
        case OP_TOUCH:
            launch_touch(op.touch, op.touch_width, op.dtype, s);
            h->counters[1] += 1;
            h->work_bytes[1] += op.work_bytes;
            break;
        case OP_TOUCH_BATCH:
            launch_touch_batch(reinterpret_cast<touch_args_t const*>(p->dev_buf + op.dev_off), (int)op.batch.size(),
                               op.batch_slots, op.touch_width, op.dtype, s);
            h->counters[1] += 1;
            h->work_bytes[1] += op.work_bytes;
            break;
        case OP_FILL_CONSTANT:
            launch_fill_constant(op.dtype, op.v0, op.nelem, s, op.out);
            h->counters[2] += 1;
            h->work_bytes[2] += op.work_bytes;
            break;
        case OP_FILL_LOWERTRI:
            launch_fill_lowertri(op.dtype, op.v0, op.v1, op.nrow, op.ncol, op.start, s, op.out);
            h->counters[2] += 1;
            h->work_bytes[2] += op.work_bytes;
            break;
        case OP_ATTENTION:
            launch_attention(op.attn, s, op.out, op.inns[0], op.inns[1], op.inns[2], op.inns[3]);
            h->counters[0] += 1;
            h->work_bytes[0] += op.work_bytes;
            h->work_flops += attention_flops(op.attn);
            break;
        case OP_COPY:
            launch_pull_copy(op.src, op.out, op.bytes, s);
            h->counters[3] += 1;
            h->work_bytes[3] += op.bytes;
            break;
        case OP_EVICT:
            ES_CUDA_CHECK(cudaMemcpyAsync(op.out, op.src, op.bytes, cudaMemcpyDeviceToHost, s));
            h->counters[3] += 1;
            h->work_bytes[3] += op.bytes;
            break;
        case OP_LOAD:
            ES_CUDA_CHECK(cudaMemcpyAsync(op.out, op.src, op.bytes, cudaMemcpyHostToDevice, s));
            h->counters[3] += 1;
            h->work_bytes[3] += op.bytes;
            break;
        case OP_SIGNAL:
            launch_signal_many(reinterpret_cast<uint32_t* const*>(p->dev_buf + op.dev_off), (int)op.flags.size(),
                               p->epoch_dev, s);
            h->counters[3] += 1;
            break;
        case OP_WAIT:
            launch_wait_many(reinterpret_cast<uint32_t* const*>(p->dev_buf + op.dev_off), (int)op.flags.size(),
                             p->epoch_dev, p->limit_ms, s);
            h->counters[3] += 1;
            break;
        case OP_PULL:
            launch_pull_batch(reinterpret_cast<pull_item_t const*>(p->dev_buf + op.dev_off),
                              reinterpret_cast<uint32_t*>(p->dev_buf + op.dev_off2), (int)op.pulls.size(),
                              op.max_ctas, p->epoch_dev, p->limit_ms, s);
            h->counters[3] += 1;
            h->work_bytes[3] += op.work_bytes;
            break;
        default: fail(ES_BAD_ARGUMENT, "program: unknown op kind");
    }
}

// One run: fork from `stream` into the lanes, issue every op on its lane behind the events of
// its dependencies, join back into `stream`.  Nothing synchronises with the host.
enum { RUN_PLAIN = 0, RUN_EVENTS = 1, RUN_STAMPS = 2 };

void launch_all(es_b200_program* p, cudaStream_t stream, int mode)
{
    bool const timed = mode == RUN_EVENTS;
    bool const stamps = mode == RUN_STAMPS;
    if (!p->h) fail(ES_BAD_ARGUMENT, "program: created without a device (planning only)");
    if (p->ws_total > 0 && (!p->ws_base || p->ws_bytes < p->ws_total))
        fail(ES_WORKSPACE_TOO_SMALL, "program: workspace of " + std::to_string(p->ws_total) + " bytes required");
    ES_CUDA_CHECK(cudaSetDevice(p->h->device));
    launch_epoch_bump(p->epoch_dev, stream);
    if (stamps) launch_stamp(p->stamps_dev + 2 * p->ops.size(), stream);
    ES_CUDA_CHECK(cudaEventRecord(p->fork_ev, stream));
    for (int l = 0; l != p->n_lanes; ++l)
        if (p->lane_last[l] >= 0) ES_CUDA_CHECK(cudaStreamWaitEvent(p->lanes[l], p->fork_ev, 0));
    for (size_t i = 0; i != p->ops.size(); ++i) {
        op_t const&  op = p->ops[i];
        cudaStream_t s = p->lanes[op.lane];
        for (int d : op.wait_on) ES_CUDA_CHECK(cudaStreamWaitEvent(s, p->events[p->event_of[d]], 0));
        if (timed) ES_CUDA_CHECK(cudaEventRecord(p->t0[i], s));
        {
            // an op may be scheduled while the op before it on its lane finishes (pdl.h)
            pdl_scope_t  scope(p->pdl);
            nvtx_range_t range(nvtx_on() ? std::string("op ") + std::to_string(i) + " lane " + std::to_string(op.lane) + " " +
                                               OP_NAMES[op.kind]
                                         : std::string());
            if (stamps) launch_stamp(p->stamps_dev + 2 * i, s);
            launch_op(p, op, s);
            if (stamps) launch_stamp(p->stamps_dev + 2 * i + 1, s);
        }
        if (timed) ES_CUDA_CHECK(cudaEventRecord(p->t1[i], s));
        if (op.record) ES_CUDA_CHECK(cudaEventRecord(p->events[p->event_of[i]], s));
    }
    for (int l = 0; l != p->n_lanes; ++l) {
        if (p->lane_last[l] < 0) continue;
        ES_CUDA_CHECK(cudaEventRecord(p->join_ev[l], p->lanes[l]));
        ES_CUDA_CHECK(cudaStreamWaitEvent(stream, p->join_ev[l], 0));
    }
    if (stamps) launch_stamp(p->stamps_dev + 2 * p->ops.size() + 1, stream);
}

cudaGraphExec_t capture(es_b200_program* p, int mode, cudaGraph_t* graph_out)
{
    if (!p->capture_stream) ES_CUDA_CHECK(cudaStreamCreateWithFlags(&p->capture_stream, cudaStreamNonBlocking));
    ES_CUDA_CHECK(cudaStreamBeginCapture(p->capture_stream, cudaStreamCaptureModeThreadLocal));
    try {
        launch_all(p, p->capture_stream, mode);
    } catch (...) {
        cudaGraph_t broken = nullptr;
        cudaStreamEndCapture(p->capture_stream, &broken);
        if (broken) cudaGraphDestroy(broken);
        cudaGetLastError();
        throw;
    }
    ES_CUDA_CHECK(cudaStreamEndCapture(p->capture_stream, graph_out));
    cudaGraphExec_t exec = nullptr;
    ES_CUDA_CHECK(cudaGraphInstantiate(&exec, *graph_out, 0));
    return exec;
}

template <typename F> int guarded(F&& f)
{
    try {
        f();
        return ES_OK;
    } catch (es_error const& e) {
        set_last_error(e.what());
        return e.status;
    } catch (std::exception const& e) {
        set_last_error(e.what());
        return ES_BAD_ARGUMENT;
    } catch (...) {
        set_last_error("unknown exception");
        return ES_BAD_ARGUMENT;
    }
}

} // namespace

extern "C" {

int es_b200_program_create(es_b200_t* h, es_b200_program_t** out)
{
    return guarded([&] {
        if (!out) fail(ES_BAD_ARGUMENT, "null out pointer");
        auto* p = new es_b200_program;
        p->h = h;
        char const* pdl = std::getenv("ES_B200_PDL");
        p->pdl = !(pdl && std::string(pdl) == "0");
        *out = p;
    });
}

int es_b200_program_destroy(es_b200_program_t* p)
{
    return guarded([&] {
        if (!p) return;
        if (p->h) cudaSetDevice(p->h->device);
        free_device_side(p);
        delete p;
    });
}

int es_b200_program_add_einsummable(es_b200_program_t* p,
                                    uint64_t           kernel_id,
                                    void*              out,
                                    const void* const* inns,
                                    int                n_inn,
                                    const int*         deps,
                                    int                n_deps,
                                    int*               op_index)
{
    return guarded([&] {
        check_program(p, false);
        if (!out || n_inn < 0 || n_inn > ES_MAX_INNS || (n_inn && !inns))
            fail(ES_BAD_ARGUMENT, "program einsummable: bad pointers");
        op_t op;
        op.kind = OP_EINSUMMABLE;
        op.kernel_id = kernel_id;
        op.out = out;
        for (int i = 0; i != n_inn; ++i) {
            if (!inns[i]) fail(ES_BAD_ARGUMENT, "program einsummable: null input pointer");
            op.inns.push_back(inns[i]);
        }
        if (p->h) {
            std::lock_guard<std::mutex> lock(p->h->build_mutex);
            if (kernel_id >= p->h->kernels.size()) fail(ES_NOT_BUILT, "kernel id was never built");
            auto const& k = *p->h->kernels[kernel_id];
            if (n_inn != (int)k.e.inns.size()) fail(ES_BAD_ARGUMENT, "program einsummable: wrong number of inputs");
            op.ws_need = k.workspace_bytes;
        }
        add_op(p, std::move(op), deps, n_deps, op_index);
    });
}

int es_b200_program_add_touch(es_b200_program_t*   p,
                              const es_touchdim_t* dims,
                              int                  rank,
                              int                  castable,
                              int                  dtype,
                              void*                out,
                              const void*          inn,
                              const int*           deps,
                              int                  n_deps,
                              int*                 op_index)
{
    return guarded([&] {
        check_program(p, false);
        op_t op;
        op.kind = OP_TOUCH;
        op.dtype = dtype;
        op.touch_width = prepare_touch(dims, rank, castable, dtype, out, inn, op.touch);
        uint64_t n = dtype_size(dtype);
        for (int i = 0; i != rank; ++i) n *= dims[i].size;
        op.work_bytes = n * (castable == ES_CASTABLE_NONE ? 2 : 3);
        add_op(p, std::move(op), deps, n_deps, op_index);
    });
}

int es_b200_program_add_remote_touch(es_b200_program_t*   p,
                                     const es_touchdim_t* dims,
                                     int                  rank,
                                     int                  castable,
                                     int                  dtype,
                                     void*                out,
                                     const void*          inn_peer,
                                     void*                done_flag,
                                     const int*           deps,
                                     int                  n_deps,
                                     int*                 op_index)
{
    return guarded([&] {
        check_program(p, false);
        if (!done_flag || (reinterpret_cast<uintptr_t>(done_flag) & 3))
            fail(ES_BAD_ARGUMENT, "program remote touch: null or unaligned flag");
        op_t op;
        op.kind = OP_TOUCH;
        op.dtype = dtype;
        op.touch_width = prepare_touch(dims, rank, castable, dtype, out, inn_peer, op.touch);
        op.touch.done = static_cast<uint32_t*>(done_flag);
        uint64_t n = dtype_size(dtype);
        for (int i = 0; i != rank; ++i) n *= dims[i].size;
        op.work_bytes = n * (castable == ES_CASTABLE_NONE ? 2 : 3);
        add_op(p, std::move(op), deps, n_deps, op_index);
    });
}

int es_b200_program_add_fill_constant(es_b200_program_t* p,
                                      int                dtype,
                                      const void*        value8,
                                      uint64_t           nelem,
                                      void*              out,
                                      const int*         deps,
                                      int                n_deps,
                                      int*               op_index)
{
    return guarded([&] {
        check_program(p, false);
        if (!value8 || !out) fail(ES_BAD_ARGUMENT, "program fill: null pointer");
        op_t op;
        op.kind = OP_FILL_CONSTANT;
        op.dtype = dtype;
        std::memcpy(op.v0, value8, 8);
        op.nelem = nelem;
        op.out = out;
        op.work_bytes = nelem * dtype_size(dtype);
        add_op(p, std::move(op), deps, n_deps, op_index);
    });
}

int es_b200_program_add_fill_lowertri(es_b200_program_t* p,
                                      int                dtype,
                                      const void*        lower8,
                                      const void*        upper8,
                                      uint64_t           nrow,
                                      uint64_t           ncol,
                                      int64_t            start,
                                      void*              out,
                                      const int*         deps,
                                      int                n_deps,
                                      int*               op_index)
{
    return guarded([&] {
        check_program(p, false);
        if (!lower8 || !upper8 || !out) fail(ES_BAD_ARGUMENT, "program fill: null pointer");
        op_t op;
        op.kind = OP_FILL_LOWERTRI;
        op.dtype = dtype;
        std::memcpy(op.v0, lower8, 8);
        std::memcpy(op.v1, upper8, 8);
        op.nrow = nrow;
        op.ncol = ncol;
        op.start = start;
        op.out = out;
        op.work_bytes = nrow * ncol * dtype_size(dtype);
        add_op(p, std::move(op), deps, n_deps, op_index);
    });
}

int es_b200_program_add_copy(es_b200_program_t* p,
                             const void*        src,
                             void*              dst,
                             uint64_t           bytes,
                             const int*         deps,
                             int                n_deps,
                             int*               op_index)
{
    return guarded([&] {
        check_program(p, false);
        if (!src || !dst) fail(ES_BAD_ARGUMENT, "program copy: null pointer");
        op_t op;
        op.kind = OP_COPY;
        op.src = src;
        op.out = dst;
        op.bytes = bytes;
        add_op(p, std::move(op), deps, n_deps, op_index);
    });
}

int es_b200_program_add_attention(es_b200_program_t* p, const es_attention_t* a, void* out,
                                  const void* q, const void* k, const void* v, const void* mask,
                                  const int* deps, int n_deps, int* op_index)
{
    return guarded([&] {
        check_program(p, false);
        if (!a) fail(ES_BAD_ARGUMENT, "program attention: null descriptor");
        check_attention(*a, out, q, k, v, mask);
        op_t op;
        op.kind = OP_ATTENTION;
        op.attn = *a;
        op.out = out;
        op.inns = {q, k, v, mask};
        op.work_bytes = attention_bytes(*a);
        add_op(p, std::move(op), deps, n_deps, op_index);
    });
}

static int add_host_copy(es_b200_program_t* p, int kind, const void* src, void* dst, uint64_t bytes,
                         const int* deps, int n_deps, int* op_index)
{
    return guarded([&] {
        check_program(p, false);
        if (!src || !dst) fail(ES_BAD_ARGUMENT, "program evict / load: null pointer");
        op_t op;
        op.kind = kind;
        op.src = src;
        op.out = dst;
        op.bytes = bytes;
        op.work_bytes = bytes;
        add_op(p, std::move(op), deps, n_deps, op_index);
    });
}

int es_b200_program_add_evict(es_b200_program_t* p, const void* dev_src, void* host_dst, uint64_t bytes,
                              const int* deps, int n_deps, int* op_index)
{
    return add_host_copy(p, OP_EVICT, dev_src, host_dst, bytes, deps, n_deps, op_index);
}

int es_b200_program_add_load(es_b200_program_t* p, const void* host_src, void* dev_dst, uint64_t bytes,
                             const int* deps, int n_deps, int* op_index)
{
    return add_host_copy(p, OP_LOAD, host_src, dev_dst, bytes, deps, n_deps, op_index);
}

int es_b200_program_add_signal(es_b200_program_t* p,
                               void* const*       flags,
                               int                n,
                               const int*         deps,
                               int                n_deps,
                               int*               op_index)
{
    return guarded([&] {
        check_program(p, false);
        if (n <= 0 || !flags) fail(ES_BAD_ARGUMENT, "program signal: no flags");
        op_t op;
        op.kind = OP_SIGNAL;
        for (int i = 0; i != n; ++i) {
            if (!flags[i] || (reinterpret_cast<uintptr_t>(flags[i]) & 3))
                fail(ES_BAD_ARGUMENT, "program signal: null or unaligned flag");
            op.flags.push_back(static_cast<uint32_t*>(flags[i]));
        }
        add_op(p, std::move(op), deps, n_deps, op_index);
    });
}

int es_b200_program_add_wait(es_b200_program_t* p,
                             void* const*       flags,
                             int                n,
                             const int*         deps,
                             int                n_deps,
                             int*               op_index)
{
    return guarded([&] {
        check_program(p, false);
        if (n <= 0 || !flags) fail(ES_BAD_ARGUMENT, "program wait: no flags");
        op_t op;
        op.kind = OP_WAIT;
        for (int i = 0; i != n; ++i) {
            if (!flags[i] || (reinterpret_cast<uintptr_t>(flags[i]) & 3))
                fail(ES_BAD_ARGUMENT, "program wait: null or unaligned flag");
            op.flags.push_back(static_cast<uint32_t*>(flags[i]));
        }
        add_op(p, std::move(op), deps, n_deps, op_index);
    });
}

int es_b200_program_add_pull(es_b200_program_t*    p,
                             const es_pull_item_t* items,
                             int                   n,
                             const int*            deps,
                             int                   n_deps,
                             int*                  op_index)
{
    return guarded([&] {
        check_program(p, false);
        if (n <= 0 || !items) fail(ES_BAD_ARGUMENT, "program pull: no items");
        op_t op;
        op.kind = OP_PULL;
        op.max_ctas = 1;
        for (int i = 0; i != n; ++i) {
            es_pull_item_t const& it = items[i];
            if (!it.src || !it.dst || !it.done_flag) fail(ES_BAD_ARGUMENT, "program pull: null pointer");
            if ((reinterpret_cast<uintptr_t>(it.src) | reinterpret_cast<uintptr_t>(it.dst)) & 15)
                fail(ES_BAD_ARGUMENT, "program pull: source and destination must be 16-byte aligned");
            if ((reinterpret_cast<uintptr_t>(it.ready_flag) | reinterpret_cast<uintptr_t>(it.done_flag)) & 3)
                fail(ES_BAD_ARGUMENT, "program pull: unaligned flag");
            pull_item_t d;
            d.src = static_cast<char const*>(it.src);
            d.dst = static_cast<char*>(it.dst);
            d.bytes = it.bytes;
            d.ready = static_cast<uint32_t*>(it.ready_flag);
            d.done = static_cast<uint32_t*>(it.done_flag);
            d.n_ctas = pull_ctas_for(it.bytes);
            d.pad = 0;
            op.max_ctas = std::max(op.max_ctas, d.n_ctas);
            op.work_bytes += it.bytes;
            op.pulls.push_back(d);
        }
        add_op(p, std::move(op), deps, n_deps, op_index);
    });
}

int es_b200_program_add_touch_batch(es_b200_program_t*     p,
                                    const es_touch_item_t* items,
                                    int                    n,
                                    int                    dtype,
                                    const int*             deps,
                                    int                    n_deps,
                                    int*                   op_index)
{
    return guarded([&] {
        check_program(p, false);
        if (n <= 0 || !items) fail(ES_BAD_ARGUMENT, "program touch batch: no items");
        op_t op;
        op.kind = OP_TOUCH_BATCH;
        op.dtype = dtype;
        std::vector<int> widths(n);
        int              w = 16;
        op.batch.resize(n);
        for (int i = 0; i != n; ++i) {
            if (items[i].rank < 1 || items[i].rank > 4) fail(ES_BAD_DESCRIPTOR, "touch batch: rank");
            widths[i] = prepare_touch(items[i].dims, items[i].rank, items[i].castable, dtype, items[i].out,
                                      items[i].inn, op.batch[i]);
            w = std::min(w, widths[i]);
            uint64_t b = dtype_size(dtype);
            for (int d = 0; d != items[i].rank; ++d) b *= items[i].dims[d].size;
            op.work_bytes += b * (items[i].castable == ES_CASTABLE_NONE ? 2 : 3);
        }
        for (int i = 0; i != n; ++i) {
            narrow_touch(op.batch[i], widths[i], w);
            op.batch_slots = std::max(op.batch_slots, op.batch[i].total_slots);
        }
        op.touch_width = w;
        add_op(p, std::move(op), deps, n_deps, op_index);
    });
}

int es_b200_program_finalize(es_b200_program_t* p, int max_lanes, uint64_t* workspace_bytes)
{
    return guarded([&] {
        check_program(p, false);
        if (max_lanes <= 0) max_lanes = 8;
        if (max_lanes > 64) fail(ES_BAD_ARGUMENT, "program: at most 64 lanes");
        schedule(p, max_lanes);
        if (workspace_bytes) *workspace_bytes = p->ws_total;
        if (p->h) {
            ES_CUDA_CHECK(cudaSetDevice(p->h->device));
            upload(p);
            p->lanes.resize(p->n_lanes);
            for (auto& s : p->lanes) ES_CUDA_CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
            p->event_of.assign(p->ops.size(), -1);
            for (size_t i = 0; i != p->ops.size(); ++i) {
                if (!p->ops[i].record) continue;
                p->event_of[i] = (int)p->events.size();
                p->events.emplace_back();
                ES_CUDA_CHECK(cudaEventCreateWithFlags(&p->events.back(), cudaEventDisableTiming));
            }
            ES_CUDA_CHECK(cudaEventCreateWithFlags(&p->fork_ev, cudaEventDisableTiming));
            p->join_ev.resize(p->n_lanes);
            for (auto& e : p->join_ev) ES_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        }
        p->finalized = true;
    });
}

int es_b200_program_set_workspace(es_b200_program_t* p, void* workspace, uint64_t bytes)
{
    return guarded([&] {
        check_program(p, true);
        if (p->ws_total > 0) {
            if (!workspace || bytes < p->ws_total)
                fail(ES_WORKSPACE_TOO_SMALL, "program: workspace of " + std::to_string(p->ws_total) + " bytes required");
            if (reinterpret_cast<uintptr_t>(workspace) & 255)
                fail(ES_BAD_ARGUMENT, "program: workspace must be 256-byte aligned");
        }
        p->ws_base = static_cast<char*>(workspace);
        p->ws_bytes = bytes;
    });
}

int es_b200_program_set_exchange_lanes(es_b200_program_t* p, int lanes)
{
    return guarded([&] {
        check_program(p, false);
        if (lanes < 1 || lanes > 4) fail(ES_BAD_ARGUMENT, "program: 1 to 4 exchange lanes");
        p->exchange_lanes = lanes;
    });
}

int es_b200_program_set_wait_limit(es_b200_program_t* p, uint32_t limit_ms)
{
    return guarded([&] {
        if (!p) fail(ES_BAD_ARGUMENT, "null program");
        p->limit_ms = limit_ms;
    });
}

int es_b200_program_launch(es_b200_program_t* p, void* stream)
{
    return guarded([&] {
        check_program(p, true);
        launch_all(p, (cudaStream_t)stream, RUN_PLAIN);
    });
}

int es_b200_program_launch_timed(es_b200_program_t* p, void* stream, float* ms_per_op, int n)
{
    return guarded([&] {
        check_program(p, true);
        if (!ms_per_op || n < (int)p->ops.size()) fail(ES_BAD_ARGUMENT, "program: timing array too small");
        if (!p->h) fail(ES_BAD_ARGUMENT, "program: created without a device (planning only)");
        ES_CUDA_CHECK(cudaSetDevice(p->h->device));
        if (p->t0.empty()) {
            p->t0.resize(p->ops.size());
            p->t1.resize(p->ops.size());
            for (auto& e : p->t0) ES_CUDA_CHECK(cudaEventCreate(&e));
            for (auto& e : p->t1) ES_CUDA_CHECK(cudaEventCreate(&e));
        }
        launch_all(p, (cudaStream_t)stream, RUN_EVENTS);
        ES_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream));
        for (size_t i = 0; i != p->ops.size(); ++i)
            ES_CUDA_CHECK(cudaEventElapsedTime(&ms_per_op[i], p->t0[i], p->t1[i]));
    });
}

int es_b200_program_instantiate(es_b200_program_t* p)
{
    return guarded([&] {
        check_program(p, true);
        if (!p->h) fail(ES_BAD_ARGUMENT, "program: created without a device (planning only)");
        ES_CUDA_CHECK(cudaSetDevice(p->h->device));
        if (p->exec) {
            cudaGraphExecDestroy(p->exec);
            p->exec = nullptr;
        }
        if (p->graph) {
            cudaGraphDestroy(p->graph);
            p->graph = nullptr;
        }
        p->exec = capture(p, RUN_PLAIN, &p->graph);
    });
}

int es_b200_program_replay_timed(es_b200_program_t* p, void* stream, unsigned long long* ns, int n)
{
    return guarded([&] {
        check_program(p, true);
        if (!p->h) fail(ES_BAD_ARGUMENT, "program: created without a device (planning only)");
        int need = 2 * (int)p->ops.size() + 2;
        if (!ns || n < need) fail(ES_BAD_ARGUMENT, "program: time stamp array too small");
        ES_CUDA_CHECK(cudaSetDevice(p->h->device));
        if (!p->exec_timed) {
            ES_CUDA_CHECK(cudaMalloc(&p->stamps_dev, sizeof(unsigned long long) * need));
            ES_CUDA_CHECK(cudaMemset(p->stamps_dev, 0, sizeof(unsigned long long) * need));
            p->exec_timed = capture(p, RUN_STAMPS, &p->graph_timed);
        }
        ES_CUDA_CHECK(cudaGraphLaunch(p->exec_timed, (cudaStream_t)stream));
        ES_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream));
        ES_CUDA_CHECK(cudaMemcpy(ns, p->stamps_dev, sizeof(unsigned long long) * need, cudaMemcpyDeviceToHost));
    });
}

int es_b200_program_replay(es_b200_program_t* p, void* stream)
{
    return guarded([&] {
        check_program(p, true);
        if (!p->exec) fail(ES_BAD_ARGUMENT, "program: instantiate first");
        ES_CUDA_CHECK(cudaSetDevice(p->h->device));
        ES_CUDA_CHECK(cudaGraphLaunch(p->exec, (cudaStream_t)stream));
    });
}

int es_b200_program_reset_epoch(es_b200_program_t* p)
{
    return guarded([&] {
        check_program(p, true);
        if (!p->h) fail(ES_BAD_ARGUMENT, "program: created without a device (planning only)");
        ES_CUDA_CHECK(cudaSetDevice(p->h->device));
        ES_CUDA_CHECK(cudaDeviceSynchronize());
        ES_CUDA_CHECK(cudaMemset(p->epoch_dev, 0, sizeof(uint32_t)));
        ES_CUDA_CHECK(cudaDeviceSynchronize());
    });
}

int es_b200_program_describe(es_b200_program_t* p, char* buf, int buf_len, int* needed)
{
    return guarded([&] {
        check_program(p, true);
        std::ostringstream os;
        os << "{\"n_lanes\": " << p->n_lanes << ", \"n_exchange_lanes\": " << p->n_exchange << ", \"workspace_bytes\": " << p->ws_total << ", \"ops\": [";
        for (size_t i = 0; i != p->ops.size(); ++i) {
            op_t const& op = p->ops[i];
            os << (i ? ", " : "") << "{\"kind\": \"" << OP_NAMES[op.kind] << "\", \"lane\": " << op.lane
               << ", \"record\": " << (op.record ? "true" : "false") << ", \"deps\": [";
            for (size_t k = 0; k != op.deps.size(); ++k) os << (k ? "," : "") << op.deps[k];
            os << "], \"wait_on\": [";
            for (size_t k = 0; k != op.wait_on.size(); ++k) os << (k ? "," : "") << op.wait_on[k];
            os << "], \"bytes\": " << op.work_bytes << "}";
        }
        os << "]}";
        std::string s = os.str();
        if (needed) *needed = (int)s.size() + 1;
        if (!buf || buf_len < (int)s.size() + 1) {
            if (needed) return;
            fail(ES_BAD_ARGUMENT, "program describe: buffer too small");
        }
        std::memcpy(buf, s.c_str(), s.size() + 1);
    });
}

} // extern "C"
