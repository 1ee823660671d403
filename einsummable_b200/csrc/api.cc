// C ABI of the es_b200 library: handle, kernel cache, launch paths.
#include <cuda_runtime.h>

#include <atomic>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "codegen.h"
#include "common.h"
#include "contraction.h"
#include "einsum.h"
#include "jit.h"
#include "handle.h"
#include "kernels.h"
#include "attention.h"
#include "nvtx_ranges.h"
#include "exchange.h"
#include "pdl.h"

namespace es {

static thread_local std::string g_last_error;

void set_last_error(std::string const& msg)
{
    g_last_error = msg;
}

bool& pdl_launch_flag()
{
    static thread_local bool flag = false;
    return flag;
}

} // namespace es

namespace {

using namespace es;

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

void check_handle(es_b200* h)
{
    if (!h) fail(ES_BAD_ARGUMENT, "null handle");
}

void set_device(es_b200* h)
{
    // one host thread drives every GPU of the box, so each entry point selects
    // its device first (src/engine/gpu/gpu_kernel_manager.cc:592,985,1006,1097)
    ES_CUDA_CHECK(cudaSetDevice(h->device));
}

void load_functions(plan_t const& plan, std::shared_ptr<module_t>& mod, std::vector<void*>& fns)
{
    std::vector<char> cubin = nvrtc_compile(plan.source);
    mod = load_module(cubin);
    fns.clear();
    for (auto const& l : plan.launches) fns.push_back(mod->function(l.entry));
}

bool pointers_aligned(void* out, void const* const* inns, int n, int align)
{
    uintptr_t bits = reinterpret_cast<uintptr_t>(out);
    for (int i = 0; i != n; ++i) bits |= reinterpret_cast<uintptr_t>(inns[i]);
    return (bits & uintptr_t(align - 1)) == 0;
}

void copy_out(std::string const& s, char* buf, int buf_len)
{
    if (!buf || buf_len <= 0) fail(ES_BAD_ARGUMENT, "null output buffer");
    if ((int)s.size() + 1 > buf_len)
        fail(ES_BAD_ARGUMENT, "output buffer too small: need " + std::to_string(s.size() + 1));
    std::memcpy(buf, s.c_str(), s.size() + 1);
}

} // namespace

namespace es {

// A fallback plan may only run with the workspace the caller was told about.
static void check_fallback_workspace(plan_t const& plan, void* workspace, uint64_t workspace_bytes)
{
    if (plan.workspace_bytes == 0) return;
    if (!workspace || workspace_bytes < plan.workspace_bytes)
        fail(ES_WORKSPACE_TOO_SMALL, "einsummable launch: the kernel for these (unaligned) pointers needs " +
                                         std::to_string(plan.workspace_bytes) + " bytes of workspace");
}

void launch_built(es_b200*           h,
                  uint64_t           kernel_id,
                  cudaStream_t       stream,
                  void*              out,
                  void const* const* inns,
                  int                n_inn,
                  void*              workspace,
                  uint64_t           workspace_bytes)
{
    built_kernel_t* k = nullptr;
    {
        std::lock_guard<std::mutex> lock(h->build_mutex);
        if (kernel_id >= h->kernels.size()) fail(ES_NOT_BUILT, "kernel id was never built");
        k = h->kernels[kernel_id].get();
    }
    if (n_inn != (int)k->e.inns.size())
        fail(ES_BAD_ARGUMENT, "einsummable launch: wrong number of inputs");
    if (!out || !inns) fail(ES_BAD_ARGUMENT, "einsummable launch: null pointer");
    for (int i = 0; i != n_inn; ++i)
        if (!inns[i]) fail(ES_BAD_ARGUMENT, "einsummable launch: null input pointer");
    if (k->workspace_bytes > 0) {
        if (!workspace) fail(ES_WORKSPACE_TOO_SMALL, "einsummable launch: workspace required");
        if (workspace_bytes < k->workspace_bytes)
            fail(ES_WORKSPACE_TOO_SMALL,
                 "einsummable launch: workspace of " + std::to_string(workspace_bytes) +
                     " bytes, need " + std::to_string(k->workspace_bytes));
        if (reinterpret_cast<uintptr_t>(workspace) & 15)
            fail(ES_BAD_ARGUMENT, "einsummable launch: workspace must be 16-byte aligned");
    }
    set_device(h);
    nvtx_range_t range(nvtx_on() ? k->kind + " " + k->e.describe() : std::string());
    if (k->contraction && contraction_pointers_ok(inns[0], inns[1])) {
        launch_contraction(*k->contraction, stream, out, inns[0], inns[1], workspace);
        h->counters[0] += k->contraction->n_launches;
        h->work_bytes[0] += k->algorithmic_bytes;
        h->work_flops += k->algorithmic_flops;
        return;
    }
    if (k->contraction) {
        // operands not 16-byte aligned: TMA cannot address them; use the
        // generated SIMT kernel, built on first need
        std::lock_guard<std::mutex> lock(h->build_mutex);
        if (k->functions.empty()) {
            k->plan = plan_pointwise(k->e, false);
            load_functions(k->plan, k->module, k->functions);
        }
    }
    plan_t const*             plan = &k->plan;
    std::vector<void*> const* fns = &k->functions;
    if (plan->align > 1 && !pointers_aligned(out, inns, n_inn, plan->align)) {
        std::lock_guard<std::mutex> lock(h->build_mutex);
        if (!k->scalar_plan) {
            auto sp = std::make_unique<plan_t>(plan_pointwise(k->e, true));
            load_functions(*sp, k->scalar_module, k->scalar_functions);
            k->scalar_plan = std::move(sp);
        }
        plan = k->scalar_plan.get();
        fns = &k->scalar_functions;
    }
    if (plan != &k->plan || k->contraction) check_fallback_workspace(*plan, workspace, workspace_bytes);
    void* args[ES_MAX_INNS + 2];
    void* out_v = out;
    void* in_v[ES_MAX_INNS];
    void* ws_v = workspace;
    args[0] = &out_v;
    for (int i = 0; i != n_inn; ++i) {
        in_v[i] = const_cast<void*>(inns[i]);
        args[1 + i] = &in_v[i];
    }
    args[1 + n_inn] = &ws_v;
    for (size_t i = 0; i != plan->launches.size(); ++i) {
        launch_t const& l = plan->launches[i];
        launch_function((*fns)[i], l.grid, l.block, l.smem, stream, args);
    }
    h->counters[0] += plan->launches.size();
    h->work_bytes[0] += k->algorithmic_bytes;
    h->work_flops += k->algorithmic_flops;
}

} // namespace es

extern "C" {

const char* es_b200_last_error(void)
{
    return es::g_last_error.c_str();
}

const char* es_b200_version(void)
{
    return "es_b200 0.1 (sm_100a)";
}

int es_b200_create(int device, es_b200_t** out)
{
    return guarded([&] {
        if (!out) fail(ES_BAD_ARGUMENT, "null out pointer");
        *out = nullptr;
        int count = 0;
        ES_CUDA_CHECK(cudaGetDeviceCount(&count));
        if (device < 0 || device >= count)
            fail(ES_BAD_ARGUMENT, "device ordinal " + std::to_string(device) + " out of range");
        ES_CUDA_CHECK(cudaSetDevice(device));
        ES_CUDA_CHECK(cudaFree(nullptr));
        cudaDeviceProp prop;
        ES_CUDA_CHECK(cudaGetDeviceProperties(&prop, device));
        if (prop.major != 10)
            fail(ES_NOT_SUPPORTED, "es_b200 kernels are built for sm_100a only; device is sm_" +
                                       std::to_string(prop.major) + std::to_string(prop.minor));
        auto* h = new es_b200;
        h->device = device;
        for (auto& c : h->counters) c = 0;
        for (auto& c : h->work_bytes) c = 0;
        h->work_flops = 0;
        *out = h;
    });
}

int es_b200_destroy(es_b200_t* h)
{
    return guarded([&] {
        if (!h) return;
        cudaSetDevice(h->device);
        delete h;
    });
}

int es_b200_set_f32_policy(es_b200_t* h, int policy)
{
    return guarded([&] {
        check_handle(h);
        if (policy != ES_F32_3XTF32 && policy != ES_F32_TF32)
            fail(ES_BAD_ARGUMENT, "unknown f32 policy");
        h->f32_policy = policy;
    });
}

int es_b200_build_einsummable(es_b200_t*                   h,
                              const es_einsummable_desc_t* desc,
                              uint64_t*                    workspace_bytes,
                              uint64_t*                    kernel_id)
{
    return guarded([&] {
        check_handle(h);
        if (!kernel_id) fail(ES_BAD_ARGUMENT, "null kernel_id");
        einsum_t    e = einsum_t::from_desc(desc).merge_adjacent_dims();
        std::string key = e.key() + "|p" + std::to_string(h->f32_policy);
        std::lock_guard<std::mutex> lock(h->build_mutex);
        auto                        it = h->by_key.find(key);
        if (it != h->by_key.end()) {
            *kernel_id = it->second;
            if (workspace_bytes) *workspace_bytes = h->kernels[it->second]->workspace_bytes;
            return;
        }
        set_device(h);
        auto k = std::make_unique<built_kernel_t>();
        k->e = e;
        if (e.is_contraction()) {
            auto cp = std::make_unique<contraction_plan_t>();
            if (plan_contraction(e, h->f32_policy, *cp)) {
                k->kind = cp->kind;
                k->workspace_bytes = cp->workspace_bytes;
                for (auto const& pp : cp->pre_plans) {
                    cp->pre_modules.emplace_back();
                    cp->pre_functions.emplace_back();
                    load_functions(pp, cp->pre_modules.back(), cp->pre_functions.back());
                }
                k->contraction = std::move(cp);
                // unaligned operands run the generated SIMT kernel instead (built on first need);
                // its workspace must be part of what build reports
                k->workspace_bytes = std::max(k->workspace_bytes, plan_pointwise(e, false).workspace_bytes);
            }
        }
        if (!k->contraction) {
            k->plan = plan_pointwise(e, false);
            k->kind = k->plan.kind;
            k->workspace_bytes = k->plan.workspace_bytes;
            load_functions(k->plan, k->module, k->functions);
        }
        // the scalar twin (pointers below the vector alignment) may split differently
        k->workspace_bytes = std::max(k->workspace_bytes, plan_pointwise(e, true).workspace_bytes);
        k->algorithmic_bytes = e.algorithmic_bytes();
        k->algorithmic_flops = e.is_contraction() ? e.algorithmic_flops() : 0;
        uint64_t id = h->kernels.size();
        h->kernels.push_back(std::move(k));
        h->by_key[key] = id;
        *kernel_id = id;
        if (workspace_bytes) *workspace_bytes = h->kernels[id]->workspace_bytes;
    });
}

int es_b200_workspace_size(es_b200_t* h, uint64_t kernel_id, uint64_t* workspace_bytes)
{
    return guarded([&] {
        check_handle(h);
        if (!workspace_bytes) fail(ES_BAD_ARGUMENT, "null workspace_bytes");
        std::lock_guard<std::mutex> lock(h->build_mutex);
        if (kernel_id >= h->kernels.size()) fail(ES_NOT_BUILT, "kernel id was never built");
        *workspace_bytes = h->kernels[kernel_id]->workspace_bytes;
    });
}

int es_b200_launch_einsummable(es_b200_t*         h,
                               uint64_t           kernel_id,
                               void*              stream,
                               void*              out,
                               const void* const* inns,
                               int                n_inn,
                               void*              workspace,
                               uint64_t           workspace_bytes)
{
    return guarded([&] {
        check_handle(h);
        es::launch_built(h, kernel_id, (cudaStream_t)stream, out, inns, n_inn, workspace, workspace_bytes);
    });
}

int es_b200_launch_touch(es_b200_t*           h,
                         const es_touchdim_t* dims,
                         int                  rank,
                         int                  castable,
                         int                  dtype,
                         void*                stream,
                         void*                out,
                         const void*          inn)
{
    return guarded([&] {
        check_handle(h);
        touch_args_t a;
        int          w = prepare_touch(dims, rank, castable, dtype, out, inn, a);
        set_device(h);
        launch_touch(a, w, dtype, (cudaStream_t)stream);
        h->counters[1] += 1;
        uint64_t n = dtype_size(dtype);
        for (int i = 0; i != rank; ++i) n *= dims[i].size;
        h->work_bytes[1] += n * (castable == ES_CASTABLE_NONE ? 2 : 3);
    });
}

int es_b200_prepare_touch_batch(es_b200_t*             h,
                                const es_touch_item_t* items,
                                int                    n,
                                int                    dtype,
                                void*                  stream,
                                void*                  items_dev,
                                es_touch_batch_t*      prepared)
{
    return guarded([&] {
        check_handle(h);
        if (!prepared) fail(ES_BAD_ARGUMENT, "touch batch: null pointer");
        std::memset(prepared, 0, sizeof *prepared);
        if (n <= 0) return;
        if (!items || !items_dev) fail(ES_BAD_ARGUMENT, "touch batch: null pointer");
        static_assert(sizeof(touch_args_t) <= sizeof(es_touch_item_t),
                      "device staging buffer is sized by the public item struct");
        std::vector<touch_args_t> args(n);
        std::vector<int>          widths(n);
        int                       w = 16;
        for (int i = 0; i != n; ++i) {
            if (items[i].rank < 1 || items[i].rank > 4) fail(ES_BAD_DESCRIPTOR, "touch batch: rank");
            widths[i] = prepare_touch(items[i].dims, items[i].rank, items[i].castable, dtype,
                                      items[i].out, items[i].inn, args[i]);
            w = std::min(w, widths[i]);
        }
        uint64_t max_slots = 0;
        for (int i = 0; i != n; ++i) {
            narrow_touch(args[i], widths[i], w);
            max_slots = std::max(max_slots, args[i].total_slots);
        }
        set_device(h);
        // the host copy is consumed before cudaMemcpyAsync returns (pageable source)
        ES_CUDA_CHECK(cudaMemcpyAsync(items_dev, args.data(), sizeof(touch_args_t) * n,
                                      cudaMemcpyHostToDevice, (cudaStream_t)stream));
        prepared->n = n;
        prepared->dtype = dtype;
        prepared->width = w;
        prepared->max_slots = max_slots;
        prepared->items_dev = items_dev;
    });
}

int es_b200_launch_prepared_touch_batch(es_b200_t* h, const es_touch_batch_t* prepared, void* stream)
{
    return guarded([&] {
        check_handle(h);
        if (!prepared) fail(ES_BAD_ARGUMENT, "touch batch: null pointer");
        if (prepared->n <= 0) return;
        dtype_size(prepared->dtype);
        if (!prepared->items_dev) fail(ES_BAD_ARGUMENT, "touch batch: not prepared");
        set_device(h);
        launch_touch_batch(static_cast<touch_args_t const*>(prepared->items_dev), prepared->n,
                           prepared->max_slots, prepared->width, prepared->dtype, (cudaStream_t)stream);
        h->counters[1] += 1;
    });
}

int es_b200_launch_touch_batch(es_b200_t*             h,
                               const es_touch_item_t* items,
                               int                    n,
                               int                    dtype,
                               void*                  stream,
                               void*                  items_dev)
{
    es_touch_batch_t prepared;
    int              st = es_b200_prepare_touch_batch(h, items, n, dtype, stream, items_dev, &prepared);
    if (st != ES_OK) return st;
    return es_b200_launch_prepared_touch_batch(h, &prepared, stream);
}

int es_b200_fill_constant(
    es_b200_t* h, int dtype, const void* value8, uint64_t nelem, void* stream, void* out)
{
    return guarded([&] {
        check_handle(h);
        dtype_size(dtype);
        set_device(h);
        launch_fill_constant(dtype, value8, nelem, (cudaStream_t)stream, out);
        h->counters[2] += 1;
        h->work_bytes[2] += nelem * dtype_size(dtype);
    });
}

int es_b200_fill_lowertri(es_b200_t*  h,
                          int         dtype,
                          const void* lower8,
                          const void* upper8,
                          uint64_t    nrow,
                          uint64_t    ncol,
                          int64_t     start,
                          void*       stream,
                          void*       out)
{
    return guarded([&] {
        check_handle(h);
        dtype_size(dtype);
        set_device(h);
        launch_fill_lowertri(dtype, lower8, upper8, nrow, ncol, start, (cudaStream_t)stream, out);
        h->counters[2] += 1;
        h->work_bytes[2] += nrow * ncol * dtype_size(dtype);
    });
}

int es_b200_move(es_b200_t*  h,
                 int         src_device,
                 const void* src,
                 int         dst_device,
                 void*       dst,
                 uint64_t    bytes,
                 void*       stream)
{
    return guarded([&] {
        check_handle(h);
        if (dst_device != h->device)
            fail(ES_BAD_ARGUMENT, "move: the handle must belong to the destination device");
        if (bytes == 0) return;
        if (!src || !dst) fail(ES_BAD_ARGUMENT, "move: null pointer");
        set_device(h);
        if (src_device != dst_device) {
            // peer mapping of the source GPU's memory into this device's address space, once per
            // pair (the reference's server enables all pairs at start-up, src/server/gpu/server.cc:54-80)
            static std::mutex           peer_mutex;
            static bool                 enabled[64][64] = {};
            std::lock_guard<std::mutex> lock(peer_mutex);
            if (src_device < 0 || src_device >= 64 || dst_device >= 64)
                fail(ES_BAD_ARGUMENT, "move: device ordinal out of range");
            if (!enabled[dst_device][src_device]) {
                int can = 0;
                ES_CUDA_CHECK(cudaDeviceCanAccessPeer(&can, dst_device, src_device));
                if (!can) fail(ES_NOT_SUPPORTED, "move: no peer access between the two GPUs");
                cudaError_t e = cudaDeviceEnablePeerAccess(src_device, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
                else if (e != cudaSuccess) fail(ES_CUDA_ERROR, std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(e));
                enabled[dst_device][src_device] = true;
            }
        }
        // Small or latency-critical blobs: SM pull kernel on the destination GPU
        // reading the peer-mapped source with 128-bit loads.  Large blobs: the
        // copy engine, which leaves the SMs to the compute kernels.
        bool aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
        if (aligned && bytes <= (4ull << 20)) {
            launch_pull_copy(src, dst, bytes, (cudaStream_t)stream);
        } else if (src_device == dst_device) {
            ES_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice,
                                          (cudaStream_t)stream));
        } else {
            ES_CUDA_CHECK(cudaMemcpyPeerAsync(dst, dst_device, src, src_device, bytes,
                                              (cudaStream_t)stream));
        }
        h->counters[3] += 1;
        h->work_bytes[3] += bytes;
    });
}

int es_b200_kernel_info(es_b200_t* h, uint64_t kernel_id, char* buf, int buf_len)
{
    return guarded([&] {
        check_handle(h);
        std::lock_guard<std::mutex> lock(h->build_mutex);
        if (kernel_id >= h->kernels.size()) fail(ES_NOT_BUILT, "kernel id was never built");
        auto const& k = *h->kernels[kernel_id];
        std::string s = k.kind + "|" + k.e.describe() + "|vec=" + std::to_string(k.plan.vec) +
                        "|ws=" + std::to_string(k.workspace_bytes);
        if (k.contraction) s += "|" + k.contraction->info;
        copy_out(s, buf, buf_len);
    });
}

int es_b200_describe(const es_einsummable_desc_t* desc, int what, char* buf, int buf_len)
{
    return guarded([&] {
        einsum_t e = einsum_t::from_desc(desc).merge_adjacent_dims();
        if (what == 0) {
            copy_out(e.describe(), buf, buf_len);
            return;
        }
        contraction_plan_t cp;
        bool               tc = e.is_contraction() && plan_contraction(e, ES_F32_3XTF32, cp);
        if (what == 1) {
            copy_out(tc ? cp.kind : plan_pointwise(e, false).kind, buf, buf_len);
        } else if (what == 2) {
            copy_out(tc ? std::string() : plan_pointwise(e, false).source, buf, buf_len);
        } else if (what == 3) {
            std::string log;
            if (!tc) {
                nvrtc_compile(plan_pointwise(e, false).source, &log);
                std::string log2;
                nvrtc_compile(plan_pointwise(e, true).source, &log2);
                log += log2;
            }
            copy_out(log, buf, buf_len);
        } else if (what == 4) {
            copy_out(tc ? cp.info : std::string(), buf, buf_len);
        } else if (what == 5) {
            // compile as build() does: through the on-disk kernel cache
            copy_out(tc ? std::string() : "cubin bytes=" + std::to_string(nvrtc_compile(plan_pointwise(e, false).source).size()),
                     buf, buf_len);
        } else {
            fail(ES_BAD_ARGUMENT, "describe: unknown selector");
        }
    });
}

int es_b200_touch_simplify(const es_touchdim_t* dims, int rank, es_touchdim_t* dims_out, int* out_rank)
{
    return guarded([&] {
        if (!dims || !dims_out || !out_rank) fail(ES_BAD_ARGUMENT, "null pointer");
        if (rank < 1 || rank > 16) fail(ES_BAD_DESCRIPTOR, "touch: bad rank");
        es_touchdim_t tmp[16];
        int           r = simplify_touch(dims, rank, tmp);
        std::memcpy(dims_out, tmp, sizeof(es_touchdim_t) * r);
        *out_rank = r;
    });
}

int es_b200_device_status(es_b200_t* h, unsigned int* error_word)
{
    return guarded([&] {
        check_handle(h);
        if (!error_word) fail(ES_BAD_ARGUMENT, "null pointer");
        set_device(h);
        ES_CUDA_CHECK(cudaDeviceSynchronize());
        unsigned int tc = read_and_clear_tc_error();
        unsigned int at = read_and_clear_attention_error();
        if (!tc) tc = at;
        unsigned int fl = read_and_clear_flag_error();
        unsigned int ex = read_and_clear_exchange_error();
        *error_word = tc | ((fl ? fl : ex) << 8);
    });
}

int es_b200_debug_trace(es_b200_t* h, unsigned long long* out, int n, int* n_out)
{
    return guarded([&] {
        check_handle(h);
        if (!out || !n_out || n < 0) fail(ES_BAD_ARGUMENT, "null pointer or negative count");
        set_device(h);
        int got = read_trace(out, n);
        if (got < 0) fail(ES_NOT_SUPPORTED, "this library was built without ES_B200_TRACE");
        // entries 8000.. : the attention kernel's samples
        if (n > 8000 && got == 8000) got += read_attention_trace(out + 8000, n - 8000);
        *n_out = got;
    });
}

int es_b200_flag_signal(es_b200_t* h, void* flag, uint32_t limit_ms, void* stream)
{
    return guarded([&] {
        check_handle(h);
        set_device(h);
        launch_flag_signal(static_cast<uint32_t*>(flag), limit_ms, (cudaStream_t)stream);
        h->counters[3] += 1;
    });
}

int es_b200_flag_wait(es_b200_t* h, void* flag, uint32_t limit_ms, void* stream)
{
    return guarded([&] {
        check_handle(h);
        set_device(h);
        launch_flag_wait(static_cast<uint32_t*>(flag), limit_ms, (cudaStream_t)stream);
        h->counters[3] += 1;
    });
}

int es_b200_pull(es_b200_t* h, const void* src, void* dst, uint64_t bytes, void* stream)
{
    return guarded([&] {
        check_handle(h);
        if (bytes == 0) return;
        if (!src || !dst) fail(ES_BAD_ARGUMENT, "pull: null pointer");
        set_device(h);
        launch_pull_copy(src, dst, bytes, (cudaStream_t)stream);
        h->counters[3] += 1;
        h->work_bytes[3] += bytes;
    });
}

int es_b200_launch_attention(es_b200_t* h, const es_attention_t* a, void* stream, void* out,
                             const void* q, const void* k, const void* v, const void* mask)
{
    return guarded([&] {
        check_handle(h);
        if (!a) fail(ES_BAD_ARGUMENT, "attention: null descriptor");
        set_device(h);
        nvtx_range_t range("attention_tc_f16");
        launch_attention(*a, (cudaStream_t)stream, out, q, k, v, mask);
        h->counters[0] += 1;
        h->work_bytes[0] += attention_bytes(*a);
        h->work_flops += attention_flops(*a);
    });
}

int es_b200_query_counters(es_b200_t* h, uint64_t launches[4])
{
    return guarded([&] {
        check_handle(h);
        if (!launches) fail(ES_BAD_ARGUMENT, "null pointer");
        for (int i = 0; i != 4; ++i) launches[i] = h->counters[i];
    });
}

int es_b200_query_work(es_b200_t* h, uint64_t bytes[4], uint64_t* contraction_flops)
{
    return guarded([&] {
        check_handle(h);
        if (!bytes || !contraction_flops) fail(ES_BAD_ARGUMENT, "null pointer");
        for (int i = 0; i != 4; ++i) bytes[i] = h->work_bytes[i];
        *contraction_flops = h->work_flops;
    });
}

} // extern "C"
