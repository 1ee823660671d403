// Test infrastructure, not product code.
//
// A recording stand-in for the part of the es_b200 C ABI that the C++ host code calls
// (einsummable_b200/host/gpu_kernel_manager.cc, gpu_program.cc), for checking on a machine without
// a GPU WHAT that code asks the library to do: every op a program is given -- its pointers, flags,
// touch dimensions, dependencies -- is written down and can be dumped as JSON (mock_dump_ops).
// Nothing is launched; launch / replay entries fail.  Linked INSTEAD of libes_b200.so into
// oracle/_ref/exchange_ops only.
#include "es_b200.h"

#include <cstdint>
#include <cstring>
#include <map>
#include <sstream>
#include <string>
#include <vector>

namespace {

struct kernel_t {
    std::string join;
    int         n_inn;
};
std::vector<kernel_t> g_kernels;
std::ostringstream    g_ops; // the ops of the program being filled, as JSON objects
int                   g_n_ops = 0;

std::string u64(void const* p)
{
    return std::to_string(static_cast<unsigned long long>(reinterpret_cast<uintptr_t>(p)));
}

void begin(char const* kind, int const* deps, int n_deps)
{
    g_ops << (g_n_ops ? ",\n" : "") << "{\"kind\":\"" << kind << "\",\"deps\":[";
    for (int i = 0; i != n_deps; ++i) g_ops << (i ? "," : "") << deps[i];
    g_ops << "]";
}

int end(int* op_index)
{
    g_ops << "}";
    if (op_index) *op_index = g_n_ops;
    g_n_ops++;
    return ES_OK;
}

void dims_json(es_touchdim_t const* dims, int rank)
{
    g_ops << ",\"dims\":[";
    for (int i = 0; i != rank; ++i) {
        g_ops << (i ? "," : "") << "[" << dims[i].d_inn << "," << dims[i].d_out << "," << dims[i].offset_inn << ","
              << dims[i].offset_out << "," << dims[i].size << "]";
    }
    g_ops << "]";
}

void flags_json(void* const* flags, int n)
{
    g_ops << ",\"flags\":[";
    for (int i = 0; i != n; ++i) g_ops << (i ? "," : "") << u64(flags[i]);
    g_ops << "]";
}

} // namespace

// the ops recorded since the last call, as the inside of a JSON array; the record is cleared
std::string mock_take_ops()
{
    std::string s = g_ops.str();
    g_ops.str("");
    g_ops.clear();
    g_n_ops = 0;
    return s;
}

extern "C" {

struct es_b200 {
    int device;
};
struct es_b200_program {
    int unused;
};

const char* es_b200_last_error(void)
{
    return "mock";
}
int es_b200_create(int device, es_b200_t** out)
{
    *out = new es_b200{device};
    return ES_OK;
}
int es_b200_destroy(es_b200_t* h)
{
    delete h;
    return ES_OK;
}
int es_b200_build_einsummable(es_b200_t*, const es_einsummable_desc_t* d, uint64_t* workspace_bytes, uint64_t* kernel_id)
{
    g_kernels.push_back({d->join, d->n_inn});
    *workspace_bytes = 0;
    *kernel_id = g_kernels.size() - 1;
    return ES_OK;
}
int es_b200_program_create(es_b200_t*, es_b200_program_t** out)
{
    *out = new es_b200_program{0};
    return ES_OK;
}
int es_b200_program_destroy(es_b200_program_t* p)
{
    delete p;
    return ES_OK;
}
int es_b200_program_add_einsummable(es_b200_program_t*, uint64_t kernel_id, void* out, const void* const* inns, int n_inn,
                                    const int* deps, int n_deps, int* op_index)
{
    begin("einsummable", deps, n_deps);
    kernel_t const& k = g_kernels.at(kernel_id);
    g_ops << ",\"join\":\"" << k.join << "\",\"built_inns\":" << k.n_inn << ",\"out\":" << u64(out) << ",\"inns\":[";
    for (int i = 0; i != n_inn; ++i) g_ops << (i ? "," : "") << u64(inns[i]);
    g_ops << "]";
    return end(op_index);
}
int es_b200_program_add_touch(es_b200_program_t*, const es_touchdim_t* dims, int rank, int castable, int dtype, void* out,
                              const void* inn, const int* deps, int n_deps, int* op_index)
{
    begin("touch", deps, n_deps);
    dims_json(dims, rank);
    g_ops << ",\"castable\":" << castable << ",\"dtype\":" << dtype << ",\"out\":" << u64(out) << ",\"inn\":" << u64(inn);
    return end(op_index);
}
int es_b200_program_add_remote_touch(es_b200_program_t*, const es_touchdim_t* dims, int rank, int castable, int dtype,
                                     void* out, const void* inn_peer, void* done_flag, const int* deps, int n_deps,
                                     int* op_index)
{
    begin("rtouch", deps, n_deps);
    dims_json(dims, rank);
    g_ops << ",\"castable\":" << castable << ",\"dtype\":" << dtype << ",\"out\":" << u64(out) << ",\"inn\":" << u64(inn_peer)
          << ",\"done_flag\":" << u64(done_flag);
    return end(op_index);
}
int es_b200_program_add_fill_constant(es_b200_program_t*, int dtype, const void*, uint64_t nelem, void* out, const int* deps,
                                      int n_deps, int* op_index)
{
    begin("fill_constant", deps, n_deps);
    g_ops << ",\"dtype\":" << dtype << ",\"nelem\":" << nelem << ",\"out\":" << u64(out);
    return end(op_index);
}
int es_b200_program_add_fill_lowertri(es_b200_program_t*, int dtype, const void*, const void*, uint64_t nrow, uint64_t ncol,
                                      int64_t start, void* out, const int* deps, int n_deps, int* op_index)
{
    begin("fill_lowertri", deps, n_deps);
    g_ops << ",\"dtype\":" << dtype << ",\"nrow\":" << nrow << ",\"ncol\":" << ncol << ",\"start\":" << start
          << ",\"out\":" << u64(out);
    return end(op_index);
}
int es_b200_program_add_copy(es_b200_program_t*, const void* src, void* dst, uint64_t bytes, const int* deps, int n_deps,
                             int* op_index)
{
    begin("copy", deps, n_deps);
    g_ops << ",\"src\":" << u64(src) << ",\"dst\":" << u64(dst) << ",\"bytes\":" << bytes;
    return end(op_index);
}
int es_b200_program_add_attention(es_b200_program_t*, const es_attention_t* a, void* out, const void* q, const void* k,
                                  const void* v, const void* mask, const int* deps, int n_deps, int* op_index)
{
    begin("attention", deps, n_deps);
    g_ops << ",\"shape\":[" << a->batch << "," << a->heads << "," << a->rows << "," << a->keys << "," << a->head_dim
          << "],\"skip_known\":" << a->skip_known << ",\"skip_from\":" << a->skip_from << ",\"q_stride\":[" << a->q_stride[0]
          << "," << a->q_stride[1] << "," << a->q_stride[2] << "],\"out\":" << u64(out) << ",\"q\":" << u64(q)
          << ",\"k\":" << u64(k) << ",\"v\":" << u64(v) << ",\"mask\":" << u64(mask);
    return end(op_index);
}
int es_b200_program_add_signal(es_b200_program_t*, void* const* flags, int n, const int* deps, int n_deps, int* op_index)
{
    begin("signal", deps, n_deps);
    flags_json(flags, n);
    return end(op_index);
}
int es_b200_program_add_wait(es_b200_program_t*, void* const* flags, int n, const int* deps, int n_deps, int* op_index)
{
    begin("wait", deps, n_deps);
    flags_json(flags, n);
    return end(op_index);
}
int es_b200_program_add_pull(es_b200_program_t*, const es_pull_item_t* items, int n, const int* deps, int n_deps, int* op_index)
{
    begin("pull", deps, n_deps);
    g_ops << ",\"items\":[";
    for (int i = 0; i != n; ++i) {
        g_ops << (i ? "," : "") << "[" << u64(items[i].src) << "," << u64(items[i].dst) << "," << items[i].bytes << ","
              << u64(items[i].ready_flag) << "," << u64(items[i].done_flag) << "]";
    }
    g_ops << "]";
    return end(op_index);
}
int es_b200_program_add_evict(es_b200_program_t*, const void* dev_src, void* host_dst, uint64_t bytes, const int* deps,
                              int n_deps, int* op_index)
{
    begin("evict", deps, n_deps);
    g_ops << ",\"dev\":" << u64(dev_src) << ",\"host\":" << u64(host_dst) << ",\"bytes\":" << bytes;
    return end(op_index);
}
int es_b200_program_add_load(es_b200_program_t*, const void* host_src, void* dev_dst, uint64_t bytes, const int* deps,
                             int n_deps, int* op_index)
{
    begin("load", deps, n_deps);
    g_ops << ",\"dev\":" << u64(dev_dst) << ",\"host\":" << u64(host_src) << ",\"bytes\":" << bytes;
    return end(op_index);
}
int es_b200_program_set_wait_limit(es_b200_program_t*, uint32_t)
{
    return ES_OK;
}
int es_b200_program_finalize(es_b200_program_t*, int, uint64_t* workspace_bytes)
{
    *workspace_bytes = 0;
    return ES_OK;
}
int es_b200_program_set_workspace(es_b200_program_t*, void*, uint64_t)
{
    return ES_OK;
}
int es_b200_program_launch(es_b200_program_t*, void*)
{
    return ES_NOT_SUPPORTED;
}
int es_b200_program_instantiate(es_b200_program_t*)
{
    return ES_NOT_SUPPORTED;
}
int es_b200_program_replay(es_b200_program_t*, void*)
{
    return ES_NOT_SUPPORTED;
}
/* the launch entries of the kernel manager: never reached by the program builders */
int es_b200_launch_einsummable(es_b200_t*, uint64_t, void*, void*, const void* const*, int, void*, uint64_t)
{
    return ES_NOT_SUPPORTED;
}
int es_b200_launch_touch(es_b200_t*, const es_touchdim_t*, int, int, int, void*, void*, const void*)
{
    return ES_NOT_SUPPORTED;
}
int es_b200_fill_constant(es_b200_t*, int, const void*, uint64_t, void*, void*)
{
    return ES_NOT_SUPPORTED;
}
int es_b200_fill_lowertri(es_b200_t*, int, const void*, const void*, uint64_t, uint64_t, int64_t, void*, void*)
{
    return ES_NOT_SUPPORTED;
}
int es_b200_move(es_b200_t*, int, const void*, int, void*, uint64_t, void*)
{
    return ES_NOT_SUPPORTED;
}
int es_b200_launch_attention(es_b200_t*, const es_attention_t*, void*, void*, const void*, const void*, const void*, const void*)
{
    return ES_NOT_SUPPORTED;
}

} // extern "C"
