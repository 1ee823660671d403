// kernel_manager_t over the es_b200 C ABI; see gpu_kernel_manager.h.
#include "gpu_kernel_manager.h"

#include <cstring>

namespace {

[[noreturn]] void throw_status(char const* what, int status)
{
    // the reference throws std::runtime_error from handle_cuda_error & co
    // (src/engine/gpu/utility.cc:114-143)
    throw std::runtime_error(string(what) + ": es_b200 status " + std::to_string(status) + ": " +
                             es_b200_last_error());
}

int dtype_code(dtype_t d)
{
    // dtype_t { f16, f32, f64, c64 } (src/einsummable/scalarop.h:10) == es_dtype_t
    return int(d);
}

int castable_code(optional<castable_t> const& c)
{
    // castable_t { add, mul, min, max } (src/einsummable/scalarop.h:4) == es_castable_t
    return c ? int(c.value()) : ES_CASTABLE_NONE;
}

struct desc_holder_t {
    es_einsummable_desc_t desc;
    string                join_text;
};

void fill_desc(einsummable_t const& e, desc_holder_t& h)
{
    if (e.join_shape.size() > ES_MAX_RANK || e.inns.size() > ES_MAX_INNS) {
        throw std::runtime_error("kernel_manager_t: einsummable exceeds ES_MAX_RANK / ES_MAX_INNS");
    }
    std::memset(&h.desc, 0, sizeof h.desc);
    h.desc.join_rank = int(e.join_shape.size());
    for (size_t i = 0; i != e.join_shape.size(); ++i) {
        h.desc.join_shape[i] = e.join_shape[i];
    }
    h.desc.n_inn = int(e.inns.size());
    for (size_t k = 0; k != e.inns.size(); ++k) {
        h.desc.inn_rank[k] = int(e.inns[k].size());
        for (size_t j = 0; j != e.inns[k].size(); ++j) {
            h.desc.inn_modes[k][j] = e.inns[k][j];
        }
    }
    h.desc.out_rank = e.out_rank;
    h.desc.castable = castable_code(e.castable);
    h.join_text = write_with_ss(e.join); // operator<< text form, src/einsummable/scalarop.cc:2995-3011
    h.desc.join = h.join_text.c_str();
}

} // namespace

kernel_manager_t::kernel_manager_t() : kernel_manager_t(0) {}

kernel_manager_t::kernel_manager_t(int device) : device(device), handle(nullptr)
{
    int status = es_b200_create(device, &handle);
    if (status != ES_OK) {
        throw_status("kernel_manager_t", status);
    }
}

kernel_manager_t::kernel_manager_t(kernel_manager_t&& other) noexcept
    : device(other.device), handle(other.handle), kernels(std::move(other.kernels))
{
    other.handle = nullptr;
}

kernel_manager_t::~kernel_manager_t()
{
    if (handle) {
        es_b200_destroy(handle);
    }
}

optional<workspace_info_t> kernel_manager_t::build(einsummable_t const& e_)
{
    einsummable_t e = e_.merge_adjacent_dims();
    auto          iter = kernels.find(e);
    if (iter != kernels.end()) {
        return workspace_info_t(iter->second.workspace_size);
    }
    desc_holder_t h;
    fill_desc(e, h);
    uint64_t ws = 0, id = 0;
    int      status = es_b200_build_einsummable(handle, &h.desc, &ws, &id);
    if (status == ES_NOT_SUPPORTED) {
        return std::nullopt;
    }
    if (status != ES_OK) {
        throw_status("kernel_manager_t::build", status);
    }
    kernels.insert({e, built_t{.kernel_id = id, .workspace_size = ws}});
    return workspace_info_t(ws);
}

workspace_info_t kernel_manager_t::workspace_size(einsummable_t const& e) const
{
    return workspace_info_t(get_built_kernel_info(e).workspace_size);
}

kernel_manager_t::built_t const& kernel_manager_t::get_built_kernel_info(einsummable_t const& e) const
{
    auto iter = kernels.find(e.merge_adjacent_dims());
    if (iter == kernels.end()) {
        throw std::runtime_error("get_built_kernel_info: this einsummable was not built");
    }
    return iter->second;
}

void kernel_manager_t::operator()(einsummable_t const&             e,
                                  cudaStream_t                     stream,
                                  void*                            out,
                                  vector<void const*>              inns,
                                  optional<tuple<void*, uint64_t>> workspace) const
{
    built_t const& info = get_built_kernel_info(e);
    void*          ws = nullptr;
    uint64_t       ws_size = 0;
    if (workspace) {
        ws = std::get<0>(workspace.value());
        ws_size = std::get<1>(workspace.value());
    }
    int status = es_b200_launch_einsummable(
        handle, info.kernel_id, stream, out, inns.data(), int(inns.size()), ws, ws_size);
    if (status != ES_OK) {
        throw_status("kernel_manager_t::operator()(einsummable_t)", status);
    }
}

void kernel_manager_t::attention(es_attention_t const& a,
                                 cudaStream_t          stream,
                                 void*                 out,
                                 void const*           q,
                                 void const*           k,
                                 void const*           v,
                                 void const*           mask) const
{
    int status = es_b200_launch_attention(handle, &a, stream, out, q, k, v, mask);
    if (status != ES_OK) {
        throw_status("kernel_manager_t::attention", status);
    }
}

void kernel_manager_t::operator()(touch_t const& touch,
                                  cudaStream_t   stream,
                                  void*          out,
                                  void const*    inn) const
{
    vector<es_touchdim_t> dims;
    dims.reserve(touch.selection.size());
    for (touchdim_t const& t : touch.selection) {
        dims.push_back(es_touchdim_t{t.d_inn, t.d_out, t.offset_inn, t.offset_out, t.size});
    }
    int status = es_b200_launch_touch(handle,
                                      dims.data(),
                                      int(dims.size()),
                                      castable_code(touch.castable),
                                      dtype_code(touch.dtype),
                                      stream,
                                      out,
                                      inn);
    if (status != ES_OK) {
        throw_status("kernel_manager_t::operator()(touch_t)", status);
    }
}

void kernel_manager_t::lowerTri_fill(fill_t::lowertri_t const& l,
                                     cudaStream_t              stream,
                                     void*                     out) const
{
    int status = es_b200_fill_lowertri(handle,
                                       dtype_code(l.lower.dtype),
                                       l.lower.raw(),
                                       l.upper.raw(),
                                       l.nrow,
                                       l.ncol,
                                       l.start,
                                       stream,
                                       out);
    if (status != ES_OK) {
        throw_status("kernel_manager_t::lowerTri_fill", status);
    }
}

void kernel_manager_t::constant_fill(fill_t::constant_t const& c,
                                     cudaStream_t              stream,
                                     void*                     out) const
{
    int status = es_b200_fill_constant(
        handle, dtype_code(c.value.dtype), c.value.raw(), product(c.shape), stream, out);
    if (status != ES_OK) {
        throw_status("kernel_manager_t::constant_fill", status);
    }
}

void kernel_manager_t::move(
    int src_device, void const* src, void* dst, uint64_t size, cudaStream_t stream) const
{
    int status = es_b200_move(handle, src_device, src, device, dst, size, stream);
    if (status != ES_OK) {
        throw_status("kernel_manager_t::move", status);
    }
}
