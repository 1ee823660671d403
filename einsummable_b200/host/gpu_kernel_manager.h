// Drop-in replacement for the reference's src/engine/gpu/gpu_kernel_manager.h.
//
// Same public surface as the reference's kernel_manager_t
// (src/engine/gpu/gpu_kernel_manager.h:274-321): build / workspace_size /
// operator()(einsummable_t) / operator()(touch_t) / lowerTri_fill /
// constant_fill, plus workspace_info_t.  The exec nodes
// (src/engine/gpu/exec_graph.cc:131-158,277-404,600-701) and the GPU server
// (src/server/gpu/server.cc:39-43) compile against it unchanged.  All work is
// forwarded to the C ABI of libes_b200.so; no cuBLAS / cuTENSOR is involved.
//
// Place this file and gpu_kernel_manager.cc in src/engine/gpu/, in place of the reference's two files of
// the same names, and link libes_b200.so instead of cuTENSOR / cuBLAS.
#pragma once
#include "../../base/setup.h"

#include "../../einsummable/einsummable.h"
#include "../../einsummable/fill.h"
#include "../../einsummable/touch.h"

#include <cuda_runtime.h>

#include <unordered_map>

#include "es_b200.h"

struct workspace_info_t {
    workspace_info_t() {}
    workspace_info_t(uint64_t sz) : workspace_size(sz) {}

    optional<uint64_t> workspace_size;

    uint64_t const& value() const
    {
        return workspace_size.value();
    }

    bool known() const
    {
        return bool(workspace_size);
    }
};

struct kernel_manager_t {
    kernel_manager_t();
    kernel_manager_t(int device);
    ~kernel_manager_t();

    kernel_manager_t(kernel_manager_t const&) = delete;
    kernel_manager_t& operator=(kernel_manager_t const&) = delete;
    kernel_manager_t(kernel_manager_t&& other) noexcept;

    // nullopt = this einsummable cannot be run (the reference's contract,
    // src/engine/gpu/gpu_kernel_manager.cc:590-958)
    optional<workspace_info_t> build(einsummable_t const& e);

    workspace_info_t workspace_size(einsummable_t const& e) const;

    void operator()(touch_t const& touch, cudaStream_t stream, void* out, void const* inn) const;

    void operator()(einsummable_t const&             e,
                    cudaStream_t                     stream,
                    void*                            out,
                    vector<void const*>              inns,
                    optional<tuple<void*, uint64_t>> workspace = std::nullopt) const;

    void lowerTri_fill(fill_t::lowertri_t const& l, cudaStream_t stream, void* out) const;
    void constant_fill(fill_t::constant_t const& c, cudaStream_t stream, void* out) const;

    // gpu_copy_t::launch (src/engine/gpu/exec_graph.cc:406-467) re-pointed here:
    // copy `size` bytes from (src_device, src) into dst on this manager's device.
    void move(int src_device, void const* src, void* dst, uint64_t size, cudaStream_t stream) const;

    // An extension without a counterpart in the reference's manager: softmax(Q K^T + mask) V, the five
    // apply nodes the graph writer emits for attention (src/einsummable/gwriter.cc:830-855,
    // llama/modules.cc:285-383), as one launch.  A caller that finds the chain in its memgraph passes the
    // shapes and strides here; see es_attention_t in es_b200.h.
    void attention(es_attention_t const& a,
                   cudaStream_t          stream,
                   void*                 out,
                   void const*           q,
                   void const*           k,
                   void const*           v,
                   void const*           mask) const;

    // For callers that hand built kernels to the library's program executor (gpu_program.h): the
    // library handle of this device and the id build() gave the (merged) einsummable.
    es_b200_t* c_handle() const
    {
        return handle;
    }
    uint64_t kernel_id(einsummable_t const& e) const
    {
        return get_built_kernel_info(e).kernel_id;
    }

private:
    struct built_t {
        uint64_t kernel_id;
        uint64_t workspace_size;
    };
    // keyed like the reference's cache: the merged einsummable
    // (src/engine/gpu/gpu_kernel_manager.cc:595-600,1254-1263)
    built_t const& get_built_kernel_info(einsummable_t const& e) const;

    int        device;
    es_b200_t* handle;

    std::unordered_map<einsummable_t, built_t> kernels;
};
