// Test infrastructure, not product code.
//
// Drives the drop-in kernel_manager_t (einsummable_b200/host/gpu_kernel_manager.*)
// with the reference's OWN types -- einsummable_t, touch_t, fill_t, scalarop_t,
// dbuffer_t -- and compares every result with the reference's own interpreter,
// the way the reference's GPU kernel checks do
// (exps/gpuexec_kernelmanager.cc:18-157: build, cudaMalloc, km(...), is_close).
// Built only where the reference tree exists; the binary travels to the GPU box.
#include "src/engine/gpu/gpu_kernel_manager.h"
#include "src/einsummable/reference.h"

#include <cuda_runtime.h>

#define CHECK_CUDA(x)                                                                              \
    do {                                                                                           \
        cudaError_t e_ = (x);                                                                      \
        if (e_ != cudaSuccess) {                                                                   \
            throw std::runtime_error(string(#x) + ": " + cudaGetErrorString(e_));                  \
        }                                                                                          \
    } while (0)

static int n_fail = 0;

static void report(string const& name, bool ok)
{
    std::cout << (ok ? "ok   " : "FAIL ") << name << std::endl;
    if (!ok) {
        n_fail++;
    }
}

static void run_einsummable(kernel_manager_t& km, string name, einsummable_t e, float eps, bool ints = false)
{
    vector<dbuffer_t> inns;
    for (int i = 0; i != e.inns.size(); ++i) {
        dbuffer_t b = make_dbuffer(e.inn_dtype(i), product(e.inn_shape(i)));
        if (ints) {
            b.random("0.5", "2.0");
        } else {
            b.random("-1.0", "1.0");
        }
        inns.push_back(b);
    }
    dbuffer_t out_ref = reference_einsummable(e, inns);

    auto maybe_ws = km.build(e);
    if (!maybe_ws) {
        report(name + " (build returned nullopt)", false);
        return;
    }
    uint64_t ws_size = maybe_ws.value().known() ? maybe_ws.value().value() : 0;

    vector<void*>       d_inns;
    vector<void const*> c_inns;
    for (auto& b : inns) {
        void* p;
        CHECK_CUDA(cudaMalloc(&p, b.size()));
        CHECK_CUDA(cudaMemcpy(p, b.raw(), b.size(), cudaMemcpyHostToDevice));
        d_inns.push_back(p);
        c_inns.push_back(p);
    }
    void* d_out;
    CHECK_CUDA(cudaMalloc(&d_out, out_ref.size()));
    void* d_ws = nullptr;
    if (ws_size) {
        CHECK_CUDA(cudaMalloc(&d_ws, ws_size));
    }
    cudaStream_t stream;
    CHECK_CUDA(cudaStreamCreate(&stream));
    optional<tuple<void*, uint64_t>> ws;
    if (ws_size) {
        ws = tuple<void*, uint64_t>{d_ws, ws_size};
    }
    km(e, stream, d_out, c_inns, ws);
    CHECK_CUDA(cudaStreamSynchronize(stream));
    dbuffer_t out = make_dbuffer(e.out_dtype(), e.out_nelem());
    CHECK_CUDA(cudaMemcpy(out.raw(), d_out, out.size(), cudaMemcpyDeviceToHost));
    report(name + " " + e.str(), is_close(out_ref, out, eps));
    for (void* p : d_inns) {
        cudaFree(p);
    }
    cudaFree(d_out);
    if (d_ws) {
        cudaFree(d_ws);
    }
    cudaStreamDestroy(stream);
}

static void run_touch(kernel_manager_t& km, string name, touch_t touch)
{
    uint64_t n_inn = 1, n_out = 1;
    for (auto const& t : touch.selection) {
        n_inn *= t.d_inn;
        n_out *= t.d_out;
    }
    dbuffer_t inn = make_dbuffer(touch.dtype, n_inn);
    dbuffer_t out_ref = make_dbuffer(touch.dtype, n_out);
    inn.random("-1.0", "1.0");
    out_ref.random("-1.0", "1.0");
    dbuffer_t out = out_ref.copy();
    reference_touch(touch, out_ref, inn);

    void *d_inn, *d_out;
    CHECK_CUDA(cudaMalloc(&d_inn, inn.size()));
    CHECK_CUDA(cudaMalloc(&d_out, out.size()));
    CHECK_CUDA(cudaMemcpy(d_inn, inn.raw(), inn.size(), cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(d_out, out.raw(), out.size(), cudaMemcpyHostToDevice));
    km(touch, 0, d_out, d_inn);
    CHECK_CUDA(cudaDeviceSynchronize());
    CHECK_CUDA(cudaMemcpy(out.raw(), d_out, out.size(), cudaMemcpyDeviceToHost));
    report(name, out == out_ref); // bit-exact, as exps/cpuexec_touch.cc:111
    cudaFree(d_inn);
    cudaFree(d_out);
}

int main()
{
    try {
        set_seed(99);
        kernel_manager_t km(0);

        // contractions (exps/gpuexec_kernelmanager.cc:432-948,3129-3132)
        run_einsummable(km, "matmul ss f32", einsummable_t::from_matmul_ss(96, 64, 80, dtype_t::f32), 1e-3);
        run_einsummable(km, "matmul st f16", einsummable_t::from_matmul_st(128, 64, 64, dtype_t::f16), 0.1);
        run_einsummable(km, "matmul ts f32", einsummable_t::from_matmul_ts(64, 64, 64, dtype_t::f32), 1e-3);
        run_einsummable(km, "matmul tt f16", einsummable_t::from_matmul_tt(64, 64, 128, dtype_t::f16), 0.1);
        {
            auto [inns, out_rank] = einsummable_t::parse_str("adbe,dec->abc");
            einsummable_t e({2, 16, 24, 3, 8}, inns, out_rank, scalarop_t::make_mul(dtype_t::f32), castable_t::add);
            run_einsummable(km, "5-mode contraction f32", e, 1e-3);
        }
        // reductions (:1399-1643)
        run_einsummable(km, "sum f32", einsummable_t::aggregate({50, 300}, {0, 1}, 1, dtype_t::f32, castable_t::add), 1e-3);
        run_einsummable(km, "max f16", einsummable_t::aggregate({20, 128}, {0, 1}, 1, dtype_t::f16, castable_t::max), 1e-3);
        // elementwise (:1656-2582)
        run_einsummable(km, "silu f16", einsummable_t({4096}, {{0}}, 1, scalarop_t::make_silu(dtype_t::f16)), 0.03);
        run_einsummable(km, "exp f32", einsummable_t({1000}, {{0}}, 1, scalarop_t::make_exp(dtype_t::f32)), 1e-3);
        run_einsummable(km, "square f32", einsummable_t({1000}, {{0}}, 1, scalarop_t::make_square(dtype_t::f32)), 1e-3);
        run_einsummable(km, "to_f32", einsummable_t({512}, {{0}}, 1, scalarop_t::make_convert_dtype(dtype_t::f16, dtype_t::f32)), 1e-3);
        run_einsummable(km, "ab,b->ab add f32", einsummable_t({30, 40}, {{0, 1}, {1}}, 2, scalarop_t::make_add(dtype_t::f32)), 1e-3);
        run_einsummable(km, "ab,a->ab div f32", einsummable_t({30, 40}, {{0, 1}, {0}}, 2, scalarop_t::make_div(dtype_t::f32)), 1e-2, true);
        run_einsummable(km, "rope c64", einsummable_t({2, 8, 4, 16}, {{0, 1, 2, 3}, {1, 3}}, 4, scalarop_t::make_mul(dtype_t::c64)), 1e-3);
        run_einsummable(km, "permute f16", einsummable_t({4, 6, 8, 16}, {{0, 2, 1, 3}}, 4, scalarop_t::make_identity(dtype_t::f16)), 0.0);

        // touches (exps/cpuexec_touch.cc:19-139)
        for (dtype_t d : {dtype_t::f16, dtype_t::f32, dtype_t::f64, dtype_t::c64}) {
            for (int c = -1; c != 4; ++c) {
                if (d == dtype_t::c64 && c >= 2) {
                    continue;
                }
                touch_t t{.selection = {{12, 10, 3, 1, 7}, {20, 24, 4, 8, 12}, {16, 16, 0, 0, 16}},
                          .castable = c < 0 ? optional<castable_t>() : optional<castable_t>(castable_t(c)),
                          .dtype = d};
                run_touch(km, "touch " + write_with_ss(d) + " castable " + std::to_string(c), t);
            }
        }

        // fills (exps/GPU_correctness.cc:740-790)
        {
            fill_t::lowertri_t l{.lower = scalar_t::zero(dtype_t::f16), .upper = scalar_t::negative_inf(dtype_t::f16),
                                 .nrow = 40, .ncol = 40, .start = 0};
            dbuffer_t ref = reference_fill(fill_t(l));
            void*     d;
            CHECK_CUDA(cudaMalloc(&d, ref.size()));
            km.lowerTri_fill(l, 0, d);
            dbuffer_t out = make_dbuffer(dtype_t::f16, 1600);
            CHECK_CUDA(cudaMemcpy(out.raw(), d, out.size(), cudaMemcpyDeviceToHost));
            report("lowerTri_fill f16 -inf", out == ref);
            fill_t::constant_t c{.value = scalar_t(float(2.5)), .shape = {33, 7}};
            dbuffer_t          cref = reference_fill(fill_t(c));
            void*              d2;
            CHECK_CUDA(cudaMalloc(&d2, cref.size()));
            km.constant_fill(c, 0, d2);
            dbuffer_t cout_ = make_dbuffer(dtype_t::f32, 231);
            CHECK_CUDA(cudaMemcpy(cout_.raw(), d2, cout_.size(), cudaMemcpyDeviceToHost));
            report("constant_fill f32", cout_ == cref);
        }

        // un-built einsummables throw, as the reference does
        bool threw = false;
        try {
            km(einsummable_t({77}, {{0}}, 1, scalarop_t::make_exp(dtype_t::f32)), 0, nullptr, {nullptr});
        } catch (std::runtime_error const&) {
            threw = true;
        }
        report("operator() before build throws", threw);
    } catch (std::exception const& e) {
        std::cout << "FAIL exception: " << e.what() << std::endl;
        return 2;
    }
    std::cout << (n_fail == 0 ? "ALL OK" : "FAILURES") << std::endl;
    return n_fail == 0 ? 0 : 1;
}
