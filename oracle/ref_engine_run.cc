// Test infrastructure, not product code.
//
// Runs the reference's OWN GPU engine -- make_gpu_exec_graph, the exec nodes, stream pool,
// workspace / group / buffer managers and exec_state_t::event_loop, compiled unchanged from
// src/engine and src/engine/gpu -- on top of the drop-in kernel_manager_t
// (einsummable_b200/host/gpu_kernel_manager.*), the way gpu_mg_server_t::execute_memgraph does
// (src/server/gpu/server.cc:96-136), on memgraphs the reference's compilers build in-process.
//
//   engine_parity <graph> <dir> <iters> [fold]
//     graph: c1:<n>:<split>:<dtype 0|1>          blocked matmul (config 1)
//            llama:<dim>:<heads>:<multiple_of>:<vocab>:<layers>:<batch>:<seq>:<dtype>
//   One location (one GPU).  Writes <dir>/memgraph.json (ref_graph_write_json), reads
//   <dir>/in.bin (the location buffer with the inputs in place; absent: the buffer is filled with
//   the byte 0x2e, finite small values in every dtype, for timing runs), runs the event loop
//   <iters> times, writes <dir>/out.bin (the location buffer afterwards); then puts the inputs back
//   and runs the same memgraph through gpu_program_t (einsummable_b200/host/gpu_program.*: the
//   library's dependency-ordered program instead of the event loop, built from the same memgraph_t by
//   C++ code alone), eagerly and as a CUDA-graph replay, and writes <dir>/out_program.bin.  With `fold`
//   the memgraph then goes through the C++ fusion passes (einsummable_b200/host/gpu_fuse.h: elementwise
//   nodes folded into their readers, every attention chain one node) and that graph through gpu_program_t:
//   <dir>/out_folded.bin; and the folded graph through gpu_exchange_program_t, the program type for one
//   process per GPU (<dir>/out_exchange.bin).  Prints one JSON line with the times.
#include "src/engine/exec_graph.h"
#include "src/engine/exec_state.h"
#include "src/engine/managers.h"
#include "src/engine/gpu/workspace.h"
#include "src/engine/gpu/stream_pool.h"
#include "src/engine/gpu/gpu_kernel_manager.h"
#include "src/engine/gpu/gpu_program.h"

#include <cuda_runtime.h>

#include <chrono>
#include <cmath>
#include <fstream>
#include <sstream>

extern "C" {
int         ref_graph_build_c1(uint64_t n, int n_split, int nlocs, int dtype_code);
int         ref_graph_build_llama(uint64_t dim, uint64_t n_heads, uint64_t multiple_of, uint64_t vocab_size,
                                  int n_layers, uint64_t batch, uint64_t seqlen, int nlocs, int dtype_code);
int         ref_graph_write_json(int h, char const* path);
char const* ref_graph_last_error();
}
memgraph_t const&     ref_graph_memgraph(int h);
std::vector<memloc_t> ref_graph_saved(int h);

static vector<string> split(string const& s, char c)
{
    vector<string>    out;
    std::stringstream ss(s);
    string            item;
    while (std::getline(ss, item, c)) out.push_back(item);
    return out;
}

// Without <dir>/in.bin and in fold mode: the buffer filled with f16 values in +-0.04 (a 16 MiB block of a
// linear congruential sequence, repeated), so that the unfolded and the folded run of a full-size graph can
// be compared on finite results; otherwise the byte 0x2e everywhere.
static void fill_buffer(void* mem, uint64_t mem_size, string const& dir, bool random_f16)
{
    std::ifstream in(dir + "/in.bin", std::ios::binary);
    if (in) {
        vector<char> host(mem_size);
        in.read(host.data(), mem_size);
        handle_cuda_error(cudaMemcpy(mem, host.data(), mem_size, cudaMemcpyHostToDevice));
    } else if (random_f16) {
        uint64_t const    block = uint64_t(16) << 20;
        vector<float16_t> host(block / 2);
        uint32_t          state = 12345u;
        for (auto& v : host) {
            state = state * 1664525u + 1013904223u;
            v = float16_t(0.08f * (float(state >> 8) / 16777216.0f - 0.5f));
        }
        for (uint64_t at = 0; at < mem_size; at += block) {
            handle_cuda_error(cudaMemcpy(static_cast<char*>(mem) + at, host.data(), std::min(block, mem_size - at),
                                         cudaMemcpyHostToDevice));
        }
    } else {
        handle_cuda_error(cudaMemset(mem, 0x2e, mem_size));
    }
}

static double now_ms()
{
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv)
{
    try {
        if (argc < 4) throw std::runtime_error("usage: engine_parity <graph> <dir> <iters> [fold]");
        bool const with_fold = argc > 4 && string(argv[4]) == "fold";
        vector<string> g = split(argv[1], ':');
        string         dir = argv[2];
        int            iters = std::stoi(argv[3]);
        int            h = -1;
        auto           u = [&](int i) { return (uint64_t)std::stoull(g.at(i)); };
        if (g.at(0) == "c1") {
            h = ref_graph_build_c1(u(1), (int)u(2), 1, (int)u(3));
        } else if (g.at(0) == "llama") {
            h = ref_graph_build_llama(u(1), u(2), u(3), u(4), (int)u(5), u(6), u(7), 1, (int)u(8));
        } else {
            throw std::runtime_error("unknown graph kind");
        }
        if (h < 0) throw std::runtime_error(string("graph build failed: ") + ref_graph_last_error());
        if (ref_graph_write_json(h, (dir + "/memgraph.json").c_str()) != 0)
            throw std::runtime_error(string("write_json failed: ") + ref_graph_last_error());
        memgraph_t const& memgraph = ref_graph_memgraph(h);
        uint64_t          mem_size = memgraph.mem_sizes().at(0);

        handle_cuda_error(cudaSetDevice(0));
        void* mem = gpu_allocate_memory(mem_size + 256, 0);
        fill_buffer(mem, mem_size, dir, with_fold);
        // as gpu_mg_server_t does: one kernel manager per GPU, 5 streams per device
        vector<kernel_manager_t> kernel_managers;
        kernel_managers.emplace_back(0);
        streampool_t  stream_pool(5, 1);
        vector<void*> mems{mem};

        double       t0 = now_ms();
        exec_graph_t graph = exec_graph_t::make_gpu_exec_graph(memgraph, 0, kernel_managers, 1, mems);
        double       t_build = now_ms() - t0;

        vector<double> loops;
        for (int it = 0; it != iters; ++it) {
            vector<rm_ptr_t> rms{rm_ptr_t(new gpu_workspace_manager_t()), rm_ptr_t(new group_manager_t()),
                                 rm_ptr_t(new global_buffers_t(mems)), rm_ptr_t(new streampool_manager_t(stream_pool))};
            rm_ptr_t         resource_manager(new resource_manager_t(rms));
            exec_state_t     state(graph, resource_manager);
            double           t1 = now_ms();
            state.event_loop();
            handle_cuda_error(cudaDeviceSynchronize());
            loops.push_back(now_ms() - t1);
        }
        {
            vector<char> host(mem_size);
            handle_cuda_error(cudaMemcpy(host.data(), mem, mem_size, cudaMemcpyDeviceToHost));
            std::ofstream out(dir + "/out.bin", std::ios::binary);
            out.write(host.data(), mem_size);
        }
        // the saved results as they stand in the buffer (fold mode: compared between the two program runs)
        bool const f16_graph = g.at(0) == "llama" ? g.back() == "0" : false;
        auto       read_saved = [&]() {
            vector<float> values;
            for (memloc_t const& m : ref_graph_saved(h)) {
                vector<char> host(m.size);
                handle_cuda_error(cudaMemcpy(host.data(), static_cast<char*>(mem) + m.offset, m.size, cudaMemcpyDeviceToHost));
                if (f16_graph) {
                    auto const* p = reinterpret_cast<float16_t const*>(host.data());
                    for (uint64_t i = 0; i != m.size / 2; ++i) values.push_back(float(p[i]));
                } else {
                    auto const* p = reinterpret_cast<float const*>(host.data());
                    values.insert(values.end(), p, p + m.size / 4);
                }
            }
            return values;
        };
        vector<float> saved_program;
        double        saved_max_abs = 0, saved_max_diff = -1;
        bool          saved_finite = true;
        // the same memgraph through the program executor
        vector<double> eager, replay;
        int            program_ops = 0;
        double         t_program_build = 0;
        if (iters > 0) {
            fill_buffer(mem, mem_size, dir, with_fold);
            double        t2 = now_ms();
            gpu_program_t program(memgraph, 0, kernel_managers[0], mem);
            t_program_build = now_ms() - t2;
            program_ops = program.num_ops();
            cudaStream_t stream;
            handle_cuda_error(cudaStreamCreate(&stream));
            for (int it = 0; it != iters; ++it) {
                double t1 = now_ms();
                program.launch(stream);
                handle_cuda_error(cudaStreamSynchronize(stream));
                eager.push_back(now_ms() - t1);
            }
            {
                vector<char> host(mem_size);
                handle_cuda_error(cudaMemcpy(host.data(), mem, mem_size, cudaMemcpyDeviceToHost));
                std::ofstream out(dir + "/out_program.bin", std::ios::binary);
                out.write(host.data(), mem_size);
            }
            if (with_fold) saved_program = read_saved();
            program.instantiate();
            for (int it = 0; it != iters; ++it) {
                double t1 = now_ms();
                program.replay(stream);
                handle_cuda_error(cudaStreamSynchronize(stream));
                replay.push_back(now_ms() - t1);
            }
            handle_cuda_error(cudaStreamDestroy(stream));
        }
        // the folded graph (C++ passes) through the program executor
        vector<double> folded_eager, folded_replay;
        int            folded_ops = 0, n_folded = 0, n_chains = 0, exchange_ops = 0;
        double         exchange_max_diff = -1;
        vector<float>  saved_folded_values;
        if (with_fold && iters > 0) {
            fill_buffer(mem, mem_size, dir, with_fold);
            vector<memloc_t>            saved = ref_graph_saved(h);
            es_fuse::folded_t           folded = es_fuse::fold_elementwise(memgraph, saved);
            es_fuse::attention_folded_t chains = es_fuse::fold_attention(folded.memgraph, saved);
            n_folded = int(folded.folded.size());
            n_chains = int(chains.attention.size());
            gpu_program_t program(chains.memgraph, 0, kernel_managers[0], mem, {}, 16, &chains.attention);
            folded_ops = program.num_ops();
            cudaStream_t stream;
            handle_cuda_error(cudaStreamCreate(&stream));
            for (int it = 0; it != iters; ++it) {
                double t1 = now_ms();
                program.launch(stream);
                handle_cuda_error(cudaStreamSynchronize(stream));
                folded_eager.push_back(now_ms() - t1);
            }
            {
                vector<char> host(mem_size);
                handle_cuda_error(cudaMemcpy(host.data(), mem, mem_size, cudaMemcpyDeviceToHost));
                std::ofstream out(dir + "/out_folded.bin", std::ios::binary);
                out.write(host.data(), mem_size);
            }
            {
                vector<float> saved_folded = read_saved();
                saved_folded_values = saved_folded;
                saved_max_diff = 0;
                for (size_t i = 0; i != saved_folded.size(); ++i) {
                    saved_finite = saved_finite && std::isfinite(saved_folded[i]) && std::isfinite(saved_program[i]);
                    saved_max_abs = std::max(saved_max_abs, double(std::fabs(saved_program[i])));
                    saved_max_diff = std::max(saved_max_diff, double(std::fabs(saved_folded[i] - saved_program[i])));
                }
            }
            program.instantiate();
            for (int it = 0; it != iters; ++it) {
                double t1 = now_ms();
                program.replay(stream);
                handle_cuda_error(cudaStreamSynchronize(stream));
                folded_replay.push_back(now_ms() - t1);
            }
            handle_cuda_error(cudaStreamDestroy(stream));
            // the same folded graph through gpu_exchange_program_t (the program type for one process per GPU:
            // units and order of service from gpu_exchange_plan.h; with one location it has no exchange ops)
            fill_buffer(mem, mem_size, dir, with_fold);
            void* flags = nullptr;
            handle_cuda_error(cudaMalloc(&flags, 256));
            handle_cuda_error(cudaMemset(flags, 0, 256));
            {
                gpu_exchange_program_t xprogram(chains.memgraph, 0, kernel_managers[0], {mem}, {flags}, {}, 16, 0,
                                                &chains.attention);
                exchange_ops = xprogram.num_ops();
                cudaStream_t xstream;
                handle_cuda_error(cudaStreamCreate(&xstream));
                xprogram.launch(xstream);
                handle_cuda_error(cudaStreamSynchronize(xstream));
                vector<float> a = read_saved();
                {
                    vector<char> host(mem_size);
                    handle_cuda_error(cudaMemcpy(host.data(), mem, mem_size, cudaMemcpyDeviceToHost));
                    std::ofstream out(dir + "/out_exchange.bin", std::ios::binary);
                    out.write(host.data(), mem_size);
                }
                xprogram.instantiate();
                xprogram.replay(xstream);
                handle_cuda_error(cudaStreamSynchronize(xstream));
                vector<float> b = read_saved();
                vector<float> f = saved_folded_values;
                exchange_max_diff = 0;
                for (size_t i = 0; i != a.size(); ++i) {
                    exchange_max_diff = std::max(exchange_max_diff, double(std::fabs(a[i] - f[i])));
                    exchange_max_diff = std::max(exchange_max_diff, double(std::fabs(b[i] - f[i])));
                }
                handle_cuda_error(cudaStreamDestroy(xstream));
            }
            handle_cuda_error(cudaFree(flags));
        }
        auto list = [](vector<double> const& v) {
            std::stringstream ss;
            ss << "[";
            for (size_t i = 0; i != v.size(); ++i) ss << (i ? ", " : "") << v[i];
            ss << "]";
            return ss.str();
        };
        std::cout << "{\"mem_size\": " << mem_size << ", \"exec_nodes\": " << graph.nodes.size()
                  << ", \"build_ms\": " << t_build << ", \"event_loop_ms\": " << list(loops)
                  << ", \"program_ops\": " << program_ops << ", \"program_build_ms\": " << t_program_build
                  << ", \"program_eager_ms\": " << list(eager) << ", \"program_replay_ms\": " << list(replay)
                  << ", \"nodes_folded\": " << n_folded << ", \"attention_chains\": " << n_chains
                  << ", \"folded_ops\": " << folded_ops << ", \"folded_eager_ms\": " << list(folded_eager)
                  << ", \"folded_replay_ms\": " << list(folded_replay) << ", \"saved_finite\": " << (saved_finite ? "true" : "false")
                  << ", \"saved_max_abs\": " << saved_max_abs << ", \"folded_vs_program_max_abs_diff\": " << saved_max_diff
                  << ", \"exchange_program_ops\": " << exchange_ops
                  << ", \"exchange_program_vs_folded_max_abs_diff\": " << exchange_max_diff << "}" << std::endl;
        return 0;
    } catch (std::exception const& e) {
        std::cerr << "engine_parity: " << e.what() << std::endl;
        return 1;
    }
}
