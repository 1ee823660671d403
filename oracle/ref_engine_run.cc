// Test infrastructure, not product code.
//
// Runs the reference's OWN GPU engine -- make_gpu_exec_graph, the exec nodes, stream pool,
// workspace / group / buffer managers and exec_state_t::event_loop, compiled unchanged from
// src/engine and src/engine/gpu -- on top of the drop-in kernel_manager_t
// (einsummable_b200/host/gpu_kernel_manager.*), the way gpu_mg_server_t::execute_memgraph does
// (src/server/gpu/server.cc:96-136), on memgraphs the reference's compilers build in-process.
//
//   engine_parity <graph> <dir> <iters>
//     graph: c1:<n>:<split>:<dtype 0|1>          blocked matmul (config 1)
//            llama:<dim>:<heads>:<multiple_of>:<vocab>:<layers>:<batch>:<seq>:<dtype>
//   One location (one GPU).  Writes <dir>/memgraph.json (ref_graph_write_json), reads
//   <dir>/in.bin (the location buffer with the inputs in place; absent: the buffer is filled with
//   the byte 0x2e, finite small values in every dtype, for timing runs), runs the event loop
//   <iters> times, writes <dir>/out.bin (the location buffer afterwards); then puts the inputs back
//   and runs the same memgraph through gpu_program_t (einsummable_b200/host/gpu_program.*: the
//   library's dependency-ordered program instead of the event loop, built from the same memgraph_t by
//   C++ code alone), eagerly and as a CUDA-graph replay, and writes <dir>/out_program.bin.  Prints one
//   JSON line with the times.
#include "src/engine/exec_graph.h"
#include "src/engine/exec_state.h"
#include "src/engine/managers.h"
#include "src/engine/gpu/workspace.h"
#include "src/engine/gpu/stream_pool.h"
#include "src/engine/gpu/gpu_kernel_manager.h"
#include "src/engine/gpu/gpu_program.h"

#include <cuda_runtime.h>

#include <chrono>
#include <fstream>
#include <sstream>

extern "C" {
int         ref_graph_build_c1(uint64_t n, int n_split, int nlocs, int dtype_code);
int         ref_graph_build_llama(uint64_t dim, uint64_t n_heads, uint64_t multiple_of, uint64_t vocab_size,
                                  int n_layers, uint64_t batch, uint64_t seqlen, int nlocs, int dtype_code);
int         ref_graph_write_json(int h, char const* path);
char const* ref_graph_last_error();
}
memgraph_t const& ref_graph_memgraph(int h);

static vector<string> split(string const& s, char c)
{
    vector<string>    out;
    std::stringstream ss(s);
    string            item;
    while (std::getline(ss, item, c)) out.push_back(item);
    return out;
}

static double now_ms()
{
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv)
{
    try {
        if (argc < 4) throw std::runtime_error("usage: engine_parity <graph> <dir> <iters>");
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
        {
            std::ifstream in(dir + "/in.bin", std::ios::binary);
            if (in) {
                vector<char> host(mem_size);
                in.read(host.data(), mem_size);
                handle_cuda_error(cudaMemcpy(mem, host.data(), mem_size, cudaMemcpyHostToDevice));
            } else {
                handle_cuda_error(cudaMemset(mem, 0x2e, mem_size));
            }
        }
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
        // the same memgraph through the program executor
        vector<double> eager, replay;
        int            program_ops = 0;
        double         t_program_build = 0;
        if (iters > 0) {
            std::ifstream in(dir + "/in.bin", std::ios::binary);
            if (in) {
                vector<char> host(mem_size);
                in.read(host.data(), mem_size);
                handle_cuda_error(cudaMemcpy(mem, host.data(), mem_size, cudaMemcpyHostToDevice));
            } else {
                handle_cuda_error(cudaMemset(mem, 0x2e, mem_size));
            }
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
            program.instantiate();
            for (int it = 0; it != iters; ++it) {
                double t1 = now_ms();
                program.replay(stream);
                handle_cuda_error(cudaStreamSynchronize(stream));
                replay.push_back(now_ms() - t1);
            }
            handle_cuda_error(cudaStreamDestroy(stream));
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
                  << ", \"program_eager_ms\": " << list(eager) << ", \"program_replay_ms\": " << list(replay) << "}"
                  << std::endl;
        return 0;
    } catch (std::exception const& e) {
        std::cerr << "engine_parity: " << e.what() << std::endl;
        return 1;
    }
}
