// Test infrastructure, not product code.
//
// What gpu_exchange_program_t (einsummable_b200/host/gpu_program.*) asks the library to do for every rank
// of a memgraph that spans several locations -- checked on a machine without a GPU: linked with the
// recording stand-in of the C ABI (oracle/mock_es_b200.cc) instead of libes_b200.so.
//
//   exchange_ops <graph> <dir> <group_sum 0|1>
//     graph: llama:<dim>:<heads>:<multiple_of>:<vocab>:<layers>:<batch>:<seq>:<dtype>:<nlocs>     autoplace01
//            llama_tp:... (the same fields)                                                       tensor-parallel by hand
//            c1_evict:<n>:<split>:<dtype>:<bytes per location>:<nlocs>    config 1 under a memory limit (evict / load)
//   Builds the memgraph in-process with the reference's compilers, writes <dir>/memgraph.json, folds it with the
//   C++ passes (einsummable_b200/host/gpu_fuse.h), builds one gpu_exchange_program_t per rank over made-up base
//   addresses -- location r's buffer at (r + 1) << 44, its flag words at ((r + 1) << 44) + (1 << 40) -- and
//   writes the ops each program was given to <dir>/ops<rank>.json (with one location also gpu_program_t's, the
//   program type for one device: <dir>/ops_program0.json).  The host block of storage id k of a graph
//   with storage is the made-up address (1 << 50) + 4096 * k.
#include "src/engine/gpu/gpu_kernel_manager.h"
#include "src/engine/gpu/gpu_program.h"

#include <fstream>
#include <sstream>

extern "C" {
int ref_graph_build_llama(uint64_t dim, uint64_t n_heads, uint64_t multiple_of, uint64_t vocab_size, int n_layers,
                          uint64_t batch, uint64_t seqlen, int nlocs, int dtype_code);
int ref_graph_build_llama_tp(uint64_t dim, uint64_t n_heads, uint64_t multiple_of, uint64_t vocab_size, int n_layers,
                             uint64_t batch, uint64_t seqlen, int nlocs, int dtype_code);
int         ref_graph_build_c1_evict(uint64_t n, int n_split, int nlocs, int dtype_code, uint64_t mem_limit);
int         ref_graph_write_json(int h, char const* path);
char const* ref_graph_last_error();
}
memgraph_t const&     ref_graph_memgraph(int h);
std::vector<memloc_t> ref_graph_saved(int h);
std::string           mock_take_ops();

int main(int argc, char** argv)
{
    try {
        if (argc < 4) throw std::runtime_error("usage: exchange_ops <graph> <dir> <group_sum 0|1>");
        vector<string>    g;
        std::stringstream ss(argv[1]);
        string            item;
        while (std::getline(ss, item, ':')) g.push_back(item);
        string const dir = argv[2];
        bool const   group_sum = string(argv[3]) == "1";
        auto         u = [&](int i) { return (uint64_t)std::stoull(g.at(i)); };
        int          h = -1;
        if (g.at(0) == "llama") {
            h = ref_graph_build_llama(u(1), u(2), u(3), u(4), (int)u(5), u(6), u(7), (int)u(9), (int)u(8));
        } else if (g.at(0) == "llama_tp") {
            h = ref_graph_build_llama_tp(u(1), u(2), u(3), u(4), (int)u(5), u(6), u(7), (int)u(9), (int)u(8));
        } else if (g.at(0) == "c1_evict") {
            h = ref_graph_build_c1_evict(u(1), (int)u(2), (int)u(5), (int)u(3), u(4));
        } else {
            throw std::runtime_error("unknown graph kind");
        }
        if (h < 0) throw std::runtime_error(string("graph build failed: ") + ref_graph_last_error());
        if (ref_graph_write_json(h, (dir + "/memgraph.json").c_str()) != 0)
            throw std::runtime_error(string("write_json failed: ") + ref_graph_last_error());
        memgraph_t const&           memgraph = ref_graph_memgraph(h);
        vector<memloc_t>            saved = ref_graph_saved(h);
        es_fuse::folded_t           folded = es_fuse::fold_elementwise(memgraph, saved);
        es_fuse::attention_folded_t chains = es_fuse::fold_attention(folded.memgraph, saved);
        int const                   world = memgraph.num_compute_locs;
        vector<void*>               peer_mem, peer_flags;
        for (int r = 0; r != world; ++r) {
            uintptr_t base = uintptr_t(r + 1) << 44;
            peer_mem.push_back(reinterpret_cast<void*>(base));
            peer_flags.push_back(reinterpret_cast<void*>(base + (uintptr_t(1) << 40)));
        }
        storage_blocks_t storage;
        for (auto const& node : memgraph.nodes) {
            auto const& op = node.op;
            if (op.is_evict() || op.is_load() || op.is_inputsto()) {
                stoloc_t at = op.is_evict() ? op.get_evict().dst : op.is_load() ? op.get_load().src : op.get_inputsto().as_stoloc();
                storage[{at.loc, at.id}] = reinterpret_cast<void*>((uintptr_t(1) << 50) + uintptr_t(4096) * uintptr_t(at.id));
            }
        }
        for (int rank = 0; rank != world; ++rank) {
            kernel_manager_t km(rank);
            mock_take_ops();
            gpu_exchange_program_t program(chains.memgraph, rank, km, peer_mem, peer_flags, {}, 16, 0, &chains.attention,
                                           group_sum, &storage);
            std::ofstream out(dir + "/ops" + std::to_string(rank) + ".json");
            out << "{\"n_ops\":" << program.num_ops() << ",\"ops\":[\n" << mock_take_ops() << "\n]}\n";
        }
        if (world == 1) {
            // one location: also gpu_program_t, the program type for one device (memgraph order)
            kernel_manager_t km(0);
            mock_take_ops();
            gpu_program_t program(chains.memgraph, 0, km, peer_mem[0], {}, 16, &chains.attention, &storage);
            std::ofstream out(dir + "/ops_program0.json");
            out << "{\"n_ops\":" << program.num_ops() << ",\"ops\":[\n" << mock_take_ops() << "\n]}\n";
        }
        std::cout << "{\"world\": " << world << ", \"nodes_folded\": " << folded.folded.size()
                  << ", \"attention_chains\": " << chains.attention.size() << "}" << std::endl;
        return 0;
    } catch (std::exception const& e) {
        std::cerr << "exchange_ops: " << e.what() << std::endl;
        return 1;
    }
}
