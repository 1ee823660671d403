#include "jit.h"
#include "pdl.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <nvrtc.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>

namespace es {

namespace {

// Compiled kernels are kept across processes: <dir>/<hash of source + compiler version>.cubin.
// The directory is $ES_B200_CACHE_DIR, else $XDG_CACHE_HOME/es_b200, else ~/.cache/es_b200;
// ES_B200_CACHE_DIR=0 turns the cache off.  A build() of an einsummable seen before then costs a file
// read instead of an NVRTC compilation (20-60 ms each; a LLaMA layer has ~25 distinct kernels).
std::string cache_dir()
{
    char const* d = std::getenv("ES_B200_CACHE_DIR");
    if (d && std::string(d) == "0") return "";
    std::string dir;
    if (d && *d) {
        dir = d;
    } else if (char const* x = std::getenv("XDG_CACHE_HOME"); x && *x) {
        dir = std::string(x) + "/es_b200";
    } else if (char const* h = std::getenv("HOME"); h && *h) {
        dir = std::string(h) + "/.cache/es_b200";
    } else {
        return "";
    }
    // two levels at most (~/.cache may not exist yet); failures just mean no cache
    std::string parent = dir.substr(0, dir.find_last_of('/'));
    ::mkdir(parent.c_str(), 0755);
    ::mkdir(dir.c_str(), 0755);
    return dir;
}

std::string cache_path(std::string const& source)
{
    static std::string const dir = cache_dir();
    if (dir.empty()) return "";
    int major = 0, minor = 0;
    nvrtcVersion(&major, &minor);
    // FNV-1a, 64 bits, over the compiler version, the target and the source
    uint64_t    h = 1469598103934665603ull;
    std::string salt = "nvrtc" + std::to_string(major) + "." + std::to_string(minor) + "|sm_100a|";
    for (unsigned char c : salt) h = (h ^ c) * 1099511628211ull;
    for (unsigned char c : source) h = (h ^ c) * 1099511628211ull;
    char name[40];
    std::snprintf(name, sizeof name, "%016llx_%zu.cubin", (unsigned long long)h, source.size());
    return dir + "/" + name;
}

bool read_file(std::string const& path, std::vector<char>& out)
{
    std::FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) return false;
    std::fseek(f, 0, SEEK_END);
    long n = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    out.resize(n > 0 ? (size_t)n : 0);
    bool ok = n > 0 && std::fread(out.data(), 1, (size_t)n, f) == (size_t)n;
    std::fclose(f);
    return ok;
}

void write_file(std::string const& path, std::vector<char> const& data)
{
    // write beside and rename: another process may be reading or writing the same kernel
    std::string tmp = path + "." + std::to_string((long)::getpid()) + ".tmp";
    std::FILE*  f = std::fopen(tmp.c_str(), "wb");
    if (!f) return;
    bool ok = std::fwrite(data.data(), 1, data.size(), f) == data.size();
    std::fclose(f);
    if (ok) std::rename(tmp.c_str(), path.c_str());
    else std::remove(tmp.c_str());
}

} // namespace

std::vector<char> nvrtc_compile(std::string const& source, std::string* log_out)
{
    std::string const cached = log_out ? std::string() : cache_path(source);
    if (!cached.empty()) {
        std::vector<char> cubin;
        if (read_file(cached, cubin)) return cubin;
    }
    nvrtcProgram prog;
    if (nvrtcCreateProgram(&prog, source.c_str(), "es_kernel.cu", 0, nullptr, nullptr) !=
        NVRTC_SUCCESS) {
        fail(ES_COMPILE_ERROR, "nvrtcCreateProgram failed");
    }
    char const* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo",
                          "--ptxas-options=-v"};
    // fast-math stays off: only f16-typed nodes use approximate intrinsics, and
    // those are chosen explicitly by the expression generator.
    nvrtcResult rc = nvrtcCompileProgram(prog, log_out ? 4 : 3, opts);
    size_t      log_size = 0;
    nvrtcGetProgramLogSize(prog, &log_size);
    std::string log(log_size, '\0');
    if (log_size > 1) nvrtcGetProgramLog(prog, log.data());
    if (log_out) *log_out = log;
    if (rc != NVRTC_SUCCESS) {
        nvrtcDestroyProgram(&prog);
        fail(ES_COMPILE_ERROR, std::string("nvrtc: ") + nvrtcGetErrorString(rc) + "\n" + log);
    }
    size_t size = 0;
    if (nvrtcGetCUBINSize(prog, &size) != NVRTC_SUCCESS || size == 0) {
        nvrtcDestroyProgram(&prog);
        fail(ES_COMPILE_ERROR, "nvrtc produced no cubin");
    }
    std::vector<char> cubin(size);
    nvrtcGetCUBIN(prog, cubin.data());
    nvrtcDestroyProgram(&prog);
    if (!cached.empty()) write_file(cached, cubin);
    return cubin;
}

void* driver_entry(char const* name)
{
    void*                            fn = nullptr;
    cudaDriverEntryPointQueryResult  qres;
    cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
        fail(ES_CUDA_ERROR, std::string("driver entry point not found: ") + name);
    }
    return fn;
}

namespace {
struct driver_t {
    decltype(&cuModuleLoadData)    module_load_data;
    decltype(&cuModuleUnload)      module_unload;
    decltype(&cuModuleGetFunction) module_get_function;
    decltype(&cuLaunchKernel)      launch_kernel;
    decltype(&cuGetErrorString)    get_error_string;
    decltype(&cuFuncSetAttribute)  func_set_attribute;
    decltype(&cuLaunchKernelEx)    launch_kernel_ex;
};

driver_t const& driver()
{
    static driver_t d = [] {
        driver_t x;
        x.module_load_data = (decltype(x.module_load_data))driver_entry("cuModuleLoadData");
        x.module_unload = (decltype(x.module_unload))driver_entry("cuModuleUnload");
        x.module_get_function =
            (decltype(x.module_get_function))driver_entry("cuModuleGetFunction");
        x.launch_kernel = (decltype(x.launch_kernel))driver_entry("cuLaunchKernel");
        x.get_error_string = (decltype(x.get_error_string))driver_entry("cuGetErrorString");
        x.func_set_attribute = (decltype(x.func_set_attribute))driver_entry("cuFuncSetAttribute");
        x.launch_kernel_ex = (decltype(x.launch_kernel_ex))driver_entry("cuLaunchKernelEx");
        return x;
    }();
    return d;
}

void cu_check(CUresult r, char const* what)
{
    if (r != CUDA_SUCCESS) {
        char const* msg = nullptr;
        driver().get_error_string(r, &msg);
        fail(ES_CUDA_ERROR, std::string(what) + ": " + (msg ? msg : "unknown driver error"));
    }
}
} // namespace

module_t::~module_t()
{
    if (cu_module) driver().module_unload((CUmodule)cu_module);
}

void* module_t::function(std::string const& name)
{
    auto it = fns.find(name);
    if (it != fns.end()) return it->second;
    CUfunction f;
    cu_check(driver().module_get_function(&f, (CUmodule)cu_module, name.c_str()),
             "cuModuleGetFunction");
    fns[name] = (void*)f;
    return (void*)f;
}

std::shared_ptr<module_t> load_module(std::vector<char> const& cubin)
{
    // make sure the runtime has a current primary context on this device
    cudaFree(nullptr);
    auto     m = std::make_shared<module_t>();
    CUmodule mod;
    cu_check(driver().module_load_data(&mod, cubin.data()), "cuModuleLoadData");
    m->cu_module = (void*)mod;
    return m;
}

void launch_function(
    void* fn, uint32_t grid, uint32_t block, uint32_t smem, void* stream, void** args)
{
    if (smem > 48 * 1024) {
        cu_check(driver().func_set_attribute((CUfunction)fn,
                                             CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                             (int)smem),
                 "cuFuncSetAttribute");
    }
    if (pdl_launch_flag()) {
        CUlaunchConfig cfg = {};
        cfg.gridDimX = grid;
        cfg.gridDimY = cfg.gridDimZ = 1;
        cfg.blockDimX = block;
        cfg.blockDimY = cfg.blockDimZ = 1;
        cfg.sharedMemBytes = smem;
        cfg.hStream = (CUstream)stream;
        CUlaunchAttribute attr[1];
        attr[0].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attr[0].value.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cu_check(driver().launch_kernel_ex(&cfg, (CUfunction)fn, args, nullptr), "cuLaunchKernelEx");
        return;
    }
    cu_check(driver().launch_kernel(
                 (CUfunction)fn, grid, 1, 1, block, 1, 1, smem, (CUstream)stream, args, nullptr),
             "cuLaunchKernel");
}

} // namespace es
