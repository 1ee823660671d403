#include "jit.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <nvrtc.h>

namespace es {

std::vector<char> nvrtc_compile(std::string const& source, std::string* log_out)
{
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
    cu_check(driver().launch_kernel(
                 (CUfunction)fn, grid, 1, 1, block, 1, 1, smem, (CUstream)stream, args, nullptr),
             "cuLaunchKernel");
}

} // namespace es
