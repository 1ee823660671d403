// Runtime compilation (NVRTC, sm_100a) and loading of generated kernels.
#pragma once
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "common.h"

namespace es {

// Compiles CUDA C++ `source` for sm_100a; returns the cubin.  Throws
// ES_COMPILE_ERROR with the compiler log on failure.  Needs no GPU.
std::vector<char> nvrtc_compile(std::string const& source, std::string* log = nullptr);

// A loaded module on the current device.  Kernels are looked up by name and
// launched through the driver API.
struct module_t {
    void* cu_module = nullptr; // CUmodule
    ~module_t();
    void* function(std::string const& name); // CUfunction
private:
    std::map<std::string, void*> fns;
};

std::shared_ptr<module_t> load_module(std::vector<char> const& cubin);

// cuLaunchKernel wrapper.  args = array of pointers to the arguments.
void launch_function(void*    cu_function,
                     uint32_t grid,
                     uint32_t block,
                     uint32_t smem,
                     void*    stream,
                     void**   args);

// Driver entry points resolved through the runtime (no link-time libcuda dependency).
void* driver_entry(char const* name);

} // namespace es
