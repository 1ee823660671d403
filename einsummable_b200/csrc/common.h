// Shared host-side definitions of the es_b200 library.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "es_b200.h"

namespace es {

// Error carrying an es_status_t; converted to a return code at the C boundary.
struct es_error : std::runtime_error {
    int status;
    es_error(int status, std::string const& msg) : std::runtime_error(msg), status(status) {}
};

[[noreturn]] inline void fail(int status, std::string const& msg)
{
    throw es_error(status, msg);
}

inline int dtype_size(int d)
{
    switch (d) {
        case ES_F16: return 2;
        case ES_F32: return 4;
        case ES_F64: return 8;
        case ES_C64: return 8;
    }
    fail(ES_BAD_DESCRIPTOR, "unknown dtype code");
}

inline char const* dtype_name(int d)
{
    switch (d) {
        case ES_F16: return "f16";
        case ES_F32: return "f32";
        case ES_F64: return "f64";
        case ES_C64: return "c64";
    }
    return "?";
}

void set_last_error(std::string const& msg);

} // namespace es

#define ES_CUDA_CHECK(expr)                                                                        \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess) {                                                                   \
            ::es::fail(ES_CUDA_ERROR,                                                              \
                       std::string(#expr) + ": " + cudaGetErrorName(_e) + ": " +                   \
                           cudaGetErrorString(_e));                                                \
        }                                                                                          \
    } while (0)
