// Host-side helpers shared by the C-ABI translation units.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/minfer_b200.h"

namespace minf {

char* last_error_buffer();  // thread-local, 512 bytes

inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

#define MINF_CUDA_OK(expr)                                                              \
    do {                                                                                \
        cudaError_t _e = (expr);                                                        \
        if (_e != cudaSuccess)                                                          \
            return ::minf::fail(MINF_E_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

#define MINF_LAUNCH_OK(name)                                                            \
    do {                                                                                \
        cudaError_t _e = cudaGetLastError();                                            \
        if (_e != cudaSuccess)                                                          \
            return ::minf::fail(MINF_E_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(_e)); \
    } while (0)

}  // namespace minf
