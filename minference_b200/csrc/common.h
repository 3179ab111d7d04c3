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

// Range-checked debug build (-DMINF_BOUNDS, `python -m minference_b200.build --bounds`): every store of the index
// kernels and every plan-derived coordinate of the attention kernel is checked against the capacity of its
// destination; a violation sets bit 3 of status[MINF_ST_ERROR] and the access is skipped.  Nothing traps.
#ifdef MINF_BOUNDS
#define MINF_IN_BOUNDS(status, cond) ((cond) ? true : (atomicOr((status) + MINF_ST_ERROR, 8), false))
#else
#define MINF_IN_BOUNDS(status, cond) (true)
#endif

}  // namespace minf
