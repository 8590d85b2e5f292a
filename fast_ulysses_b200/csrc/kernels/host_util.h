#pragma once
// Host-side helpers shared by the launchers: a thread-local error string and CUDA call checking
// that reports instead of aborting, because these launchers are called from inside a framework.
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdio>

namespace fu {

char* error_buffer();  // thread-local, 512 bytes

inline int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

}  // namespace fu

#define FU_CUDA_OK(expr)                                                                                      \
    do {                                                                                                      \
        cudaError_t fu_err__ = (expr);                                                                        \
        if (fu_err__ != cudaSuccess) {                                                                        \
            return ::fu::fail(FU_E_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(fu_err__),        \
                              __FILE__, __LINE__);                                                            \
        }                                                                                                     \
    } while (0)
