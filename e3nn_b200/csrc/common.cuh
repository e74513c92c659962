// Shared helpers of the C-ABI library: status codes, the per-thread error string, launch checks.
#pragma once
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/e3nn_b200.h"

namespace e3b {

// Per-thread message of the last failing call (returned by e3b_last_error()).
inline char* error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

inline int check_launch(const char* what) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(E3B_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
    return E3B_OK;
}

#define E3B_CUDA_TRY(expr)                                                                   \
    do {                                                                                     \
        cudaError_t _e = (expr);                                                             \
        if (_e != cudaSuccess) return ::e3b::fail(E3B_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

constexpr int kNumSMs = 148;  // B200

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace e3b
