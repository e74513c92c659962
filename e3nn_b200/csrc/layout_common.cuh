// Helpers shared by every generated per-layout module (see include/e3nn_b200_layout.h).
#pragma once
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

// Declared here so that layouts without fused spherical harmonics still parse; the
// specialisations come from the generated sh_gen.cuh when a layout uses them.
template <int L> __device__ __forceinline__ void e3b_sh_fwd(float x, float y, float z, float* Y);
template <int L> __device__ __forceinline__ void e3b_sh_bwd(float x, float y, float z, const float* Y, float* g,
                                                            float& gx, float& gy, float& gz);

static inline char* e3b_layout_error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

static inline int e3b_layout_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(e3b_layout_error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

static inline int e3b_layout_check(const char* what) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return e3b_layout_fail(-2, "%s: %s", what, cudaGetErrorString(err));
    return 0;
}

// Y^0..Y^L ('component') of the unit vector along v; a zero vector gives (1, 0, ..., 0)
// exactly as torch's F.normalize followed by the polynomials does.
template <int L>
__device__ __forceinline__ void e3b_sh_unit(const float* __restrict__ v, float* __restrict__ Y) {
    if constexpr (L >= 0) {
        float x = v[0], y = v[1], z = v[2];
        const float inv = 1.0f / fmaxf(sqrtf(x * x + y * y + z * z), 1e-12f);
        e3b_sh_fwd<L>(x * inv, y * inv, z * inv, Y);
    }
}

// Cotangent gY of e3b_sh_unit's output -> cotangent of v (gY is clobbered).
template <int L>
__device__ __forceinline__ void e3b_sh_unit_bwd(float vx, float vy, float vz, float* __restrict__ gY, float& gx,
                                                float& gy, float& gz) {
    if constexpr (L >= 0) {
        const float len = sqrtf(vx * vx + vy * vy + vz * vz);
        const float inv = 1.0f / fmaxf(len, 1e-12f);
        const float x = vx * inv, y = vy * inv, z = vz * inv;
        float Y[(L + 1) * (L + 1)];
        e3b_sh_fwd<L>(x, y, z, Y);
        e3b_sh_bwd<L>(x, y, z, Y, gY, gx, gy, gz);
        if (len > 1e-12f) {
            const float dot = gx * x + gy * y + gz * z;
            gx = (gx - dot * x) * inv; gy = (gy - dot * y) * inv; gz = (gz - dot * z) * inv;
        } else {
            gx *= inv; gy *= inv; gz *= inv;
        }
    } else {
        gx = gy = gz = 0.0f;
    }
}

// Sum vals[0..N) over the G threads that share a row (G: power of two <= 32, or a multiple of 32).
// After the call (which contains one __syncthreads: every thread of the block must reach it)
// part[q * N + j] holds the sum over warp q of the group, q < max(1, G/32).
template <int G, int N>
__device__ __forceinline__ void e3b_group_reduce(float* vals, float* part, int u) {
    constexpr int W = G < 32 ? G : 32;
#pragma unroll
    for (int j = 0; j < N; ++j) {
        float v = vals[j];
#pragma unroll
        for (int o = W / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        vals[j] = v;
    }
    if ((u & (W - 1)) == 0) {
        const int q = u / 32;
#pragma unroll
        for (int j = 0; j < N; ++j) part[q * N + j] = vals[j];
    }
    __syncthreads();
}
