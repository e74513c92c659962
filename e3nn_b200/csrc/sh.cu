// Spherical harmonics of edge vectors: forward and vector-Jacobian product.
//
// One thread evaluates one vector with straight-line generated polynomials (sh_gen.cuh).
// The (lmax+1)^2 values per vector are transposed through shared memory (tiles of 128 vectors) so
// that every global access of the block is a contiguous, fully used line, moved 16 bytes per thread
// when (lmax+1)^2 is a multiple of 4; the 12-byte vectors are read and written directly (a warp's
// 384 bytes are contiguous).  The kernel is bound by HBM: 12 B in, 4*(lmax+1)^2 B out.
#include "common.cuh"
#include "sh_gen.cuh"

namespace e3b {

constexpr int kShTile = 128;

__device__ __forceinline__ float sh_scale(int normalization, int l) {
    // e3nn/o3/_spherical_harmonics.py:103-110
    if (normalization == E3B_SH_INTEGRAL) return 0.28209479177387814f;  // 1/sqrt(4 pi)
    if (normalization == E3B_SH_NORM) return 1.0f / sqrtf(static_cast<float>(2 * l + 1));
    return 1.0f;
}

template <int L>
__global__ void __launch_bounds__(kShTile) sh_fwd_kernel(const float* __restrict__ xyz, float* __restrict__ out,
                                                         int64_t n, int normalize, int normalization) {
    constexpr int NC = (L + 1) * (L + 1);
    constexpr int LD = kShTile + 1;  // padded leading dimension: conflict-free column writes
    extern __shared__ float smem[];
    float* s_out = smem + 3 * kShTile;  // [NC][LD]

    const int64_t e0 = static_cast<int64_t>(blockIdx.x) * kShTile;
    const int cnt = static_cast<int>(min(static_cast<int64_t>(kShTile), n - e0));
    const int t = threadIdx.x;

    if (t < cnt) {
        // three 4-byte loads per thread; the warp's 384 bytes are contiguous, every line is fully used
        const float* v = xyz + (e0 + t) * 3;
        float x = v[0], y = v[1], z = v[2];
        if (normalize) {
            const float inv = 1.0f / fmaxf(sqrtf(x * x + y * y + z * z), 1e-12f);
            x *= inv; y *= inv; z *= inv;
        }
        float Y[NC];
        e3b_sh_fwd<L>(x, y, z, Y);
#pragma unroll
        for (int l = 0; l <= L; ++l) {
            const float s = sh_scale(normalization, l);
#pragma unroll
            for (int m = 0; m < 2 * l + 1; ++m) s_out[(l * l + m) * LD + t] = Y[l * l + m] * s;
        }
    }
    __syncthreads();

    float* dst = out + e0 * NC;
    if (NC % 4 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        // 16-byte stores: four consecutive components of one vector per thread, consecutive threads consecutive addresses
        constexpr int Q = NC / 4 > 0 ? NC / 4 : 1;
        for (int i = t; i < cnt * Q; i += kShTile) {
            const int e = i / Q, c = (i - e * Q) * 4;
            reinterpret_cast<float4*>(dst)[i] =
                make_float4(s_out[c * LD + e], s_out[(c + 1) * LD + e], s_out[(c + 2) * LD + e], s_out[(c + 3) * LD + e]);
        }
    } else {
        for (int i = t; i < cnt * NC; i += kShTile) {
            const int e = i / NC, c = i - e * NC;
            dst[i] = s_out[c * LD + e];
        }
    }
}

template <int L>
__global__ void __launch_bounds__(kShTile) sh_bwd_kernel(const float* __restrict__ xyz, const float* __restrict__ gout,
                                                         float* __restrict__ gxyz, int64_t n, int normalize,
                                                         int normalization) {
    constexpr int NC = (L + 1) * (L + 1);
    constexpr int LD = kShTile + 1;
    extern __shared__ float smem[];
    float* s_g = smem + 3 * kShTile;    // [NC][LD]

    const int64_t e0 = static_cast<int64_t>(blockIdx.x) * kShTile;
    const int cnt = static_cast<int>(min(static_cast<int64_t>(kShTile), n - e0));
    const int t = threadIdx.x;

    const float* src = gout + e0 * NC;
    if (NC % 4 == 0 && (reinterpret_cast<uintptr_t>(gout) & 15) == 0) {
        constexpr int Q = NC / 4 > 0 ? NC / 4 : 1;
        for (int i = t; i < cnt * Q; i += kShTile) {   // 16-byte loads, transposed into shared memory
            const int e = i / Q, c = (i - e * Q) * 4;
            const float4 v = reinterpret_cast<const float4*>(src)[i];
            s_g[c * LD + e] = v.x; s_g[(c + 1) * LD + e] = v.y; s_g[(c + 2) * LD + e] = v.z; s_g[(c + 3) * LD + e] = v.w;
        }
    } else {
        for (int i = t; i < cnt * NC; i += kShTile) {
            const int e = i / NC, c = i - e * NC;
            s_g[c * LD + e] = src[i];
        }
    }
    __syncthreads();

    if (t < cnt) {
        const float* v = xyz + (e0 + t) * 3;
        const float vx = v[0], vy = v[1], vz = v[2];
        float x = vx, y = vy, z = vz, inv = 1.0f;
        const float len = sqrtf(vx * vx + vy * vy + vz * vz);
        if (normalize) {
            inv = 1.0f / fmaxf(len, 1e-12f);
            x *= inv; y *= inv; z *= inv;
        }
        float Y[NC], g[NC];
        e3b_sh_fwd<L>(x, y, z, Y);
#pragma unroll
        for (int l = 0; l <= L; ++l) {
            const float s = sh_scale(normalization, l);
#pragma unroll
            for (int m = 0; m < 2 * l + 1; ++m) g[l * l + m] = s_g[(l * l + m) * LD + t] * s;
        }
        float gx, gy, gz;
        e3b_sh_bwd<L>(x, y, z, Y, g, gx, gy, gz);
        if (normalize) {
            // d/dv of v / max(|v|, eps): projector for |v| > eps, plain 1/eps scaling below
            if (len > 1e-12f) {
                const float dot = gx * x + gy * y + gz * z;
                gx = (gx - dot * x) * inv; gy = (gy - dot * y) * inv; gz = (gz - dot * z) * inv;
            } else {
                gx *= inv; gy *= inv; gz *= inv;
            }
        }
        float* r = gxyz + (e0 + t) * 3;   // the warp's 384 bytes are contiguous
        r[0] = gx; r[1] = gy; r[2] = gz;
    }
}

template <int L>
int launch_sh(bool backward, const float* xyz, const float* gout, float* out, int64_t n, int normalize,
              int normalization, cudaStream_t stream) {
    constexpr int NC = (L + 1) * (L + 1);
    const size_t smem = sizeof(float) * (3 * kShTile + NC * (kShTile + 1));
    const unsigned blocks = static_cast<unsigned>(ceil_div(n, kShTile));
    if (!backward) {
        if (smem > 48 * 1024)
            E3B_CUDA_TRY(cudaFuncSetAttribute(sh_fwd_kernel<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        sh_fwd_kernel<L><<<blocks, kShTile, smem, stream>>>(xyz, out, n, normalize, normalization);
    } else {
        if (smem > 48 * 1024)
            E3B_CUDA_TRY(cudaFuncSetAttribute(sh_bwd_kernel<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        sh_bwd_kernel<L><<<blocks, kShTile, smem, stream>>>(xyz, gout, out, n, normalize, normalization);
    }
    return check_launch(backward ? "e3b_sh_bwd" : "e3b_sh_fwd");
}

int dispatch_sh(bool backward, const float* xyz, const float* gout, float* out, int64_t n, int lmax, int normalize,
                int normalization, void* stream) {
    if (n < 0 || lmax < 0 || lmax > E3B_SH_LMAX) return fail(E3B_ERR_ARG, "sh: lmax %d outside 0..%d or n < 0", lmax, E3B_SH_LMAX);
    if (normalization < 0 || normalization > 2) return fail(E3B_ERR_ARG, "sh: unknown normalization %d", normalization);
    if (n == 0) return E3B_OK;
    if (!xyz || !out || (backward && !gout)) return fail(E3B_ERR_ARG, "sh: null pointer");
    if (ceil_div(n, kShTile) > 0x7fffffffLL) return fail(E3B_ERR_ARG, "sh: n too large");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (lmax) {
#define E3B_CASE(L) case L: return launch_sh<L>(backward, xyz, gout, out, n, normalize, normalization, s);
        E3B_CASE(0) E3B_CASE(1) E3B_CASE(2) E3B_CASE(3) E3B_CASE(4) E3B_CASE(5) E3B_CASE(6)
        E3B_CASE(7) E3B_CASE(8) E3B_CASE(9) E3B_CASE(10) E3B_CASE(11) E3B_CASE(12)
#undef E3B_CASE
    }
    return fail(E3B_ERR_ARG, "sh: lmax");
}

}  // namespace e3b

extern "C" int e3b_sh_fwd(const float* xyz, float* out, int64_t n, int lmax, int normalize, int normalization,
                          void* stream) {
    return e3b::dispatch_sh(false, xyz, nullptr, out, n, lmax, normalize, normalization, stream);
}

extern "C" int e3b_sh_bwd(const float* xyz, const float* grad_out, float* grad_xyz, int64_t n, int lmax,
                          int normalize, int normalization, void* stream) {
    return e3b::dispatch_sh(true, xyz, grad_out, grad_xyz, n, lmax, normalize, normalization, stream);
}
