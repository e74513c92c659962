// Edge embedding of an interaction block in one kernel per direction: edge vectors from positions, the
// Bessel radial basis and the first (narrow) layer of the radial network with its activation.
//
//   edge_vec = pos[src] - pos[dst] + shift                        (e3nn/nn/models/gate_points_2101.py:328)
//   B_k      = sqrt(2/c) sin(k pi r / c) / r,  k = 1..num_basis   (e3nn/math/_bessel.py:6-37), or one of the
//              soft_one_hot_linspace families                       (e3nn/math/_soft_one_hot_linspace.py:100-140)
//   h        = act_scale * act((B @ W0) * w_scale) [* smooth_cutoff(r / end)]   (e3nn/nn/_fc.py:38-48, 70-88;
//                                                                 e3nn/nn/models/gate_points_2101.py:136-141)
//
// The reference evaluates these as a few dozen elementwise launches over [E, .] temporaries.  Here a warp
// takes 32 edges at a time: first one lane per edge (vector, radius and basis; the basis in fp64 through the
// Chebyshev recurrence of sin(k theta), because fp32 argument reduction alone costs a digit of the 1e-5
// error budget), then one edge per step with the hidden units across the lanes (coalesced rows of h).
// The gradient kernel recomputes the pre-activations instead of storing [E, hidden], reduces the basis
// cotangent over the lanes by recursive halving and adds the position gradient with float atomics.
#include "common.cuh"

namespace e3b {
namespace {

constexpr int kMaxBasis = 16;
constexpr int kEmbedWarps = 8;

enum Act { kSilu = 0, kTanh = 1, kRelu = 2, kIdentity = 3 };

__device__ __forceinline__ float act_fwd(int kind, float x) {
    switch (kind) {
        case kSilu: return x / (1.0f + expf(-x));
        case kTanh: return tanhf(x);
        case kRelu: return fmaxf(x, 0.0f);
        default: return x;
    }
}
__device__ __forceinline__ float act_grad(int kind, float x) {
    switch (kind) {
        case kSilu: {
            const float s = 1.0f / (1.0f + expf(-x));
            return s * (1.0f + x * (1.0f - s));
        }
        case kTanh: {
            const float t = tanhf(x);
            return 1.0f - t * t;
        }
        case kRelu: return x > 0.0f ? 1.0f : 0.0f;
        default: return 1.0f;
    }
}

struct EdgeGeom {
    float vx, vy, vz;
    double r;
    int64_t s, d;
};

// vector and radius of edge e (one lane per edge); indices out of range raise status 2 and are clamped
__device__ __forceinline__ EdgeGeom edge_geom(const float* __restrict__ pos, const int64_t* __restrict__ src,
                                              const int64_t* __restrict__ dst, const float* __restrict__ shift, int64_t e,
                                              int64_t num_nodes, int* status) {
    EdgeGeom g;
    g.s = src[e];
    g.d = dst[e];
    if (g.s < 0 || g.s >= num_nodes || g.d < 0 || g.d >= num_nodes) {
        atomicExch(status, 2);
        g.s = g.s < 0 ? 0 : (g.s >= num_nodes ? num_nodes - 1 : g.s);
        g.d = g.d < 0 ? 0 : (g.d >= num_nodes ? num_nodes - 1 : g.d);
    }
    g.vx = pos[g.s * 3] - pos[g.d * 3];
    g.vy = pos[g.s * 3 + 1] - pos[g.d * 3 + 1];
    g.vz = pos[g.s * 3 + 2] - pos[g.d * 3 + 2];
    if (shift) {
        g.vx += shift[e * 3];
        g.vy += shift[e * 3 + 1];
        g.vz += shift[e * 3 + 2];
    }
    g.r = sqrt(static_cast<double>(g.vx) * g.vx + static_cast<double>(g.vy) * g.vy + static_cast<double>(g.vz) * g.vz);
    return g;
}

// Parameters of the radial embedding, passed by value to the kernels.
//   kind 0: e3nn.math.bessel(r, nb, end)                         (e3nn/math/_bessel.py:6-37)
//   kind 1-5: soft_one_hot_linspace(r, start, end, nb, basis, cutoff) with basis gaussian, cosine, smooth_finite,
//             fourier, bessel                                     (e3nn/math/_soft_one_hot_linspace.py:100-140)
//   scale: factor on every basis value (models multiply by sqrt(nb));
//   envelope 1: h is multiplied by smooth_cutoff(r / end)          (e3nn/nn/models/gate_points_2101.py:136-141)
struct RadialSpec {
    int kind, cutoff, envelope, nb;
    double start, end, scale;
};

__device__ __forceinline__ double soft_unit_step(double x) { return x > 0.0 ? exp(-1.0 / x) : 0.0; }
__device__ __forceinline__ double soft_unit_step_grad(double x) { return x > 0.0 ? exp(-1.0 / x) / (x * x) : 0.0; }

// basis[k] (and optionally d basis[k] / dr), k = 0..nb-1, evaluated in fp64 and rounded once
__device__ __forceinline__ void radial_basis(const RadialSpec& sp, double r, float* basis, float* dbasis) {
    const int nb = sp.nb;
    const double pi = 3.14159265358979323846;
    if (sp.kind == 0 || sp.kind == 5) {
        // sqrt(2/c) sin(k pi x / c) / x: sin(k theta), cos(k theta) by the Chebyshev recurrence
        const double x = sp.kind == 0 ? r : r - sp.start;
        const double c = sp.kind == 0 ? sp.end : sp.end - sp.start;
        const double c0 = sqrt(2.0 / c) * sp.scale, a = pi / c;
        const bool inside = sp.kind == 0 || !sp.cutoff || (x > 0.0 && x < c);
        if (x == 0.0 || !inside) {
            for (int k = 1; k <= nb; ++k) {
                basis[k - 1] = static_cast<float>(inside ? c0 * k * a : 0.0);   // the x -> 0 limit (kind 0 defines it so)
                if (dbasis) dbasis[k - 1] = 0.0f;
            }
            return;
        }
        double s1, c1;
        sincos(a * x, &s1, &c1);
        const double inv = 1.0 / x;
        double s_prev = 0.0, s_cur = s1, c_prev = 1.0, c_cur = c1;
        for (int k = 1; k <= nb; ++k) {
            basis[k - 1] = static_cast<float>(c0 * s_cur * inv);
            if (dbasis) dbasis[k - 1] = static_cast<float>(c0 * (k * a * c_cur * x - s_cur) * inv * inv);
            const double s_next = 2.0 * c1 * s_cur - s_prev, c_next = 2.0 * c1 * c_cur - c_prev;
            s_prev = s_cur; s_cur = s_next;
            c_prev = c_cur; c_cur = c_next;
        }
        return;
    }
    if (sp.kind == 4) {   // fourier
        const double span = sp.end - sp.start, x = (r - sp.start) / span;
        const double norm = sp.scale / sqrt(0.25 + nb / 2.0);
        for (int k = 0; k < nb; ++k) {
            double f, df;
            if (!sp.cutoff) {
                f = cos(pi * k * x); df = -pi * k * sin(pi * k * x) / span;
            } else {
                const bool inside = x > 0.0 && x < 1.0;
                f = inside ? sin(pi * (k + 1) * x) : 0.0;
                df = inside ? pi * (k + 1) * cos(pi * (k + 1) * x) / span : 0.0;
            }
            basis[k] = static_cast<float>(norm * f);
            if (dbasis) dbasis[k] = static_cast<float>(norm * df);
        }
        return;
    }
    // gaussian, cosine, smooth_finite on nb centres: linspace(start, end, nb), or the interior of nb + 2 points
    const double step = sp.cutoff ? (sp.end - sp.start) / (nb + 1) : (nb > 1 ? (sp.end - sp.start) / (nb - 1) : 0.0);
    for (int k = 0; k < nb; ++k) {
        const double centre = sp.start + (sp.cutoff ? k + 1 : k) * step;
        const double d = (r - centre) / step;
        double f, df;
        if (sp.kind == 1) {
            f = exp(-d * d) / 1.12; df = f * (-2.0 * d);
        } else if (sp.kind == 2) {
            const bool inside = d < 1.0 && d > -1.0;
            f = inside ? cos(0.5 * pi * d) : 0.0; df = inside ? -0.5 * pi * sin(0.5 * pi * d) : 0.0;
        } else {
            const double cst = 8.433573722839355;   // 1.14136 e^2 as the reference evaluates it (in float32)
            const double a1 = soft_unit_step(d + 1.0), a2 = soft_unit_step(1.0 - d);
            f = cst * a1 * a2;
            df = cst * (soft_unit_step_grad(d + 1.0) * a2 - a1 * soft_unit_step_grad(1.0 - d));
        }
        basis[k] = static_cast<float>(sp.scale * f);
        if (dbasis) dbasis[k] = static_cast<float>(sp.scale * df / step);
    }
}

// smooth_cutoff(r / end) and its derivative with respect to r
__device__ __forceinline__ void radial_envelope(const RadialSpec& sp, double r, float& env, float& denv) {
    env = 1.0f; denv = 0.0f;
    if (sp.envelope != 1) return;
    const double u = 2.0 * (r / sp.end - 1.0), pi = 3.14159265358979323846;
    if (u > 0.0) { env = 0.0f; return; }
    if (u < -1.0) return;
    env = static_cast<float>(0.5 * (1.0 - cos(pi * u)));
    denv = static_cast<float>(0.5 * pi * sin(pi * u) * 2.0 / sp.end);
}

// H2 = hidden / 32 hidden units per lane (unit j of a lane is column lane + 32 j); NB = basis count padded to 8 or 16
template <int H2, int NB>
__global__ void __launch_bounds__(kEmbedWarps * 32) radial_embed_fwd_kernel(
        const float* __restrict__ pos, const int64_t* __restrict__ src, const int64_t* __restrict__ dst,
        const float* __restrict__ shift, const float* __restrict__ w0, int64_t num_edges, int64_t num_nodes, RadialSpec sp,
        float w_scale, float act_scale, int act, float* __restrict__ edge_vec, float* __restrict__ h,
        int* __restrict__ status) {
    __shared__ float s_basis[kEmbedWarps][32][kMaxBasis + 1];
    __shared__ float s_env[kEmbedWarps][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = sp.nb;
    constexpr int H = 32 * H2;
    float w[NB][H2];
#pragma unroll
    for (int k = 0; k < NB; ++k)
#pragma unroll
        for (int j = 0; j < H2; ++j) w[k][j] = k < nb ? w0[k * H + lane + 32 * j] * w_scale : 0.0f;
    const int64_t batches = (num_edges + 31) / 32;
    for (int64_t b = static_cast<int64_t>(blockIdx.x) * kEmbedWarps + warp; b < batches;
         b += static_cast<int64_t>(gridDim.x) * kEmbedWarps) {
        const int64_t e = b * 32 + lane;
        if (e < num_edges) {
            const EdgeGeom g = edge_geom(pos, src, dst, shift, e, num_nodes, status);
            edge_vec[e * 3] = g.vx; edge_vec[e * 3 + 1] = g.vy; edge_vec[e * 3 + 2] = g.vz;
            radial_basis(sp, g.r, s_basis[warp][lane], nullptr);
            float env, denv;
            radial_envelope(sp, g.r, env, denv);
            s_env[warp][lane] = env;
        }
        __syncwarp();
        const int count = static_cast<int>(num_edges - b * 32 < 32 ? num_edges - b * 32 : 32);
        for (int i = 0; i < count; ++i) {
            float pre[H2];
#pragma unroll
            for (int j = 0; j < H2; ++j) pre[j] = 0.0f;
#pragma unroll
            for (int k = 0; k < NB; ++k) {
                if (k < nb) {
                    const float bk = s_basis[warp][i][k];
#pragma unroll
                    for (int j = 0; j < H2; ++j) pre[j] = fmaf(bk, w[k][j], pre[j]);
                }
            }
            float* hrow = h + (b * 32 + i) * H;
#pragma unroll
            for (int j = 0; j < H2; ++j) hrow[lane + 32 * j] = (s_env[warp][i] * act_scale) * act_fwd(act, pre[j]);
        }
        __syncwarp();
    }
}

// one step of a recursive-halving reduction over the lanes: lanes with bit O set keep the upper half
template <int O, int HALF>
__device__ __forceinline__ void halve(float* v, int lane) {
    const bool up = (lane & O) != 0;
#pragma unroll
    for (int i = 0; i < HALF; ++i) {
        const float send = up ? v[i] : v[i + HALF];
        const float keep = up ? v[i + HALF] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, O);
    }
}

template <int H2, int NB>
__global__ void __launch_bounds__(kEmbedWarps * 32) radial_embed_bwd_kernel(
        const float* __restrict__ pos, const int64_t* __restrict__ src, const int64_t* __restrict__ dst,
        const float* __restrict__ shift, const float* __restrict__ w0, const float* __restrict__ grad_h,
        const float* __restrict__ grad_vec, int64_t num_edges, int64_t num_nodes, RadialSpec sp, float w_scale,
        float act_scale, int act, float* __restrict__ grad_pos, int* __restrict__ status) {
    __shared__ float s_basis[kEmbedWarps][32][kMaxBasis + 1];
    __shared__ float s_cot[kEmbedWarps][32][kMaxBasis + 1];
    __shared__ float s_env[kEmbedWarps][32];     // envelope value of the batch's edges
    __shared__ float s_genv[kEmbedWarps][32];    // cotangent of the envelope
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = sp.nb;
    constexpr int H = 32 * H2;
    float w[NB][H2];
#pragma unroll
    for (int k = 0; k < NB; ++k)
#pragma unroll
        for (int j = 0; j < H2; ++j) w[k][j] = k < nb ? w0[k * H + lane + 32 * j] * w_scale : 0.0f;
    const int64_t batches = (num_edges + 31) / 32;
    for (int64_t b = static_cast<int64_t>(blockIdx.x) * kEmbedWarps + warp; b < batches;
         b += static_cast<int64_t>(gridDim.x) * kEmbedWarps) {
        const int64_t e = b * 32 + lane;
        EdgeGeom g;
        float env = 1.0f, denv = 0.0f;
        float dbasis[kMaxBasis];
#pragma unroll
        for (int k = 0; k < kMaxBasis; ++k) dbasis[k] = 0.0f;
        if (e < num_edges) {
            g = edge_geom(pos, src, dst, shift, e, num_nodes, status);
            radial_basis(sp, g.r, s_basis[warp][lane], dbasis);
            radial_envelope(sp, g.r, env, denv);
            s_env[warp][lane] = env;
        }
        __syncwarp();
        const int count = static_cast<int>(num_edges - b * 32 < 32 ? num_edges - b * 32 : 32);
        // cotangent rows are read one edge ahead of their use: the load of edge i + 1 is in flight during edge i
        float gh_next[H2];
#pragma unroll
        for (int j = 0; j < H2; ++j) gh_next[j] = count > 0 ? grad_h[(b * 32) * H + lane + 32 * j] : 0.0f;
        for (int i = 0; i < count; ++i) {
            float gh_cur[H2];
#pragma unroll
            for (int j = 0; j < H2; ++j) gh_cur[j] = gh_next[j];
            if (i + 1 < count) {
#pragma unroll
                for (int j = 0; j < H2; ++j) gh_next[j] = grad_h[(b * 32 + i + 1) * H + lane + 32 * j];
            }
            float pre[H2];
#pragma unroll
            for (int j = 0; j < H2; ++j) pre[j] = 0.0f;
#pragma unroll
            for (int k = 0; k < NB; ++k) {
                if (k < nb) {
                    const float bk = s_basis[warp][i][k];
#pragma unroll
                    for (int j = 0; j < H2; ++j) pre[j] = fmaf(bk, w[k][j], pre[j]);
                }
            }
            float cot[NB];
#pragma unroll
            for (int k = 0; k < NB; ++k) cot[k] = 0.0f;
            const float envi = s_env[warp][i];
            float genv = 0.0f;
#pragma unroll
            for (int j = 0; j < H2; ++j) {
                const float gh = gh_cur[j];
                if (sp.envelope) genv = fmaf(gh * act_scale, act_fwd(act, pre[j]), genv);
                const float dpre = gh * (envi * act_scale) * act_grad(act, pre[j]);
#pragma unroll
                for (int k = 0; k < NB; ++k) cot[k] = fmaf(w[k][j], dpre, cot[k]);
            }
            if (NB == 16) {
                halve<16, NB / 2>(cot, lane); halve<8, 4>(cot, lane); halve<4, 2>(cot, lane); halve<2, 1>(cot, lane);
                cot[0] += __shfl_xor_sync(0xffffffffu, cot[0], 1);
                // after the four halvings lane l holds component (l >> 1) & 15 (bit 4 chose the upper 8, bit 3 the upper 4, ...)
                if ((lane & 1) == 0) s_cot[warp][i][(lane >> 1) & 15] = cot[0];
            } else {
                halve<16, 4>(cot, lane); halve<8, 2>(cot, lane); halve<4, 1>(cot, lane);
                cot[0] += __shfl_xor_sync(0xffffffffu, cot[0], 2);
                cot[0] += __shfl_xor_sync(0xffffffffu, cot[0], 1);
                // three halvings over lane bits 4, 3, 2: lane l holds component (l >> 2) & 7
                if ((lane & 3) == 0) s_cot[warp][i][(lane >> 2) & 7] = cot[0];
            }
            if (sp.envelope) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) genv += __shfl_xor_sync(0xffffffffu, genv, o);
                if (lane == 0) s_genv[warp][i] = genv;
            }
        }
        __syncwarp();
        if (e < num_edges) {
            double dr = sp.envelope ? static_cast<double>(s_genv[warp][lane]) * denv : 0.0;
#pragma unroll
            for (int k = 0; k < kMaxBasis; ++k)
                if (k < nb) dr += static_cast<double>(s_cot[warp][lane][k]) * dbasis[k];
            float gx = 0.0f, gy = 0.0f, gz = 0.0f;
            if (grad_vec) { gx = grad_vec[e * 3]; gy = grad_vec[e * 3 + 1]; gz = grad_vec[e * 3 + 2]; }
            if (g.r > 0.0) {
                const double f = dr / g.r;
                gx += static_cast<float>(f * g.vx); gy += static_cast<float>(f * g.vy); gz += static_cast<float>(f * g.vz);
            }
            atomicAdd(grad_pos + g.s * 3, gx); atomicAdd(grad_pos + g.s * 3 + 1, gy); atomicAdd(grad_pos + g.s * 3 + 2, gz);
            atomicAdd(grad_pos + g.d * 3, -gx); atomicAdd(grad_pos + g.d * 3 + 1, -gy); atomicAdd(grad_pos + g.d * 3 + 2, -gz);
        }
        __syncwarp();
    }
}

int check_embed_args(int64_t num_edges, int64_t num_nodes, int num_basis, int hidden, int act) {
    if (num_edges < 0 || num_nodes < 0) return fail(E3B_ERR_ARG, "radial_embed: negative size");
    if (num_basis < 1 || num_basis > kMaxBasis) return fail(E3B_ERR_ARG, "radial_embed: num_basis must be in 1..%d", kMaxBasis);
    if (hidden != 32 && hidden != 64 && hidden != 96 && hidden != 128)
        return fail(E3B_ERR_ARG, "radial_embed: hidden must be 32, 64, 96 or 128");
    if (act < 0 || act > kIdentity) return fail(E3B_ERR_ARG, "radial_embed: unknown activation %d", act);
    return E3B_OK;
}

int embed_grid(int64_t num_edges) {
    const int64_t want = ceil_div(ceil_div(num_edges, 32), kEmbedWarps);
    const int64_t cap = static_cast<int64_t>(kNumSMs) * 8;
    return static_cast<int>(want < cap ? want : cap);
}

}  // namespace
}  // namespace e3b

namespace e3b {
namespace {
int make_spec(RadialSpec* sp, int basis, int cutoff, int envelope, int num_basis, float start, float end, float basis_scale) {
    if (basis < 0 || basis > 5) return fail(E3B_ERR_ARG, "radial_embed: unknown basis %d", basis);
    if (envelope < 0 || envelope > 1) return fail(E3B_ERR_ARG, "radial_embed: unknown envelope %d", envelope);
    if (!(end > start)) return fail(E3B_ERR_ARG, "radial_embed: end must be larger than start");
    if (basis == 0 && start != 0.0f) return fail(E3B_ERR_ARG, "radial_embed: the plain Bessel basis starts at 0");
    if ((basis >= 1 && basis <= 3) && !cutoff && num_basis < 2) return fail(E3B_ERR_ARG, "radial_embed: this basis needs two centres");
    sp->kind = basis; sp->cutoff = cutoff != 0; sp->envelope = envelope; sp->nb = num_basis;
    sp->start = start; sp->end = end; sp->scale = basis_scale;
    return E3B_OK;
}
}  // namespace
}  // namespace e3b

extern "C" int e3b_radial_embed_fwd(const float* pos, const int64_t* edge_src, const int64_t* edge_dst, const float* shift,
                                    const float* w0, int64_t num_edges, int64_t num_nodes, int num_basis, int hidden,
                                    int basis, int cutoff, int envelope, float start, float end, float basis_scale,
                                    float w_scale, float act_scale, int act, float* edge_vec, float* h,
                                    int32_t* status, void* stream) {
    using namespace e3b;
    if (int rc = check_embed_args(num_edges, num_nodes, num_basis, hidden, act)) return rc;
    RadialSpec sp;
    if (int rc = make_spec(&sp, basis, cutoff, envelope, num_basis, start, end, basis_scale)) return rc;
    if (num_edges == 0) return E3B_OK;
    if (!pos || !edge_src || !edge_dst || !w0 || !edge_vec || !h || !status) return fail(E3B_ERR_ARG, "radial_embed_fwd: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int grid = embed_grid(num_edges), threads = kEmbedWarps * 32;
#define E3B_LAUNCH(H2)                                                                                                   \
    if (num_basis <= 8) E3B_LAUNCH_NB(H2, 8); else E3B_LAUNCH_NB(H2, 16)
#define E3B_LAUNCH_NB(H2, NBP)                                                                                           \
    radial_embed_fwd_kernel<H2, NBP><<<grid, threads, 0, s>>>(pos, edge_src, edge_dst, shift, w0, num_edges, num_nodes, sp, \
                                                              w_scale, act_scale, act, edge_vec, h, status)
    switch (hidden / 32) {
        case 1: E3B_LAUNCH(1); break;
        case 2: E3B_LAUNCH(2); break;
        case 3: E3B_LAUNCH(3); break;
        default: E3B_LAUNCH(4); break;
    }
#undef E3B_LAUNCH
#undef E3B_LAUNCH_NB
    return check_launch("radial_embed_fwd");
}

extern "C" int e3b_radial_embed_bwd(const float* pos, const int64_t* edge_src, const int64_t* edge_dst, const float* shift,
                                    const float* w0, const float* grad_h, const float* grad_edge_vec, int64_t num_edges,
                                    int64_t num_nodes, int num_basis, int hidden, int basis, int cutoff, int envelope,
                                    float start, float end, float basis_scale, float w_scale, float act_scale, int act,
                                    float* grad_pos, int32_t* status, void* stream) {
    using namespace e3b;
    if (int rc = check_embed_args(num_edges, num_nodes, num_basis, hidden, act)) return rc;
    RadialSpec sp;
    if (int rc = make_spec(&sp, basis, cutoff, envelope, num_basis, start, end, basis_scale)) return rc;
    if (num_edges == 0) return E3B_OK;
    if (!pos || !edge_src || !edge_dst || !w0 || !grad_h || !grad_pos || !status) return fail(E3B_ERR_ARG, "radial_embed_bwd: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int grid = embed_grid(num_edges), threads = kEmbedWarps * 32;
#define E3B_LAUNCH(H2)                                                                                                   \
    if (num_basis <= 8) E3B_LAUNCH_NB(H2, 8); else E3B_LAUNCH_NB(H2, 16)
#define E3B_LAUNCH_NB(H2, NBP)                                                                                           \
    radial_embed_bwd_kernel<H2, NBP><<<grid, threads, 0, s>>>(pos, edge_src, edge_dst, shift, w0, grad_h, grad_edge_vec,  \
                                                              num_edges, num_nodes, sp, w_scale, act_scale, act, grad_pos, status)
    switch (hidden / 32) {
        case 1: E3B_LAUNCH(1); break;
        case 2: E3B_LAUNCH(2); break;
        case 3: E3B_LAUNCH(3); break;
        default: E3B_LAUNCH(4); break;
    }
#undef E3B_LAUNCH
#undef E3B_LAUNCH_NB
    return check_launch("radial_embed_bwd");
}
