// fp32 CUDA-core evaluation of weight-shared contractions: 'uvw' tensor-product paths and the
// per-irrep Linear.  Table driven (no per-layout code): the host describes the contraction as a
// "dense plan" and this kernel evaluates, per output irrep ("group"),
//
//     out[z, w, k] = sum_K  A[z, k, K] * W[wbase(K) + w * wstride]
//     A[z, k, K]   = sum_{(i,j,c) in cg(path(K), k)}  c * x1[z, x1off(K) + i] * x2[z, x2off(K) + j]
//
// where K runs over the (path, u, v) triples feeding that output irrep.  A block stages the A
// rows of a tile of z in shared memory (phase 1) and then runs a register-tiled FFMA product
// against W, which stays L2-resident (phase 2).  This is the fp32-accurate mode (<= 1e-5 x RMS);
// the tensor-core mode lives in uvw_tc.cu.
//
// Plan layout (int32 words, floats bit-cast), built by e3nn_b200/o3/_dense_plan.py:
//   [0] magic 0x65336250  [1] d1  [2] d2  [3] dout  [4] n_groups  [5] n_paths  [6] total words
//   [7] off_groups [8] off_kent [9] off_pathk [10] off_cg   [11] max K over groups
//   groups  : n_groups x 6 : out_off, mul_out, dim3, K, kent_start, w_stride
//   kent    : sum K   x 4 : path, x1off, x2off (-1: factor 1), wbase
//   pathk   : per path, per k (path base in word [off_pathk + path]) -> (cg_start, cg_count) pairs
//   cg      : triples (i, j, coef)
#include "common.cuh"
#include "gate_act.cuh"

namespace e3b {

constexpr int kDenseMagic = 0x65336250;
constexpr int kDenseThreads = 256;
constexpr int kTM = 8;   // rows per thread
constexpr int kTN = 4;   // output channels per thread
constexpr int kRowsPerPass = (kDenseThreads / 32) * kTM;  // 64
constexpr int kColsPerPass = 32 * kTN;                    // 128
constexpr int kKBlock = 32;                               // summation block of the contraction index

struct DenseGroup { int out_off, mul_out, dim3, K, kent_start, w_stride; };

// Gate applied where the contraction's result is still in registers (Linear followed by Gate).  Column c of the
// contraction's output row is described by tbl[4 c ..] = {kind, destination column, activation, gate slot} and
// cst[c]: kind 0 = scalar: final[z, dst] = cst * act(v); kind 2 = gate: gates[z, slot] = cst * act(v);
// kind 1 = gated component: final[z, dst] = v * gates[z, slot] (its gate's launch ran before); kind 3 = unused.
struct DenseGateEpilogue {
    const int32_t* tbl;
    const float* cst;
    float* gates;       // [rows, n_slots] activated gates
    float* final_out;   // [rows, dout_final]
    int n_slots, dout_final;
};

template <bool VEC4>
__global__ void __launch_bounds__(kDenseThreads) dense_fwd_kernel(const int32_t* __restrict__ plan,
        const float* __restrict__ x1, const float* __restrict__ x2, const float* __restrict__ W,
        float* __restrict__ out, int64_t Z, int group, int rows_z /* z per tile */, int accumulate,
        int64_t w_row_stride /* 0: shared weights, else floats between the weight rows of consecutive z */,
        int k_chunk /* entries of the contraction staged at a time (= K when the whole A tile fits) */,
        DenseGateEpilogue ep /* tbl == nullptr: plain store */) {
    extern __shared__ float smem[];
    const int d1 = plan[1], d2 = plan[2], dout = plan[3];
    const int32_t* gp = plan + plan[7] + 6 * group;
    const DenseGroup g{gp[0], gp[1], gp[2], gp[3], gp[4], gp[5]};
    const int32_t* kent = plan + plan[8] + 4 * g.kent_start;
    const int32_t* pathk_dir = plan + plan[9];
    const int32_t* cg = plan + plan[10];

    const int RT = rows_z * g.dim3;                 // rows of the A tile (<= kRowsPerPass)
    float* sA = smem;                               // [k_chunk][kRowsPerPass]
    int* sW = reinterpret_cast<int*>(smem + static_cast<size_t>(k_chunk) * kRowsPerPass);  // [k_chunk] wbase
    const bool chunked = k_chunk < g.K;

    const int tid = threadIdx.x;
    for (int kk = tid; kk < k_chunk; kk += kDenseThreads) sW[kk] = kent[4 * kk + 3];   // (chunked: reloaded per chunk)

    const int64_t tiles = (Z + rows_z - 1) / rows_z;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t z0 = tile * rows_z;
        // ---- phase 1: A tile, entries [kc0, kc1) of the contraction.  element index = (kk - kc0) * RT + r,
        // r = zl * dim3 + k.  When the contraction does not fit shared memory it is staged in chunks and
        // the accumulators of phase 2 live across the chunks (phase 1 is then repeated per 128-column pass).
        auto stage = [&](int kc0, int kc1) {
            __syncthreads();
            if (chunked)
                for (int kl = tid; kl < kc1 - kc0; kl += kDenseThreads) sW[kl] = kent[4 * (kc0 + kl) + 3];
            const int total = (kc1 - kc0) * RT;
            for (int idx = tid; idx < total; idx += kDenseThreads) {
                const int kl = idx / RT, r = idx - kl * RT, kk = kc0 + kl;
                const int zl = r / g.dim3, k = r - zl * g.dim3;
                const int64_t z = z0 + zl;
                float a = 0.0f;
                if (z < Z) {
                    const int path = kent[4 * kk], x1off = kent[4 * kk + 1], x2off = kent[4 * kk + 2];
                    const int32_t* pk = plan + pathk_dir[path] + 2 * k;
                    const int cstart = pk[0], ccount = pk[1];
                    const float* xr = x1 + z * d1 + x1off;
                    const float* yr = x2off >= 0 ? x2 + z * d2 + x2off : nullptr;
                    for (int c = 0; c < ccount; ++c) {
                        const int32_t* t = cg + 3 * (cstart + c);
                        const float coef = __int_as_float(t[2]);
                        a = fmaf(coef * xr[t[0]], yr ? yr[t[1]] : 1.0f, a);
                    }
                }
                sA[kl * kRowsPerPass + r] = a;
            }
            // rows RT..kRowsPerPass of the tile are never read by live outputs
            __syncthreads();
        };
        if (!chunked) stage(0, g.K);
        // ---- phase 2: out rows x channels, passes of 64 rows (one pass: RT <= 64) x 128 channels
        const int tx = tid & 31, ty = tid >> 5;
        const int r0 = ty * kTM;
        for (int c0 = 0; c0 < g.mul_out; c0 += kColsPerPass) {
            const int w0 = c0 + tx * kTN;
            float acc[kTM][kTN];
#pragma unroll
            for (int i = 0; i < kTM; ++i)
#pragma unroll
                for (int j = 0; j < kTN; ++j) acc[i][j] = 0.0f;
            for (int kc0 = 0; kc0 < g.K; kc0 += k_chunk) {
            const int kc1 = min(kc0 + k_chunk, g.K);
            if (chunked) stage(kc0, kc1);
            if (r0 < RT && w0 < g.mul_out && w_row_stride != 0) {
                // per-row weights: every row of the tile reads its own weight vector
                int64_t wrow[kTM];
#pragma unroll
                for (int i = 0; i < kTM; ++i) {
                    const int64_t z = z0 + (r0 + i) / g.dim3;
                    wrow[i] = (z < Z ? z : 0) * w_row_stride;
                }
                for (int kk = kc0; kk < kc1; ++kk) {
                    const float4 a0 = *reinterpret_cast<const float4*>(sA + (kk - kc0) * kRowsPerPass + r0);
                    const float4 a1 = *reinterpret_cast<const float4*>(sA + (kk - kc0) * kRowsPerPass + r0 + 4);
                    const float a[kTM] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
                    for (int i = 0; i < kTM; ++i) {
                        if (r0 + i >= RT) continue;
                        const float* wp = W + wrow[i] + sW[kk - kc0];
#pragma unroll
                        for (int j = 0; j < kTN; ++j)
                            if (w0 + j < g.mul_out)
                                acc[i][j] = fmaf(a[i], __ldg(wp + static_cast<int64_t>(w0 + j) * g.w_stride), acc[i][j]);
                    }
                }
            } else if (r0 < RT && w0 < g.mul_out) {
                // K is summed in blocks of kKBlock with a fresh partial accumulator per block: the fp32
                // rounding error then grows with sqrt(kKBlock) + sqrt(K / kKBlock) instead of sqrt(K)
                for (int kb = kc0; kb < kc1; kb += kKBlock) {
                    float part[kTM][kTN];
#pragma unroll
                    for (int i = 0; i < kTM; ++i)
#pragma unroll
                        for (int j = 0; j < kTN; ++j) part[i][j] = 0.0f;
                    const int kend = min(kb + kKBlock, kc1);
#pragma unroll 4
                    for (int kk = kb; kk < kend; ++kk) {
                        const float4 a0 = *reinterpret_cast<const float4*>(sA + (kk - kc0) * kRowsPerPass + r0);
                        const float4 a1 = *reinterpret_cast<const float4*>(sA + (kk - kc0) * kRowsPerPass + r0 + 4);
                        const float a[kTM] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                        float wv[kTN];
                        const float* wp = W + sW[kk - kc0];
                        if (VEC4) {
                            const float4 t = __ldg(reinterpret_cast<const float4*>(wp + w0));
                            wv[0] = t.x; wv[1] = t.y; wv[2] = t.z; wv[3] = t.w;
                        } else {
#pragma unroll
                            for (int j = 0; j < kTN; ++j)
                                wv[j] = (w0 + j < g.mul_out) ? __ldg(wp + static_cast<int64_t>(w0 + j) * g.w_stride) : 0.0f;
                        }
#pragma unroll
                        for (int i = 0; i < kTM; ++i)
#pragma unroll
                            for (int j = 0; j < kTN; ++j) part[i][j] = fmaf(a[i], wv[j], part[i][j]);
                    }
#pragma unroll
                    for (int i = 0; i < kTM; ++i)
#pragma unroll
                        for (int j = 0; j < kTN; ++j) acc[i][j] += part[i][j];
                }
            }
            }
            if (r0 < RT && w0 < g.mul_out) {
                // gated epilogue: one table entry per channel (the components of a channel are consecutive columns
                // with consecutive destinations and share the gate), fetched once per pass
                int e_kind[kTN], e_dst[kTN], e_act[kTN], e_slot[kTN];
                float e_cst[kTN];
                if (ep.tbl != nullptr) {
#pragma unroll
                    for (int j = 0; j < kTN; ++j) {
                        const int c = g.out_off + (w0 + j < g.mul_out ? w0 + j : 0) * g.dim3;
                        const int4 t = *reinterpret_cast<const int4*>(ep.tbl + 4 * c);
                        e_kind[j] = t.x; e_dst[j] = t.y; e_act[j] = t.z; e_slot[j] = t.w;
                        e_cst[j] = ep.cst[c];
                    }
                }
#pragma unroll
                for (int i = 0; i < kTM; ++i) {
                    const int r = r0 + i;
                    if (r >= RT) continue;
                    const int zl = r / g.dim3, k = r - zl * g.dim3;
                    const int64_t z = z0 + zl;
                    if (z >= Z) continue;
                    float* orow = out + z * dout + g.out_off;
#pragma unroll
                    for (int j = 0; j < kTN; ++j) {
                        if (w0 + j >= g.mul_out) continue;
                        if (ep.tbl == nullptr) {
                            float* p = orow + (w0 + j) * g.dim3 + k;
                            *p = accumulate ? *p + acc[i][j] : acc[i][j];
                        } else if (e_kind[j] == 0) {
                            ep.final_out[z * ep.dout_final + e_dst[j]] = e_cst[j] * gate_act(e_act[j], acc[i][j]);
                        } else if (e_kind[j] == 2) {
                            ep.gates[z * ep.n_slots + e_slot[j]] = e_cst[j] * gate_act(e_act[j], acc[i][j]);
                        } else if (e_kind[j] == 1) {
                            ep.final_out[z * ep.dout_final + e_dst[j] + k] = acc[i][j] * __ldg(ep.gates + z * ep.n_slots + e_slot[j]);
                        }
                    }
                }
            }
        }
    }
}

// Gradient w.r.t. the shared weights of the same plan:
//
//     grad_W[wbase(K) + w * wstride] += sum_{z, k}  A[z, k, K] * grad_out[z, out_off + w * dim3 + k]
//
// i.e. per group the product A^T G whose summation index is (row, component).  A block owns a
// kBwKc x kBwWc block of (K, w), keeps its accumulators in registers over all the row tiles it
// visits (rounding: one partial sum per tile, added to the running sum) and adds them to the zeroed
// gradient with float atomics at the end.  Per tile it stages the A columns of its K block (same
// construction as phase 1 of the forward kernel) and the cotangent columns of its w block.
constexpr int kBwKc = 64;    // contraction entries per block
constexpr int kBwWc = 128;   // output channels per block
constexpr int kBwTK = 8;     // contraction entries per thread
constexpr int kBwTW = 4;     // output channels per thread

__global__ void __launch_bounds__(kDenseThreads) dense_bwd_w_kernel(const int32_t* __restrict__ plan,
        const float* __restrict__ x1, const float* __restrict__ x2, const float* __restrict__ gout,
        float* __restrict__ grad_w, int64_t Z, int group, int rows_z, int n_wc) {
    extern __shared__ __align__(16) float smem[];
    float* sA = smem;                                          // [r][kk]
    float* sG = smem + kRowsPerPass * kBwKc;                   // [r][w]
    int* sWb = reinterpret_cast<int*>(sG + kRowsPerPass * kBwWc);
    const int d1 = plan[1], d2 = plan[2], dout = plan[3];
    const int32_t* gp = plan + plan[7] + 6 * group;
    const DenseGroup g{gp[0], gp[1], gp[2], gp[3], gp[4], gp[5]};
    const int32_t* pathk_dir = plan + plan[9];
    const int32_t* cg = plan + plan[10];
    const int kc0 = (blockIdx.y / n_wc) * kBwKc, wc0 = (blockIdx.y % n_wc) * kBwWc;
    const int32_t* kent = plan + plan[8] + 4 * (g.kent_start + kc0);
    const int nk = min(kBwKc, g.K - kc0), nw = min(kBwWc, g.mul_out - wc0);
    const int RT = rows_z * g.dim3;
    const int tid = threadIdx.x, tx = tid & 31, ty = tid >> 5;
    if (tid < kBwKc) sWb[tid] = tid < nk ? kent[4 * tid + 3] : 0;

    float acc[kBwTK][kBwTW];
#pragma unroll
    for (int i = 0; i < kBwTK; ++i)
#pragma unroll
        for (int j = 0; j < kBwTW; ++j) acc[i][j] = 0.0f;

    const int64_t tiles = (Z + rows_z - 1) / rows_z;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t z0 = tile * rows_z;
        __syncthreads();
        for (int idx = tid; idx < RT * kBwKc; idx += kDenseThreads) {
            const int r = idx / kBwKc, kk = idx - r * kBwKc;
            const int zl = r / g.dim3, k = r - zl * g.dim3;
            const int64_t z = z0 + zl;
            float a = 0.0f;
            if (z < Z && kk < nk) {
                const int path = kent[4 * kk], x1off = kent[4 * kk + 1], x2off = kent[4 * kk + 2];
                const int32_t* pk = plan + pathk_dir[path] + 2 * k;
                const int cstart = pk[0], ccount = pk[1];
                const float* xr = x1 + z * d1 + x1off;
                const float* yr = x2off >= 0 ? x2 + z * d2 + x2off : nullptr;
                for (int c = 0; c < ccount; ++c) {
                    const int32_t* t = cg + 3 * (cstart + c);
                    a = fmaf(__int_as_float(t[2]) * xr[t[0]], yr ? yr[t[1]] : 1.0f, a);
                }
            }
            sA[idx] = a;
        }
        for (int idx = tid; idx < RT * kBwWc; idx += kDenseThreads) {
            const int r = idx / kBwWc, w = idx - r * kBwWc;
            const int zl = r / g.dim3, k = r - zl * g.dim3;
            const int64_t z = z0 + zl;
            sG[idx] = (z < Z && w < nw) ? gout[z * dout + g.out_off + (wc0 + w) * g.dim3 + k] : 0.0f;
        }
        __syncthreads();
        float part[kBwTK][kBwTW];
#pragma unroll
        for (int i = 0; i < kBwTK; ++i)
#pragma unroll
            for (int j = 0; j < kBwTW; ++j) part[i][j] = 0.0f;
#pragma unroll 4
        for (int r = 0; r < RT; ++r) {
            const float4 a0 = *reinterpret_cast<const float4*>(sA + r * kBwKc + ty * kBwTK);
            const float4 a1 = *reinterpret_cast<const float4*>(sA + r * kBwKc + ty * kBwTK + 4);
            const float4 gv = *reinterpret_cast<const float4*>(sG + r * kBwWc + tx * kBwTW);
            const float a[kBwTK] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[kBwTW] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
            for (int i = 0; i < kBwTK; ++i)
#pragma unroll
                for (int j = 0; j < kBwTW; ++j) part[i][j] = fmaf(a[i], b[j], part[i][j]);
        }
#pragma unroll
        for (int i = 0; i < kBwTK; ++i)
#pragma unroll
            for (int j = 0; j < kBwTW; ++j) acc[i][j] += part[i][j];
    }
    __syncthreads();   // sWb (written before the loop) is visible even when this block had no tile
#pragma unroll
    for (int i = 0; i < kBwTK; ++i) {
        const int kk = ty * kBwTK + i;
        if (kk >= nk) continue;
#pragma unroll
        for (int j = 0; j < kBwTW; ++j) {
            const int w = tx * kBwTW + j;
            if (w < nw) atomicAdd(grad_w + sWb[kk] + static_cast<int64_t>(wc0 + w) * g.w_stride, acc[i][j]);
        }
    }
}

// out[z, c] (+)= bias[c] over listed column ranges / zero fill of untouched columns.
__global__ void dense_fill_kernel(float* __restrict__ out, int64_t Z, int dout, int col0, int ncol,
                                  const float* __restrict__ bias /* may be null: zero fill */, int add) {
    const int64_t total = Z * ncol;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t z = i / ncol;
        const int c = static_cast<int>(i - z * ncol);
        float* p = out + z * dout + col0 + c;
        const float v = bias ? bias[c] : 0.0f;
        *p = add ? *p + v : v;
    }
}

}  // namespace e3b

namespace e3b {
namespace {

// Launches of the groups of a plan; pass 0 = every group, 1 = groups of scalars (2l+1 == 1), 2 = the others.
int launch_dense_groups(const int32_t* plan_host, const int32_t* plan_dev, const float* x1, const float* x2,
                        const float* weight, int64_t weight_row_stride, float* out, int64_t num_rows, int accumulate,
                        const DenseGateEpilogue& ep, int pass, cudaStream_t s) {
    const int n_groups = plan_host[4];
    const int32_t* groups = plan_host + plan_host[7];
    const int32_t* kent_all = plan_host + plan_host[8];
    for (int g = 0; g < n_groups; ++g) {
        const int mul_out = groups[6 * g + 1], dim3 = groups[6 * g + 2], K = groups[6 * g + 3];
        const int kent_start = groups[6 * g + 4], w_stride = groups[6 * g + 5];
        if (K == 0 || mul_out == 0) continue;
        if ((pass == 1 && dim3 != 1) || (pass == 2 && dim3 == 1)) continue;
        if (dim3 > kRowsPerPass) return fail(E3B_ERR_UNSUPPORTED, "dense_fwd: irrep dimension %d too large", dim3);
        const int rows_z = kRowsPerPass / dim3;
        // the A tile of the whole contraction when it fits (K <= 768), else chunks of 512 entries
        const int k_chunk = K <= 768 ? K : 512;
        const size_t smem = sizeof(float) * static_cast<size_t>(k_chunk) * kRowsPerPass + sizeof(int) * static_cast<size_t>(k_chunk);
        bool vec4 = (weight_row_stride == 0) && (w_stride == 1) && (mul_out % 4 == 0) && (reinterpret_cast<uintptr_t>(weight) % 16 == 0);
        if (vec4)
            for (int kk = 0; kk < K && vec4; ++kk) vec4 = (kent_all[4 * (kent_start + kk) + 3] % 4) == 0;
        const int64_t tiles = ceil_div(num_rows, rows_z);
        const unsigned grid = static_cast<unsigned>(std::min<int64_t>(tiles, kNumSMs * 4));
        if (vec4) {
            E3B_CUDA_TRY(cudaFuncSetAttribute(dense_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            dense_fwd_kernel<true><<<grid, kDenseThreads, smem, s>>>(plan_dev, x1, x2, weight, out, num_rows, g, rows_z, accumulate, weight_row_stride, k_chunk, ep);
        } else {
            E3B_CUDA_TRY(cudaFuncSetAttribute(dense_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            dense_fwd_kernel<false><<<grid, kDenseThreads, smem, s>>>(plan_dev, x1, x2, weight, out, num_rows, g, rows_z, accumulate, weight_row_stride, k_chunk, ep);
        }
        int rc = check_launch("e3b_dense_fwd");
        if (rc != E3B_OK) return rc;
    }
    return E3B_OK;
}

}  // namespace
}  // namespace e3b

extern "C" int e3b_dense_fwd(const int32_t* plan_host, const int32_t* plan_dev, const float* x1, const float* x2,
                             const float* weight, int64_t weight_row_stride, float* out, int64_t num_rows,
                             int accumulate, void* stream) {
    using namespace e3b;
    if (!plan_host || plan_host[0] != kDenseMagic) return fail(E3B_ERR_ARG, "dense_fwd: bad plan");
    if (num_rows < 0) return fail(E3B_ERR_ARG, "dense_fwd: negative row count");
    if (num_rows == 0) return E3B_OK;
    if (!plan_dev || !x1 || !out || !weight) return fail(E3B_ERR_ARG, "dense_fwd: null pointer");
    const DenseGateEpilogue none{nullptr, nullptr, nullptr, nullptr, 0, 0};
    return launch_dense_groups(plan_host, plan_dev, x1, x2, weight, weight_row_stride, out, num_rows, accumulate, none, 0,
                               static_cast<cudaStream_t>(stream));
}

extern "C" int e3b_dense_fwd_gate(const int32_t* plan_host, const int32_t* plan_dev, const float* x, const float* weight,
                                  const int32_t* gate_table, const float* gate_const, float* gates, int n_slots,
                                  float* out, int dout, int64_t num_rows, void* stream) {
    using namespace e3b;
    if (!plan_host || plan_host[0] != kDenseMagic) return fail(E3B_ERR_ARG, "dense_fwd_gate: bad plan");
    if (num_rows < 0 || n_slots < 0 || dout < 0) return fail(E3B_ERR_ARG, "dense_fwd_gate: negative size");
    if (num_rows == 0) return E3B_OK;
    if (!plan_dev || !x || !weight || !gate_table || !gate_const || !out || (n_slots > 0 && !gates))
        return fail(E3B_ERR_ARG, "dense_fwd_gate: null pointer");
    const DenseGateEpilogue ep{gate_table, gate_const, gates, out, n_slots, dout};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // scalars and gates first: the launches of the gated irreps read the activated gates of the same rows
    if (int rc = launch_dense_groups(plan_host, plan_dev, x, nullptr, weight, 0, out, num_rows, 0, ep, 1, s)) return rc;
    return launch_dense_groups(plan_host, plan_dev, x, nullptr, weight, 0, out, num_rows, 0, ep, 2, s);
}

extern "C" int e3b_dense_bwd_w(const int32_t* plan_host, const int32_t* plan_dev, const float* x1, const float* x2,
                               const float* grad_out, float* grad_weight, int64_t num_rows, void* stream) {
    using namespace e3b;
    if (!plan_host || plan_host[0] != kDenseMagic) return fail(E3B_ERR_ARG, "dense_bwd_w: bad plan");
    if (num_rows < 0) return fail(E3B_ERR_ARG, "dense_bwd_w: negative row count");
    if (num_rows == 0) return E3B_OK;
    if (!plan_dev || !x1 || !grad_out || !grad_weight) return fail(E3B_ERR_ARG, "dense_bwd_w: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int n_groups = plan_host[4];
    const int32_t* groups = plan_host + plan_host[7];
    for (int g = 0; g < n_groups; ++g) {
        const int mul_out = groups[6 * g + 1], dim_out = groups[6 * g + 2], K = groups[6 * g + 3];
        if (K == 0 || mul_out == 0) continue;
        if (dim_out > kRowsPerPass) return fail(E3B_ERR_UNSUPPORTED, "dense_bwd_w: irrep dimension %d too large", dim_out);
        const int rows_z = kRowsPerPass / dim_out;
        const int n_kc = (K + kBwKc - 1) / kBwKc, n_wc = (mul_out + kBwWc - 1) / kBwWc;
        const int64_t tiles = ceil_div(num_rows, rows_z);
        const int64_t want = std::max<int64_t>(1, (static_cast<int64_t>(kNumSMs) * 3 + n_kc * n_wc - 1) / (n_kc * n_wc));
        const dim3 grid(static_cast<unsigned>(std::min<int64_t>(tiles, want)), static_cast<unsigned>(n_kc * n_wc));
        constexpr int smem = static_cast<int>(sizeof(float)) * (kRowsPerPass * (kBwKc + kBwWc) + kBwKc);
        E3B_CUDA_TRY(cudaFuncSetAttribute(dense_bwd_w_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        dense_bwd_w_kernel<<<grid, kDenseThreads, smem, s>>>(plan_dev, x1, x2, grad_out, grad_weight, num_rows, g, rows_z, n_wc);
        int rc = check_launch("e3b_dense_bwd_w");
        if (rc != E3B_OK) return rc;
    }
    return E3B_OK;
}

extern "C" int e3b_fill_columns(float* out, int64_t num_rows, int row_stride, int col0, int ncol, const float* bias,
                                int add, void* stream) {
    using namespace e3b;
    if (num_rows < 0 || ncol < 0 || col0 < 0 || col0 + ncol > row_stride) return fail(E3B_ERR_ARG, "fill_columns: bad range");
    if (num_rows == 0 || ncol == 0) return E3B_OK;
    if (!out) return fail(E3B_ERR_ARG, "fill_columns: null pointer");
    const int64_t total = num_rows * ncol;
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(ceil_div(total, 256), kNumSMs * 16));
    dense_fill_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(out, num_rows, row_stride, col0, ncol, bias, add);
    return check_launch("e3b_fill_columns");
}
