/*
 * e3nn_b200 -- C ABI of a generated per-layout module.
 *
 * A layout module is a shared object generated (e3nn_b200/codegen/uvu.py) and compiled for ONE
 * irreps layout: irreps_in1 (x) irreps_in2 -> irreps_out with a fixed list of channel-wise
 * ('uvu') paths, whose Clebsch-Gordan coefficients and path normalisation are baked into the
 * code.  Every module exports exactly the entry points below; different layouts live in
 * different .so files (load them with RTLD_LOCAL).  Conventions are those of e3nn_b200.h:
 * device pointers, fp32 rows, int64 indices, status return (0 or negative), work enqueued on the
 * given stream, no allocation, no retained pointers.
 *
 * Row layouts: x1 [*, d1], x2 [*, d2], out [*, dout] laid out irrep after irrep, each irrep
 * block [mul, 2l+1] row-major (e3nn/o3/_tensor_product/_codegen.py:79-94); weights
 * [*, weight_numel] flat in instruction order, each path block [u, v] row-major (:123-128).
 */
#ifndef E3NN_B200_LAYOUT_H
#define E3NN_B200_LAYOUT_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dims[0..5] = d1, d2, dout, weight_numel, L (irreps_in2 == Y^0..Y^L, else -1), threads per row. */
int e3b_layout_info(int32_t* dims);

/* Hash of the layout this module was generated for (host string). */
const char* e3b_layout_key(void);

/* Message of the last failing call on the calling thread (host string). */
const char* e3b_layout_last_error(void);

/*
 * Channel-wise tensor product on Z rows: replaces the 'uvu' branch of the generated graph,
 * e3nn/o3/_tensor_product/_codegen.py:166-187, with the path weight (:312) and the per-output
 * sum and concatenation (:328-341) folded in.  Outputs no path writes are zero-filled.
 *   w: [weight_numel] if w_shared != 0, else [Z, weight_numel].
 */
int e3b_uvu_fwd(const float* x1, const float* x2, const float* w, float* out, int64_t Z, int w_shared, void* stream);

/*
 * Vector-Jacobian product of e3b_uvu_fwd (replaces autograd through the same graph):
 * grad_out [Z,dout] -> grad_x1 [Z,d1], grad_x2 [Z,d2], grad_w ([weight_numel] summed over rows if
 * w_shared != 0, else [Z, weight_numel]).
 */
int e3b_uvu_bwd(const float* x1, const float* x2, const float* w, const float* grad_out, float* grad_x1,
                float* grad_x2, float* grad_w, int64_t Z, int w_shared, void* stream);

/*
 * Fused message-passing step
 *     out[n] = scale * sum_{e : dst(e) = n} uvu(node_x[edge_src[e]], x2[e], w[e])
 * replacing gather + tp + scatter of e3nn/nn/models/v2106/points_convolution.py:105-106 (and
 * :13-17).  Destinations are given as a CSR over edge slots: slots rowptr[n]..rowptr[n+1]-1
 * belong to node n; slot ee refers to edge perm[ee] (perm == NULL: edge ee).
 *   in2_mode 0: x2 = rows [E, d2].
 *   in2_mode 1: x2 = edge vectors [E,3]; the spherical harmonics Y^0..Y^L of the normalised
 *               vector ('component' normalisation) are evaluated in the kernel
 *               (e3nn/o3/_spherical_harmonics.py:93-112).  Needs L >= 0 in e3b_layout_info.
 *   node_x [num_src, d1], w [E, weight_numel] (per-edge weights), out [num_nodes, dout].
 *   status: one int32 in device memory, zeroed by the caller; set to 2 if an edge_src value is
 *   outside [0, num_src) (that edge is skipped).
 */
int e3b_conv_fwd(const float* node_x, const float* x2, int in2_mode, const int64_t* edge_src, const int64_t* rowptr,
                 const int64_t* perm, const float* w, float* out, int64_t num_nodes, int64_t num_src,
                 int64_t num_edges, float scale, int32_t* status, void* stream);

/*
 * Kernel selection for e3b_conv_fwd (testing / profiling; no reference counterpart).  impl 0: the
 * bulk-copy pipelined kernel whenever the layout and the call are eligible (64-channel paths,
 * in2_mode 1, perm == NULL, 16-byte aligned rows), else the direct-load kernel; impl 1: always the
 * direct-load kernel.  Returns 1 if this module contains the pipelined kernel, else 0.
 */
int e3b_conv_select(int impl);

/*
 * Gradient of e3b_conv_fwd w.r.t. the per-edge weights and x2 (rows or edge vectors, as
 * in2_mode says) for a cotangent grad_out [num_nodes, dout]; replaces autograd through the same
 * three reference steps.  grad_w [E, weight_numel], grad_x2 [E, d2] or [E, 3].
 */
int e3b_conv_bwd(const float* node_x, const float* x2, int in2_mode, const int64_t* edge_src, const int64_t* rowptr,
                 const int64_t* perm, const float* w, const float* grad_out, float* grad_w, float* grad_x2,
                 int64_t num_nodes, int64_t num_src, int64_t num_edges, float scale, int32_t* status, void* stream);

/*
 * Gradient of e3b_conv_fwd w.r.t. the node features, the transpose of the gather
 * x[edge_src] (e3nn/nn/models/v2106/points_convolution.py:105) composed with the tensor product:
 *   grad_node_x[src[e], u, i] += sum_paths sum_k (sum_j C_ijk Y_e[j]) w[e, p, u] grad_out[dst(e), p, u, k].
 * grad_node_x [num_src, d1] is overwritten (zeroed, then accumulated with float atomics: edges are
 * sorted by destination, not by source).  The other arguments are those of e3b_conv_bwd.
 */
int e3b_conv_bwd_x(const float* x2, int in2_mode, const int64_t* edge_src, const int64_t* rowptr, const int64_t* perm,
                   const float* w, const float* grad_out, float* grad_node_x, int64_t num_nodes, int64_t num_src,
                   int64_t num_edges, float scale, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* E3NN_B200_LAYOUT_H */
