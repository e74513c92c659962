/*
 * e3nn_b200 -- C ABI of the B200 (sm_100a) kernels behind the e3nn message-passing hot path.
 *
 * Conventions (all entry points):
 *   - plain C linkage, plain pointers and sizes; every pointer is a DEVICE pointer unless a
 *     parameter is documented as host memory;
 *   - the return value is E3B_OK (0) or a negative E3B_ERR_* code; e3b_last_error() gives a
 *     per-thread message for the last failing call.  Nothing throws across the ABI;
 *   - work is enqueued on the CUDA stream passed in (a cudaStream_t cast to void*; NULL is
 *     the default stream) and the call returns without synchronising;
 *   - the library allocates no device memory and keeps no pointer after a call returns:
 *     outputs and scratch buffers belong to the caller;
 *   - tensors are dense, row-major, fp32 unless stated; indices are int64 unless stated.
 *
 * Each declaration cites the part of e3nn 0.6.0 whose arithmetic it replaces
 * (paths inside the e3nn repository).
 */
#ifndef E3NN_B200_H
#define E3NN_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define E3B_OK 0
#define E3B_ERR_ARG (-1)     /* bad argument (size, enum, null pointer, alignment)   */
#define E3B_ERR_CUDA (-2)    /* a CUDA runtime call or a launch failed               */
#define E3B_ERR_UNSUPPORTED (-3)
#define E3B_ERR_DEVICE (-4)  /* a kernel reported an error word (bad index, timeout) */

/* normalisation of spherical harmonics, e3nn/o3/_spherical_harmonics.py:103-110 */
#define E3B_SH_COMPONENT 0
#define E3B_SH_INTEGRAL 1
#define E3B_SH_NORM 2

#define E3B_SH_LMAX 12

/* ABI version of this header (bumped on any signature change). */
int e3b_abi_version(void);

/* Message of the last failing call on the calling thread ("" if none). Host string. */
const char* e3b_last_error(void);

/*
 * Real spherical harmonics Y^0..Y^lmax of n 3-vectors.
 * Replaces SphericalHarmonics.forward, e3nn/o3/_spherical_harmonics.py:93-112 with the
 * polynomials of :193-249 (and the generator's recurrence above l = 3).
 *   xyz [n,3] -> out [n,(lmax+1)^2], columns l-major then m.
 *   normalize != 0: the vector is divided by max(|v|, 1e-12) first (torch F.normalize).
 */
int e3b_sh_fwd(const float* xyz, float* out, int64_t n, int lmax, int normalize, int normalization,
               void* stream);

/*
 * Vector-Jacobian product of e3b_sh_fwd: grad_out [n,(lmax+1)^2] -> grad_xyz [n,3].
 * Replaces autograd through e3nn/o3/_spherical_harmonics.py:93-112.
 */
int e3b_sh_bwd(const float* xyz, const float* grad_out, float* grad_xyz, int64_t n, int lmax, int normalize,
               int normalization, void* stream);

/*
 * Destination-sorted CSR of an edge list: a stable counting sort of the edges by dst.
 * Replaces nothing in e3nn (its scatter is an unordered scatter_add_,
 * e3nn/nn/models/v2106/points_convolution.py:13-17); it is what lets the fused kernels sum
 * messages per destination row without atomics.  Bit-exact with
 *   perm = argsort(dst, stable=True); rowptr = [0, cumsum(bincount(dst, num_nodes))].
 *   dst [E] (values in [0,num_nodes)) -> perm [E], rowptr [num_nodes+1].
 *   scratch: e3b_csr_scratch_bytes(E, num_nodes) bytes of device memory, 256-byte aligned.
 *   status: one int32 in device memory, set non-zero if a dst value is out of range.
 */
int64_t e3b_csr_scratch_bytes(int64_t num_edges, int64_t num_nodes);
int e3b_csr_from_dst(const int64_t* dst, int64_t num_edges, int64_t num_nodes, int64_t* perm, int64_t* rowptr,
                     void* scratch, int64_t scratch_bytes, int32_t* status, void* stream);

/*
 * e3b_csr_from_dst without any caller-provided scratch.  (No counterpart in e3nn: this entry
 * point exists only for hosts that cannot allocate device memory.)
 *
 * Same result as e3b_csr_from_dst, bit for bit, but the work area is a fixed array inside this
 * library's device image, so the call (and the library) allocates nothing: no cudaMalloc, no
 * cudaFree, no allocating library routine.  It is meant for callers that only own the buffers
 * they were given -- a plug-in running inside somebody else's pre-sized memory arena, a
 * latency-critical loop that must not hit the device-wide synchronisation of an allocation, a
 * language binding without a device allocator.  Inputs and outputs are still the caller's.
 *
 * Limits and rules:
 *   - at most e3b_csr_static_max_edges() edges (262,144) and e3b_csr_static_max_nodes() nodes
 *     (65,536); larger problems are rejected with E3B_ERR_ARG and a message naming the limits;
 *   - every GPU that loads the library holds the work area (about 4.4 MiB) until the process exits;
 *   - the first call on each device looks up the work area's device address (with that device
 *     current); make that first call before starting any stream capture;
 *   - all calls on a device share the one work area: it keeps the previous call's contents, the
 *     parts that must start at zero are cleared on the caller's stream at the start of every
 *     call, and two calls whose GPU work overlaps (different streams, or different host threads
 *     without ordering between their streams) race on it -- serialise them.
 */
int64_t e3b_csr_static_max_edges(void);
int64_t e3b_csr_static_max_nodes(void);
int e3b_csr_from_dst_static(const int64_t* dst, int64_t num_edges, int64_t num_nodes, int64_t* perm, int64_t* rowptr,
                            int32_t* status, void* stream);

/*
 * Neighbour list of a periodic cubic box (cell list on the device), the graph construction every caller of
 * the path needs: e3nn ships only the O(N^2) radius_graph (e3nn/nn/models/gate_points_2101.py:27-32)
 * and fixes the convention edge_vec = pos[src] - pos[dst] + shift (gate_points_2101.py:328,
 * docs/guide/periodic_boundary_conditions.rst:134-136).  One edge per ordered pair src != dst whose
 * nearest-image distance is <= cutoff; edges sorted by destination, then by source; rowptr is their CSR.
 * Requires box >= 3 * cutoff (E3B_ERR_UNSUPPORTED otherwise).  Two calls, because the caller allocates:
 *   e3b_neighbor_count -> rowptr [num_atoms + 1] (rowptr[num_atoms] = number of edges, read it back),
 *   e3b_neighbor_fill  -> edge_src, edge_dst [E] int64 and shift [E,3] float.
 * scratch: e3b_neighbor_scratch_bytes(...) bytes of device memory, 256-byte aligned, the same buffer
 * (untouched in between) for both calls.  The result does not depend on scheduling (rows are sorted).
 */
int64_t e3b_neighbor_scratch_bytes(int64_t num_atoms, double box, double cutoff);
int e3b_neighbor_count(const float* pos, int64_t num_atoms, double box, double cutoff, void* scratch, int64_t scratch_bytes,
                       int64_t* rowptr, void* stream);
int e3b_neighbor_fill(const float* pos, int64_t num_atoms, double box, double cutoff, void* scratch, int64_t scratch_bytes,
                      const int64_t* rowptr, int64_t* edge_src, int64_t* edge_dst, float* shift, void* stream);
/*
 * The same list restricted to the destination rows [row0, row1) (a rank's shard of a graph partitioned by
 * destination ranges; the reference has no partitioned graphs): every atom is binned, only the rows of the range
 * are walked.  rowptr [row1 - row0 + 1] is the CSR of the range starting at 0, edge_dst holds GLOBAL atom numbers.
 * Concatenating the ranges of a partition gives exactly the edges of the full list, in the same order.
 */
int e3b_neighbor_count_rows(const float* pos, int64_t num_atoms, double box, double cutoff, void* scratch,
                            int64_t scratch_bytes, int64_t row0, int64_t row1, int64_t* rowptr, void* stream);
int e3b_neighbor_fill_rows(const float* pos, int64_t num_atoms, double box, double cutoff, void* scratch,
                           int64_t scratch_bytes, int64_t row0, int64_t row1, const int64_t* rowptr, int64_t* edge_src,
                           int64_t* edge_dst, float* shift, void* stream);

/*
 * Edge embedding of an interaction block, one kernel per direction:
 *   edge_vec[e] = pos[src[e]] - pos[dst[e]] + shift[e]        (e3nn/nn/models/gate_points_2101.py:328)
 *   B[e,k]      = basis_scale * basis_k(r), r = |edge_vec[e]|, k = 1..num_basis, with
 *                 basis 0: e3nn.math.bessel(r, num_basis, end)            (e3nn/math/_bessel.py:6-37; start = 0)
 *                 basis 1..5: soft_one_hot_linspace(r, start, end, num_basis, 'gaussian' | 'cosine' |
 *                             'smooth_finite' | 'fourier' | 'bessel', cutoff)
 *                                                             (e3nn/math/_soft_one_hot_linspace.py:100-140)
 *   h[e,:]      = env(r) * act_scale * act(w_scale * B[e,:] @ w0)   (first layer of FullyConnectedNet,
 *                 e3nn/nn/_fc.py:38-48 and :70-88); envelope 0: env = 1, envelope 1: env = smooth_cutoff(r / end)
 *                 (e3nn/nn/models/gate_points_2101.py:136-141; scaling h scales the network's linear output,
 *                 i.e. the per-edge weights, which is where those models apply it through the edge attributes)
 * pos [num_nodes,3]; edge_src, edge_dst [num_edges] int64; shift [num_edges,3] or NULL; w0 row-major
 * [num_basis, hidden]; num_basis <= 16; hidden in {32, 64, 96, 128}; act: 0 silu, 1 tanh, 2 relu, 3 identity.
 * Outputs edge_vec [num_edges,3] and h [num_edges,hidden].  An index outside [0, num_nodes) sets *status = 2
 * (device word, zeroed by the caller) and is clamped.
 *
 * e3b_radial_embed_bwd: cotangents grad_h [num_edges,hidden] and grad_edge_vec [num_edges,3] (or NULL) are
 * pulled back to the positions; the result is ADDED to grad_pos [num_nodes,3] (float atomics; the caller
 * zeroes it).  Replaces autograd through the same reference lines.
 */
int e3b_radial_embed_fwd(const float* pos, const int64_t* edge_src, const int64_t* edge_dst, const float* shift,
                         const float* w0, int64_t num_edges, int64_t num_nodes, int num_basis, int hidden, int basis,
                         int cutoff, int envelope, float start, float end, float basis_scale, float w_scale,
                         float act_scale, int act, float* edge_vec, float* h, int32_t* status, void* stream);
int e3b_radial_embed_bwd(const float* pos, const int64_t* edge_src, const int64_t* edge_dst, const float* shift,
                         const float* w0, const float* grad_h, const float* grad_edge_vec, int64_t num_edges,
                         int64_t num_nodes, int num_basis, int hidden, int basis, int cutoff, int envelope, float start,
                         float end, float basis_scale, float w_scale, float act_scale, int act, float* grad_pos,
                         int32_t* status, void* stream);

/*
 * Gate non-linearity on rows (e3nn/nn/_gate.py:127-144: Extract, two Activations of
 * e3nn/nn/_activation.py:80-98 and the scalar-gate ElementwiseTensorProduct, fused):
 *   out[z, j] = c_j * act_j(x[z, src_j])                      for scalar outputs,
 *   out[z, j] = x[z, src_j] * c_j * act_j(x[z, gate_j])       for gated components.
 * The irreps bookkeeping is done by the host and passed as device tables:
 *   out_table [dout,3] int32 = {src column, gate column or -1, activation}, out_const [dout] float;
 *   in_table  [din,5]  int32 = {kind, first output column, count, partner column, activation},
 *   in_const  [din] float; kind 0 scalar, 1 gated component (partner = its gate), 2 gate (count = 2l+1
 *   components starting at input column `partner` / output column `first`), 3 unused column.
 * activation: 0 silu, 1 tanh, 2 relu, 3 identity, 4 sigmoid, 5 abs.  x [rows,din], out [rows,dout];
 * e3b_gate_bwd writes grad_x [rows,din] for a cotangent grad_out [rows,dout] (replaces autograd).
 */
int e3b_gate_fwd(const float* x, const int32_t* out_table, const float* out_const, float* out, int64_t rows, int din,
                 int dout, void* stream);
/* The same forward map driven by a per-CHANNEL table (a scalar, or the 2l+1 components of one gated channel):
 * channel_table [num_channels,5] int32 = {first input column, count, gate column or -1, activation, first output
 * column}, channel_const [num_channels]; every output column must belong to exactly one channel.  The activation of
 * a gate is evaluated once per channel instead of once per gated component. */
int e3b_gate_fwd_channels(const float* x, const int32_t* channel_table, const float* channel_const, float* out,
                          int64_t rows, int din, int dout, int num_channels, void* stream);
int e3b_gate_bwd(const float* x, const float* grad_out, const int32_t* in_table, const float* in_const, float* grad_x,
                 int64_t rows, int din, int dout, void* stream);

/*
 * Weight-shared dense contractions in fp32 (CUDA cores): 'uvw' tensor-product paths
 *   out[z,w,k] = sum_paths pw sum_{u,v} W[u,v,w] sum_{ij} C_ijk x1[z,u,i] x2[z,v,j]
 * (e3nn/o3/_tensor_product/_codegen.py:148-165 with the accumulation of :312-343) and the
 * per-irrep Linear out[z,w,i] = pw sum_u W[u,w] x[z,u,i] (e3nn/o3/_linear.py:445-469).
 * The contraction is described by a "dense plan": int32 words built on the host
 * (layout documented in e3nn_b200/csrc/dense.cu); plan_host is that array in HOST memory,
 * plan_dev a copy in device memory.  x2 may be NULL for plans that never read it (Linear).
 * weight_row_stride: 0 for shared weights [weight_numel]; otherwise row z reads its own weights at
 * weight + z * weight_row_stride (e3nn's shared_weights=False).
 * accumulate != 0 adds to out instead of overwriting the columns the plan writes; columns no
 * path writes are left untouched (zero them with e3b_fill_columns).
 */
int e3b_dense_fwd(const int32_t* plan_host, const int32_t* plan_dev, const float* x1, const float* x2,
                  const float* weight, int64_t weight_row_stride, float* out, int64_t num_rows, int accumulate,
                  void* stream);

/*
 * A per-irrep Linear (e3nn/o3/_linear.py:445-469) followed by Gate (e3nn/nn/_gate.py:127-144) without the
 * intermediate row: the plan is the Linear's, whose output row would be the Gate's input row; the gate is applied
 * where the Linear's result is still in registers.  gate_table [din_gate, 4] int32 = {kind, destination column,
 * activation, gate slot} and gate_const [din_gate] float per column of that (never materialised) row:
 *   kind 0 scalar:  out[z, dst]    = const * act(y)        kind 2 gate: gates[z, slot] = const * act(y)
 *   kind 1 gated:   out[z, dst]    = y * gates[z, slot]    kind 3: no output depends on the column.
 * gates [rows, n_slots] is written and read by this call (the only extra traffic: the gate scalars, once each way);
 * out [rows, dout] is the Gate's output row.  Scalar irreps are launched before the gated ones on `stream`.
 * Activation codes as in e3b_gate_fwd.
 */
int e3b_dense_fwd_gate(const int32_t* plan_host, const int32_t* plan_dev, const float* x, const float* weight,
                       const int32_t* gate_table, const float* gate_const, float* gates, int n_slots, float* out,
                       int dout, int64_t num_rows, void* stream);

/*
 * Gradient of e3b_dense_fwd w.r.t. its SHARED weights (what autograd derives from the einsums of
 * e3nn/o3/_tensor_product/_codegen.py:148-165 and e3nn/o3/_linear.py:420-469 for `weight`):
 *   grad_weight[wbase(K) + w * wstride] += sum_{z,k} A[z,k,K] * grad_out[z, out_off + w * dim3 + k]
 * with the same plan as the forward call.  grad_weight [weight_numel] must be zeroed by the caller
 * (the kernel adds with float atomics; summation order is not fixed).  x2 may be NULL for Linear plans.
 */
int e3b_dense_bwd_w(const int32_t* plan_host, const int32_t* plan_dev, const float* x1, const float* x2,
                    const float* grad_out, float* grad_weight, int64_t num_rows, void* stream);

/*
 * out[z, col0 + c] = (add ? out[z, col0 + c] : 0) + (bias ? bias[c] : 0) for c < ncol: zero fill of
 * outputs no path writes (e3nn/o3/_tensor_product/_codegen.py:15-21) and the scalar biases of
 * Linear (e3nn/o3/_linear.py:423-427).
 */
int e3b_fill_columns(float* out, int64_t num_rows, int row_stride, int col0, int ncol, const float* bias, int add,
                     void* stream);

/*
 * Self-test of the bounded-wait convention of the pipelined kernels (no counterpart in the reference, which has
 * no device code): one small block waits on an mbarrier that nothing arrives at, gives up after `limit` polls
 * (1 .. 100000, each a try_wait with a short back-off), stores 3 in *status and returns.  The host reads the
 * word like that of any other kernel; the device context stays usable.
 */
int e3b_selftest_bounded_wait(int32_t* status, unsigned limit, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* E3NN_B200_H */
