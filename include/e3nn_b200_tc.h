/*
 * e3nn_b200 -- C ABI of the generated tensor-core modules (tcgen05 / tensor memory, sm_100a).
 *
 * Two kinds of generated modules hold the weight-shared dense contractions of the path, each compiled
 * for ONE layout (RTLD_LOCAL, like the 'uvu' layout modules; conventions of e3nn_b200.h: device
 * pointers, fp32 rows, status return 0 or negative, work enqueued on the given stream, no allocation,
 * no retained pointers).  Both also export e3b_layout_info / e3b_layout_key / e3b_layout_last_error
 * with the meaning given in e3nn_b200_layout.h (dims[3] and dims[4] unused by the tc_gemm modules).
 *
 * "tcg" modules (e3nn_b200/codegen/tc_gemm.py): out[z, :] = contraction(x1[z, :], x2[z, :]) @ W with
 *   - the fully-connected 'uvw' tensor product, e3nn/o3/_tensor_product/_codegen.py:148-165 (+ :312-343),
 *   - the per-irrep Linear and its transpose, e3nn/o3/_linear.py:445-469,
 *   - a dense layer x @ W * scale and its transpose, e3nn/nn/_fc.py:38-48
 *   as the layout it was generated for.  Operands are split into tf32 pieces in the kernel.
 * "uvwpost" / "uvwtc" modules (e3nn_b200/codegen/uvw_post.py, uvw_tc.py): the 'uvw' tensor product with plain tf32
 *   operands; the first applies the Clebsch-Gordan coupling after the matrix product (raw input rows as the left
 *   operand), the second before it, for layouts the first does not take.  Same entry point.
 */
#ifndef E3NN_B200_TC_H
#define E3NN_B200_TC_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Bytes of device scratch e3b_tc_gemm_fwd needs for the prepared (scaled, split, swizzled) weights. */
long long e3b_tc_gemm_scratch_bytes(void);

/*
 * x1 [Z, d1], x2 [Z, d2] or NULL when the layout has no second operand, weight: the flat weight vector
 * of the reference module (instruction order, each path [u, w] row-major), out [Z, dout] (16-byte
 * aligned).  precision: 1 = plain tf32 operands (one MMA per k-step, ~1e-3 relative), 2 = hi/lo-split
 * operands (three MMAs, ~2e-5 x RMS).  scratch: e3b_tc_gemm_scratch_bytes() bytes, 16-byte aligned.
 * cta_split: NULL, or a host array with the number of CTAs per output group (a caller that overlaps the launch with
 * a collective passes fewer than one CTA per SM in total, see e3nn_b200/_lib.py: tc_gemm_cta_limit).  status: one device int32
 * zeroed by the caller; 3 = a bounded wait inside the kernel gave up (results invalid).
 */
int e3b_tc_gemm_fwd(const float* x1, const float* x2, const float* weight, float* out, int64_t Z, int precision,
                    void* scratch, const int* cta_split, int32_t* status, void* stream);

/*
 * The contraction of a "tcg" Linear module with Gate (e3nn/nn/_gate.py:127-144) as its epilogue; the Linear's output
 * row (the Gate's input row, `dout` columns) is never written.  gate_table [dout,4] int32 (16-byte aligned) =
 * {kind, destination column, activation, gate slot} and gate_const [dout] per column of that row: kind 0 scalar:
 * out[z, dst] = const * act(y); kind 2 gate: gates[z, slot] = const * act(y); kind 1 component k of a gated channel
 * (entry of its component 0): out[z, dst + k] = y * gates[z, slot]; kind 3 unused.  gates [Z, n_slots], out
 * [Z, dout_final] (the Gate's output row).  Activation codes of e3b_gate_fwd.  Two launches on `stream`.
 */
int e3b_tc_gemm_fwd_gate(const float* x1, const float* weight, const int32_t* gate_table, const float* gate_const,
                         float* gates, int n_slots, float* out, int dout_final, int64_t Z, int precision, void* scratch,
                         int32_t* status, void* stream);

/*
 * 'uvw' tensor product with plain tf32 operands: x1 [Z, d1], x2 [Z, d2], weight [weight_numel] shared,
 * out [Z, dout].  num_ctas: 0 = one per SM.  status as above.  x1 and out 16-byte aligned (row lengths of
 * "uvwpost" modules are multiples of four floats), Z < 2^31: blocks of scalars of x1 are fetched through a tensor
 * map that the call encodes on the host (cuTensorMapEncodeTiled, reached through the runtime's entry-point query).
 * Returns -2 when the driver does not provide that entry point.
 */
int e3b_uvw_tc_fwd(const float* x1, const float* x2, const float* weight, float* out, int64_t Z, int num_ctas,
                   int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* E3NN_B200_TC_H */
