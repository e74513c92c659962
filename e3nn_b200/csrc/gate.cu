// Gate non-linearity on rows of irreps features: the step after the Linear in every model
// (e3nn/nn/_gate.py:35-144 with e3nn/nn/_activation.py:9-111 and the 'uuu' product of
// e3nn/o3/_tensor_product/_sub.py ElementwiseTensorProduct, which for a scalar second operand is a plain
// per-channel multiplication):
//
//   out = [ c_i * phi_i(scalars_i) ]  (+)  [ gated_j * c_j * phi_j(gates_j) ]
//
// The reference runs an Extract (three narrow + cat), two Activations (narrow + cat per block) and a
// generated tensor product; here one elementwise kernel per direction reads a row once and writes it once.
// The irreps bookkeeping lives on the host: per OUTPUT column {input column, gate column or -1,
// activation code, constant}, per INPUT column {kind, first output column, count, partner column}.
#include "common.cuh"
#include "gate_act.cuh"

namespace e3b {
namespace {

// A thread owns one column (its table entry stays in registers) and walks the rows: consecutive threads touch
// consecutive addresses, no per-element index arithmetic beyond one multiply-add per row.
// out_tbl[j] = {input column, gate column or -1, activation code}, out_cst[j] = constant
__global__ void __launch_bounds__(256) gate_fwd_kernel(const float* __restrict__ x, const int32_t* __restrict__ out_tbl,
                                                       const float* __restrict__ out_cst, float* __restrict__ out, int64_t rows,
                                                       int din, int dout) {
    const int j = blockIdx.y * blockDim.x + threadIdx.x;
    if (j >= dout) return;
    const int src = out_tbl[3 * j], gate = out_tbl[3 * j + 1], act = out_tbl[3 * j + 2];
    const float cst = out_cst[j];
    // four rows per trip: their loads are independent and in flight together
    for (int64_t z0 = static_cast<int64_t>(blockIdx.x) * 4; z0 < rows; z0 += static_cast<int64_t>(gridDim.x) * 4) {
        float v[4], gv[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int64_t z = z0 + r < rows ? z0 + r : rows - 1;
            v[r] = x[z * din + src];
            gv[r] = gate < 0 ? 0.0f : x[z * din + gate];
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (z0 + r < rows) out[(z0 + r) * dout + j] = gate < 0 ? cst * gate_act(act, v[r]) : v[r] * (cst * gate_act(act, gv[r]));
    }
}

// One thread per CHANNEL (a scalar, or the 2l+1 components of a gated channel): the gate's activation, the only
// transcendental work of the row, is evaluated once per channel instead of once per output column.
// ch_tbl[q] = {first input column, count (1 or 2l+1), gate column or -1, activation code, first output column},
// ch_cst[q] = constant.  Lanes are consecutive channels, i.e. adjacent runs of 2l+1 floats: full lines are used.
__global__ void __launch_bounds__(256) gate_fwd_channel_kernel(const float* __restrict__ x, const int32_t* __restrict__ ch_tbl,
                                                               const float* __restrict__ ch_cst, float* __restrict__ out,
                                                               int64_t rows, int din, int dout, int nch) {
    const int q = blockIdx.y * blockDim.x + threadIdx.x;
    if (q >= nch) return;
    const int src = ch_tbl[5 * q], cnt = ch_tbl[5 * q + 1], gate = ch_tbl[5 * q + 2], act = ch_tbl[5 * q + 3], dst = ch_tbl[5 * q + 4];
    const float cst = ch_cst[q];
    for (int64_t z0 = static_cast<int64_t>(blockIdx.x) * 2; z0 < rows; z0 += static_cast<int64_t>(gridDim.x) * 2) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int64_t z = z0 + r;
            if (z >= rows) break;
            const float* xr = x + z * din;
            float* orow = out + z * dout + dst;
            if (gate < 0) {
                orow[0] = cst * gate_act(act, xr[src]);
            } else {
                const float gv = cst * gate_act(act, xr[gate]);
                for (int m = 0; m < cnt; ++m) orow[m] = xr[src + m] * gv;
            }
        }
    }
}

// in_tbl[c] = {kind, first output column, count, partner, activation code}, in_cst[c] = constant:
// kind 0 = scalar, 1 = gated component (partner = its gate's input column, activation of that gate),
// 2 = gate (count = 2l+1 components of its channel, partner = input column of the first component),
// 3 = column no output depends on
__global__ void __launch_bounds__(256) gate_bwd_kernel(const float* __restrict__ x, const float* __restrict__ gout,
                                                       const int32_t* __restrict__ in_tbl, const float* __restrict__ in_cst,
                                                       float* __restrict__ gin, int64_t rows, int din, int dout) {
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= din) return;
    const int kind = in_tbl[5 * c], o0 = in_tbl[5 * c + 1], cnt = in_tbl[5 * c + 2], partner = in_tbl[5 * c + 3],
              act = in_tbl[5 * c + 4];
    const float cst = in_cst[c];
    for (int64_t z = blockIdx.x; z < rows; z += gridDim.x) {
        const float* xr = x + z * din;
        const float* gr = gout + z * dout;
        float g = 0.0f;
        if (kind == 0) {
            g = gr[o0] * cst * gate_act_grad(act, xr[c]);
        } else if (kind == 1) {
            g = gr[o0] * (cst * gate_act(act, xr[partner]));
        } else if (kind == 2) {
            float acc = 0.0f;
            for (int m = 0; m < cnt; ++m) acc = fmaf(gr[o0 + m], xr[partner + m], acc);
            g = acc * cst * gate_act_grad(act, xr[c]);
        }
        gin[z * din + c] = g;
    }
}

// grid: y covers the columns in blocks of 256, x walks the rows with enough blocks to fill the machine
dim3 gate_grid(int64_t rows, int cols) {
    const int ny = (cols + 255) / 256;
    int64_t nx = (static_cast<int64_t>(kNumSMs) * 16 + ny - 1) / ny;
    if (nx > rows) nx = rows;
    if (nx < 1) nx = 1;
    return dim3(static_cast<unsigned>(nx), static_cast<unsigned>(ny));
}

}  // namespace
}  // namespace e3b

extern "C" int e3b_gate_fwd(const float* x, const int32_t* out_table, const float* out_const, float* out, int64_t rows,
                            int din, int dout, void* stream) {
    using namespace e3b;
    if (rows < 0 || din < 0 || dout < 0) return fail(E3B_ERR_ARG, "gate_fwd: negative size");
    if (rows == 0 || dout == 0) return E3B_OK;
    if (!x || !out_table || !out_const || !out) return fail(E3B_ERR_ARG, "gate_fwd: null pointer");
    gate_fwd_kernel<<<gate_grid(rows, dout), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, out_table, out_const, out, rows, din, dout);
    return check_launch("gate_fwd");
}

extern "C" int e3b_gate_fwd_channels(const float* x, const int32_t* channel_table, const float* channel_const, float* out,
                                     int64_t rows, int din, int dout, int num_channels, void* stream) {
    using namespace e3b;
    if (rows < 0 || din < 0 || dout < 0 || num_channels < 0) return fail(E3B_ERR_ARG, "gate_fwd_channels: negative size");
    if (rows == 0 || num_channels == 0) return E3B_OK;
    if (!x || !channel_table || !channel_const || !out) return fail(E3B_ERR_ARG, "gate_fwd_channels: null pointer");
    gate_fwd_channel_kernel<<<gate_grid(rows, num_channels), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, channel_table, channel_const, out, rows, din, dout, num_channels);
    return check_launch("gate_fwd_channels");
}

extern "C" int e3b_gate_bwd(const float* x, const float* grad_out, const int32_t* in_table, const float* in_const,
                            float* grad_x, int64_t rows, int din, int dout, void* stream) {
    using namespace e3b;
    if (rows < 0 || din < 0 || dout < 0) return fail(E3B_ERR_ARG, "gate_bwd: negative size");
    if (rows == 0 || din == 0) return E3B_OK;
    if (!x || !grad_out || !in_table || !in_const || !grad_x) return fail(E3B_ERR_ARG, "gate_bwd: null pointer");
    gate_bwd_kernel<<<gate_grid(rows, din), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, grad_out, in_table, in_const, grad_x, rows, din, dout);
    return check_launch("gate_bwd");
}
