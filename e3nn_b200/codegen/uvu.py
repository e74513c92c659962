"""CUDA source generator for channel-wise ('uvu') tensor products.

A 'uvu' path computes, per row z and channel u (``e3nn/o3/_tensor_product/_codegen.py:166-187``),

    out[z, u, k] += pw * sum_v w[z, u, v] * sum_{i,j} C_{ijk} x1[z, u, i] x2[z, v, j] .

The generated code keeps one channel u per thread and evaluates, for every path and v,

    t[i][k] = pw * sum_j C_{ijk} x2[v][j]          (depends on the row only)
    s[k]    = sum_i t[i][k] * x1[u][i]
    acc[k] += w[u][v] * s[k]

with the Clebsch-Gordan non-zeros as immediates and every loop unrolled, so x1, x2, t and
the accumulators live in registers.  Only non-zero (i,k) pairs of t are emitted.

The same per-row body is instantiated in four kernels of a layout module:

  * ``uvu_fwd``   rows in, rows out (drop-in for ``TensorProduct.forward``);
  * ``uvu_bwd``   its vector-Jacobian product (grad x1, grad x2, grad w);
  * ``conv_fwd``  gather x1 = node_x[src] -> optional in-kernel spherical harmonics of the
                  edge vector -> 'uvu' -> per-destination sum over a destination-sorted CSR
                  (``e3nn/nn/models/v2106/points_convolution.py:105-106``); messages never
                  reach HBM and rows are summed in a fixed order (no float atomics);
  * ``conv_bwd``  gradient of ``conv_fwd`` w.r.t. the per-edge weights and the edge vectors
                  (or x2), for a cotangent given per destination row.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

from ..o3._spec import TPSpec
from ..o3._wigner import wigner_3j_numpy
from . import uvu_tma, uvu_tma_bwd, uvu_tma_bwdx


def _f(v: float) -> str:
    return f"{np.float32(v):.9e}f"


@dataclass
class Path:
    index: int          # instruction index in the spec
    i1: int
    i2: int
    io: int
    l1: int
    l2: int
    l3: int
    mul1: int
    mul2: int
    off1: int
    off2: int
    offo: int
    woff: int           # offset in the flat weight vector, -1 when unweighted
    pw: float


class UvuLayout:
    """Everything the generator needs, extracted from a `TPSpec` whose paths are all 'uvu'."""

    def __init__(self, spec: TPSpec):
        assert all(i.connection_mode == "uvu" for _, i in spec.live_instructions()), "uvu generator got a non-uvu path"
        self.spec = spec
        self.d1, self.d2, self.dout = spec.irreps_in1.dim, spec.irreps_in2.dim, spec.irreps_out.dim
        self.wn = spec.weight_numel
        o1, o2, oo = spec.irreps_in1.offsets(), spec.irreps_in2.offsets(), spec.irreps_out.offsets()
        woffs = spec.weight_offsets()
        live = dict(spec.live_instructions())
        self.paths: List[Path] = []
        for n, ins in enumerate(spec.instructions):
            if n not in live:
                continue
            a, b, c = spec.irreps_in1[ins.i_in1], spec.irreps_in2[ins.i_in2], spec.irreps_out[ins.i_out]
            assert a.mul == c.mul
            self.paths.append(
                Path(n, ins.i_in1, ins.i_in2, ins.i_out, a.ir.l, b.ir.l, c.ir.l, a.mul, b.mul,
                     o1[ins.i_in1], o2[ins.i_in2], oo[ins.i_out], woffs[n], float(ins.path_weight))
            )
        self.U = max([p.mul1 for p in self.paths], default=1)
        # threads per row: a power of two up to 32, else a multiple of 32
        if self.U <= 32:
            g = 1
            while g < self.U:
                g *= 2
            self.G = g
        else:
            self.G = (self.U + 31) // 32 * 32
        self.in1_used = sorted({p.i1 for p in self.paths})
        self.out_used = sorted({p.io for p in self.paths})
        self.x2_in_registers = self.d2 <= 64

    # SH fusion is possible when in2 is exactly Y^0..Y^L with multiplicity one each
    def sh_lmax(self) -> Optional[int]:
        irreps = self.spec.irreps_in2
        for n, (mul, ir) in enumerate(irreps):
            if mul != 1 or ir.l != n or ir.p != (-1) ** n:
                return None
        return len(irreps) - 1 if len(irreps) > 0 else None


def _t_pairs(p: Path, v: int, layout: UvuLayout) -> Tuple[List[str], Dict[Tuple[int, int], str]]:
    """Code computing the non-zero t[i][k] of a path for a given v, and their variable names."""
    c = wigner_3j_numpy(p.l1, p.l2, p.l3) * p.pw
    lines, names = [], {}
    for i in range(2 * p.l1 + 1):
        for k in range(2 * p.l3 + 1):
            terms = [(j, c[i, j, k]) for j in range(2 * p.l2 + 1) if c[i, j, k] != 0.0]
            if not terms:
                continue
            name = f"t{p.index}_{v}_{i}_{k}"
            expr = " + ".join(f"{_f(coef)} * {_y(p, v, j, layout)}" for j, coef in terms)
            lines.append(f"const float {name} = {expr};")
            names[(i, k)] = name
    return lines, names


def _y(p: Path, v: int, j: int, layout: UvuLayout) -> str:
    idx = p.off2 + v * (2 * p.l2 + 1) + j
    return f"Y[{idx}]" if layout.x2_in_registers else f"yrow[{idx}]"


def emit_forward_body(layout: UvuLayout) -> str:
    """Per-(row, u) forward body.

    Expects in scope: ``u`` (channel), ``xrow`` (const float* to the in1 row), ``Y`` (register
    array with the in2 row) or ``yrow``, ``wrow`` (const float* to the row's or the shared
    weights).  Accumulates into ``acc<io>[k]`` which the caller declares and zeroes.
    """
    spec = layout.spec
    out: List[str] = []
    for i1 in layout.in1_used:
        mul, ir = spec.irreps_in1[i1]
        off = spec.irreps_in1.offsets()[i1]
        dim = ir.dim
        out.append(f"float x{i1}[{dim}];")
        out.append(f"if (u < {mul}) {{")
        for i in range(dim):
            out.append(f"  x{i1}[{i}] = xrow[{off} + u * {dim} + {i}];")
        out.append("} else {")
        for i in range(dim):
            out.append(f"  x{i1}[{i}] = 0.0f;")
        out.append("}")
    for p in layout.paths:
        out.append(f"// path {p.index}: {p.mul1}x l={p.l1} (x) {p.mul2}x l={p.l2} -> l={p.l3}")
        out.append(f"if (u < {p.mul1}) {{")
        for v in range(p.mul2):
            out.append("  {")
            t_lines, t = _t_pairs(p, v, layout)
            out += ["    " + s for s in t_lines]
            if p.woff >= 0:
                out.append(f"    const float w = wrow[{p.woff} + u * {p.mul2} + {v}];")
            for k in range(2 * p.l3 + 1):
                terms = [f"{t[(i, k)]} * x{p.i1}[{i}]" for i in range(2 * p.l1 + 1) if (i, k) in t]
                if not terms:
                    continue
                s = " + ".join(terms)
                if p.woff >= 0:
                    out.append(f"    acc{p.io}[{k}] = fmaf(w, {s}, acc{p.io}[{k}]);")
                else:
                    out.append(f"    acc{p.io}[{k}] += {s};")
            out.append("  }")
        out.append("}")
    return "\n".join(out)


def emit_backward_body(layout: UvuLayout, want_dx: bool = True) -> str:
    """Per-(row, u) backward body.

    In scope: ``u``, ``xrow``, ``Y``/``yrow``, ``wrow``, ``g<io>[k]`` (cotangent of this channel's
    outputs, already scaled).  Produces ``dxi<i1>[i]`` (when ``want_dx``), ``dY[d2]`` (this thread's partial
    sum over its channel; the caller reduces over u) and stores dw through the macro
    ``E3B_STORE_DW(index, value)``.
    """
    spec = layout.spec
    out: List[str] = []
    for i1 in layout.in1_used:
        mul, ir = spec.irreps_in1[i1]
        off = spec.irreps_in1.offsets()[i1]
        dim = ir.dim
        out.append(f"float x{i1}[{dim}];")
        if want_dx:
            out.append(f"float dxi{i1}[{dim}];")
        out.append(f"#pragma unroll\nfor (int i = 0; i < {dim}; ++i) {{ x{i1}[i] = (u < {mul}) ? xrow[{off} + u * {dim} + i] : 0.0f;"
                   + (f" dxi{i1}[i] = 0.0f;" if want_dx else "") + " }")
    for p in layout.paths:
        c = wigner_3j_numpy(p.l1, p.l2, p.l3) * p.pw
        out.append(f"// path {p.index}: l={p.l1} (x) l={p.l2} -> l={p.l3}")
        out.append(f"if (u < {p.mul1}) {{")
        for v in range(p.mul2):
            out.append("  {")
            t_lines, t = _t_pairs(p, v, layout)
            out += ["    " + s for s in t_lines]
            if p.woff >= 0:
                out.append(f"    const float w = wrow[{p.woff} + u * {p.mul2} + {v}];")
                # dw = sum_k g_k s_k
                parts = []
                for k in range(2 * p.l3 + 1):
                    terms = [f"{t[(i, k)]} * x{p.i1}[{i}]" for i in range(2 * p.l1 + 1) if (i, k) in t]
                    if terms:
                        parts.append(f"g{p.io}[{k}] * ({' + '.join(terms)})")
                out.append(f"    E3B_STORE_DW({p.woff} + u * {p.mul2} + {v}, {' + '.join(parts) if parts else '0.0f'});")
                wname = "w"
            else:
                wname = "1.0f"
            # wg_k = w * g_k
            for k in range(2 * p.l3 + 1):
                out.append(f"    const float wg{k} = {wname} * g{p.io}[{k}];")
            if want_dx:
                for i in range(2 * p.l1 + 1):
                    terms = [f"{t[(i, k)]} * wg{k}" for k in range(2 * p.l3 + 1) if (i, k) in t]
                    if terms:
                        out.append(f"    dxi{p.i1}[{i}] += {' + '.join(terms)};")
            # dY_j += sum_{ik} C_ijk x_i wg_k
            for j in range(2 * p.l2 + 1):
                terms = []
                for i in range(2 * p.l1 + 1):
                    for k in range(2 * p.l3 + 1):
                        if c[i, j, k] != 0.0:
                            terms.append(f"{_f(c[i, j, k])} * x{p.i1}[{i}] * wg{k}")
                if terms:
                    idx = p.off2 + v * (2 * p.l2 + 1) + j
                    out.append(f"    dY[{idx}] += {' + '.join(terms)};")
            out.append("  }")
        out.append("}")
    return "\n".join(out)


def emit_dx_body(layout: UvuLayout) -> str:
    """Per-(edge, u) cotangent of the first operand only: ``dxi<i1>[i] = sum_paths sum_k t_ik w g_k``.

    In scope: ``u``, ``Y``/``yrow``, ``wrow``, ``g<io>[k]``.  Does not read the first operand at all."""
    spec = layout.spec
    out: List[str] = []
    for i1 in layout.in1_used:
        dim = spec.irreps_in1[i1].ir.dim
        out.append(f"float dxi{i1}[{dim}];")
        out.append(f"#pragma unroll\nfor (int i = 0; i < {dim}; ++i) dxi{i1}[i] = 0.0f;")
    for p in layout.paths:
        out.append(f"// path {p.index}: l={p.l1} (x) l={p.l2} -> l={p.l3}")
        out.append(f"if (u < {p.mul1}) {{")
        for v in range(p.mul2):
            out.append("  {")
            t_lines, t = _t_pairs(p, v, layout)
            out += ["    " + line for line in t_lines]
            wname = f"wrow[{p.woff} + u * {p.mul2} + {v}]" if p.woff >= 0 else "1.0f"
            for k in range(2 * p.l3 + 1):
                out.append(f"    const float wg{k} = {wname} * g{p.io}[{k}];")
            for i in range(2 * p.l1 + 1):
                terms = [f"{t[(i, k)]} * wg{k}" for k in range(2 * p.l3 + 1) if (i, k) in t]
                if terms:
                    out.append(f"    dxi{p.i1}[{i}] += {' + '.join(terms)};")
            out.append("  }")
        out.append("}")
    return "\n".join(out)


def _indent(text: str, n: int) -> str:
    pad = " " * n
    return "\n".join(pad + line if line else line for line in text.split("\n"))


def emit_module(spec: TPSpec) -> str:
    """Complete .cu translation unit for one 'uvu' layout."""
    L = UvuLayout(spec)
    sh_l = L.sh_lmax()
    G = L.G
    threads = max(128, G) if G <= 128 else G  # block size: whole groups
    if threads % G != 0:
        threads = G
    rows_per_block = threads // G
    if not L.x2_in_registers:
        raise NotImplementedError("uvu layouts with irreps_in2.dim > 64 are not generated yet")

    acc_decl = []
    acc_store_rows = []
    acc_store_conv = []
    g_load_rows = []
    g_load_conv = []
    for io in L.out_used:
        mul, ir = spec.irreps_out[io]
        off = spec.irreps_out.offsets()[io]
        dim = ir.dim
        acc_decl.append(f"float acc{io}[{dim}];\n#pragma unroll\nfor (int k = 0; k < {dim}; ++k) acc{io}[k] = 0.0f;")
        acc_store_rows.append(
            f"if (u < {mul}) {{\n#pragma unroll\n  for (int k = 0; k < {dim}; ++k) orow[{off} + u * {dim} + k] = acc{io}[k];\n}}"
        )
        acc_store_conv.append(
            f"if (u < {mul}) {{\n#pragma unroll\n  for (int k = 0; k < {dim}; ++k) orow[{off} + u * {dim} + k] = acc{io}[k] * scale;\n}}"
        )
        g_load_rows.append(
            f"float g{io}[{dim}];\n#pragma unroll\nfor (int k = 0; k < {dim}; ++k) g{io}[k] = (u < {mul}) ? grow[{off} + u * {dim} + k] : 0.0f;"
        )
        g_load_conv.append(
            f"float g{io}[{dim}];\n#pragma unroll\nfor (int k = 0; k < {dim}; ++k) g{io}[k] = (u < {mul}) ? grow[{off} + u * {dim} + k] * scale : 0.0f;"
        )
    # outputs nobody writes: zero-filled by a generic loop over the gaps
    zero_ranges = []
    for io, (mul, ir) in enumerate(spec.irreps_out):
        if io not in L.out_used and mul * ir.dim > 0:
            zero_ranges.append((spec.irreps_out.offsets()[io], mul * ir.dim))
    zero_code = "\n".join(
        f"for (int c = u; c < {n}; c += {G}) orow[{off} + c] = 0.0f;" for off, n in zero_ranges
    )

    dx_store = []
    for i1 in L.in1_used:
        mul, ir = spec.irreps_in1[i1]
        off = spec.irreps_in1.offsets()[i1]
        dx_store.append(
            f"if (u < {mul}) {{\n#pragma unroll\n  for (int i = 0; i < {ir.dim}; ++i) dxrow[{off} + u * {ir.dim} + i] = dxi{i1}[i];\n}}"
        )
    dx_zero = []
    for i1, (mul, ir) in enumerate(spec.irreps_in1):
        if i1 not in L.in1_used and mul * ir.dim > 0:
            dx_zero.append(f"for (int c = u; c < {mul * ir.dim}; c += {G}) dxrow[{spec.irreps_in1.offsets()[i1]} + c] = 0.0f;")

    fwd_body = emit_forward_body(L)
    bwd_body = emit_backward_body(L, want_dx=True)
    bwd_body_nodx = emit_backward_body(L, want_dx=False)
    dx_body = emit_dx_body(L)
    dx_atomic = "\n".join(
        f"if (u < {spec.irreps_in1[i1].mul}) {{\n#pragma unroll\n  for (int i = 0; i < {spec.irreps_in1[i1].ir.dim}; ++i) "
        f"atomicAdd(dxrow + {spec.irreps_in1.offsets()[i1]} + u * {spec.irreps_in1[i1].ir.dim} + i, dxi{i1}[i]);\n}}"
        for i1 in L.in1_used)
    y_load = f"float Y[{max(L.d2, 1)}];\n#pragma unroll\nfor (int j = 0; j < {L.d2}; ++j) Y[j] = yrow[j];"

    has_sh = sh_l is not None
    warps_per_group = max(1, G // 32)
    v2 = uvu_tma.emit(L)
    v2_kernel = v2["kernel"] if v2 else ""
    v2_launch = v2["launch"] if v2 else ""
    b2 = uvu_tma_bwd.emit(L) if v2 else None
    if b2:
        v2_kernel += b2["kernel"]
    b2_launch = b2["launch"] if b2 else ""
    x2k = uvu_tma_bwdx.emit(L) if b2 else None
    if x2k:
        v2_kernel += x2k["kernel"]
    x2_launch = x2k["launch"] if x2k else ""

    src = f"""// Generated by e3nn_b200/codegen/uvu.py -- do not edit.
// layout: {spec.irreps_in1} (x) {spec.irreps_in2} -> {spec.irreps_out}, {len(L.paths)} 'uvu' paths, key {spec.key()}
#include <cuda_runtime.h>
#include <cstdint>
#include "layout_common.cuh"
#include "tc_common.cuh"
{'#include "sh_gen.cuh"' if has_sh else ''}

namespace {{

int g_conv_impl = 0;   // 0: pick the fastest eligible kernel, 1: always the direct-load kernel

constexpr int kD1 = {L.d1};
constexpr int kD2 = {L.d2};
constexpr int kDout = {L.dout};
constexpr int kWn = {L.wn};
constexpr int kG = {G};                 // threads per row (one channel each)
constexpr int kThreads = {threads};
constexpr int kRowsPerBlock = {rows_per_block};
constexpr int kShLmax = {sh_l if has_sh else -1};
constexpr int kWarpsPerGroup = {warps_per_group};

// ---------------------------------------------------------------- rows -> rows
__global__ void __launch_bounds__(kThreads) uvu_fwd_kernel(const float* __restrict__ x1, const float* __restrict__ x2,
        const float* __restrict__ w, float* __restrict__ out, int64_t Z, int w_shared) {{
    const int u = threadIdx.x % kG;
    const int slot = threadIdx.x / kG;
    for (int64_t z = static_cast<int64_t>(blockIdx.x) * kRowsPerBlock + slot; z < Z;
         z += static_cast<int64_t>(gridDim.x) * kRowsPerBlock) {{
        const float* xrow = x1 + z * kD1;
        const float* yrow = x2 + z * kD2;
        const float* wrow = w_shared ? w : w + z * kWn;
        float* orow = out + z * kDout;
{_indent(y_load, 8)}
{_indent(chr(10).join(acc_decl), 8)}
{_indent(fwd_body, 8)}
{_indent(chr(10).join(acc_store_rows), 8)}
{_indent(zero_code, 8)}
    }}
}}

// ---------------------------------------------------------------- rows: vector-Jacobian product
// dw_mode: 0 = per-row weights (plain store), 1 = shared weights (atomicAdd into a zeroed buffer)
__global__ void __launch_bounds__(kThreads) uvu_bwd_kernel(const float* __restrict__ x1, const float* __restrict__ x2,
        const float* __restrict__ w, const float* __restrict__ gout, float* __restrict__ grad_x1, float* __restrict__ grad_x2,
        float* __restrict__ grad_w, int64_t Z, int w_shared) {{
    __shared__ float s_dy[kRowsPerBlock][kWarpsPerGroup][kD2 > 0 ? kD2 : 1];
    const int u = threadIdx.x % kG;
    const int slot = threadIdx.x / kG;
    const int64_t rounds = (Z + static_cast<int64_t>(gridDim.x) * kRowsPerBlock - 1) / (static_cast<int64_t>(gridDim.x) * kRowsPerBlock);
    for (int64_t r = 0; r < rounds; ++r) {{
        const int64_t z = (r * gridDim.x + blockIdx.x) * kRowsPerBlock + slot;
        const bool live = z < Z;
        float dY[kD2 > 0 ? kD2 : 1];
#pragma unroll
        for (int j = 0; j < kD2; ++j) dY[j] = 0.0f;
        if (live) {{
            const float* xrow = x1 + z * kD1;
            const float* yrow = x2 + z * kD2;
            const float* wrow = w_shared ? w : w + z * kWn;
            const float* grow = gout + z * kDout;
            float* dxrow = grad_x1 + z * kD1;
            float* dwrow = w_shared ? grad_w : grad_w + z * kWn;
#define E3B_STORE_DW(idx, val) do {{ if (w_shared) atomicAdd(dwrow + (idx), (val)); else dwrow[(idx)] = (val); }} while (0)
{_indent(y_load, 12)}
{_indent(chr(10).join(g_load_rows), 12)}
{_indent(bwd_body, 12)}
#undef E3B_STORE_DW
{_indent(chr(10).join(dx_store), 12)}
{_indent(chr(10).join(dx_zero), 12)}
        }}
        // reduce dY over the channels of the row: lanes, then warps of the group
        e3b_group_reduce<kG, kD2>(dY, &s_dy[slot][0][0], u);
        if (live && u < kD2) {{
            float v = 0.0f;
#pragma unroll
            for (int q = 0; q < kWarpsPerGroup; ++q) v += s_dy[slot][q][u];
            grad_x2[z * kD2 + u] = v;
        }}
        if (live) for (int j = kG + u; j < kD2; j += kG) {{
            float v = 0.0f;
            for (int q = 0; q < kWarpsPerGroup; ++q) v += s_dy[slot][q][j];
            grad_x2[z * kD2 + j] = v;
        }}
        __syncthreads();
    }}
}}

// ---------------------------------------------------------------- fused gather -> (SH) -> uvu -> per-destination sum
// One group of kG threads owns a destination row at a time and walks its CSR segment.
// in2_mode: 0 = x2 holds precomputed rows [E,kD2]; 1 = x2 holds edge vectors [E,3] and the
// spherical harmonics (normalize=True, 'component') are evaluated here.
template <int IN2_MODE>
__global__ void __launch_bounds__(kThreads) conv_fwd_kernel(const float* __restrict__ node_x, const float* __restrict__ x2,
        const int64_t* __restrict__ edge_src, const int64_t* __restrict__ rowptr, const int64_t* __restrict__ perm,
        const float* __restrict__ w, float* __restrict__ out, int64_t num_nodes, int64_t num_src, float scale,
        int* __restrict__ status) {{
    const int u = threadIdx.x % kG;
    const int slot = threadIdx.x / kG;
    for (int64_t n = static_cast<int64_t>(blockIdx.x) * kRowsPerBlock + slot; n < num_nodes;
         n += static_cast<int64_t>(gridDim.x) * kRowsPerBlock) {{
        float* orow = out + n * kDout;
{_indent(chr(10).join(acc_decl), 8)}
        const int64_t e_begin = rowptr[n], e_end = rowptr[n + 1];
        for (int64_t ee = e_begin; ee < e_end; ++ee) {{
            const int64_t e = perm ? perm[ee] : ee;
            const int64_t s = edge_src[e];
            if (s < 0 || s >= num_src) {{ if (u == 0) atomicExch(status, 2); continue; }}
            const float* xrow = node_x + s * kD1;
            const float* wrow = w + e * kWn;
            float Y[kD2 > 0 ? kD2 : 1];
            if (IN2_MODE == 1) {{
                e3b_sh_unit<kShLmax>(x2 + e * 3, Y);
            }} else {{
                const float* yrow = x2 + e * kD2;
#pragma unroll
                for (int j = 0; j < kD2; ++j) Y[j] = yrow[j];
            }}
{_indent(fwd_body, 12)}
        }}
{_indent(chr(10).join(acc_store_conv), 8)}
{_indent(zero_code, 8)}
    }}
}}

// ---------------------------------------------------------------- gradient of conv_fwd w.r.t. the node features
// grad_node_x[src[e], u, i] += sum_paths sum_k t_ik(Y_e) w[e, p, u] g[dst, p, u, k]: one group per destination
// row (its cotangent stays in registers), float atomics into the zeroed table (sources are not sorted).
template <int IN2_MODE>
__global__ void __launch_bounds__(kThreads) conv_bwd_x_kernel(const float* __restrict__ x2, const int64_t* __restrict__ edge_src,
        const int64_t* __restrict__ rowptr, const int64_t* __restrict__ perm, const float* __restrict__ w,
        const float* __restrict__ gout, float* __restrict__ grad_node_x, int64_t num_nodes, int64_t num_src, float scale,
        int* __restrict__ status) {{
    const int u = threadIdx.x % kG;
    const int slot = threadIdx.x / kG;
    for (int64_t n = static_cast<int64_t>(blockIdx.x) * kRowsPerBlock + slot; n < num_nodes;
         n += static_cast<int64_t>(gridDim.x) * kRowsPerBlock) {{
        const float* grow = gout + n * kDout;
{_indent(chr(10).join(g_load_conv), 8)}
        const int64_t e_begin = rowptr[n], e_end = rowptr[n + 1];
        for (int64_t ee = e_begin; ee < e_end; ++ee) {{
            const int64_t e = perm ? perm[ee] : ee;
            const int64_t s = edge_src[e];
            if (s < 0 || s >= num_src) {{ if (u == 0) atomicExch(status, 2); continue; }}
            const float* wrow = w + e * kWn;
            float* dxrow = grad_node_x + s * kD1;
            float Y[kD2 > 0 ? kD2 : 1];
            if (IN2_MODE == 1) {{
                e3b_sh_unit<kShLmax>(x2 + e * 3, Y);
            }} else {{
                const float* yrow = x2 + e * kD2;
#pragma unroll
                for (int j = 0; j < kD2; ++j) Y[j] = yrow[j];
            }}
{_indent(dx_body, 12)}
{_indent(dx_atomic, 12)}
        }}
    }}
}}

// ---------------------------------------------------------------- gradient of conv_fwd w.r.t. weights and in2 / edge vectors
template <int IN2_MODE>
__global__ void __launch_bounds__(kThreads) conv_bwd_kernel(const float* __restrict__ node_x, const float* __restrict__ x2,
        const int64_t* __restrict__ edge_src, const int64_t* __restrict__ rowptr, const int64_t* __restrict__ perm,
        const float* __restrict__ w, const float* __restrict__ gout, float* __restrict__ grad_w, float* __restrict__ grad_x2,
        int64_t num_nodes, int64_t num_src, float scale, int* __restrict__ status) {{
    __shared__ float s_dy[kRowsPerBlock][kWarpsPerGroup][kD2 > 0 ? kD2 : 1];
    const int u = threadIdx.x % kG;
    const int slot = threadIdx.x / kG;
    const int64_t per_round = static_cast<int64_t>(gridDim.x) * kRowsPerBlock;
    const int64_t rounds = (num_nodes + per_round - 1) / per_round;
    for (int64_t r = 0; r < rounds; ++r) {{
        const int64_t n = (r * gridDim.x + blockIdx.x) * kRowsPerBlock + slot;
        const bool node_live = n < num_nodes;
        const int64_t e_begin = node_live ? rowptr[n] : 0, e_end = node_live ? rowptr[n + 1] : 0;
        // longest segment among the rows of this block decides the trip count (block-uniform barriers)
        __shared__ long long s_len[kRowsPerBlock];
        if (u == 0) s_len[slot] = e_end - e_begin;
        __syncthreads();
        long long trips = 0;
        for (int q = 0; q < kRowsPerBlock; ++q) trips = max(trips, s_len[q]);
        const float* grow = gout + (node_live ? n : 0) * kDout;
{_indent(chr(10).join(g_load_conv), 8)}
        for (long long it = 0; it < trips; ++it) {{
            const int64_t ee = e_begin + it;
            const bool live = ee < e_end;
            float dY[kD2 > 0 ? kD2 : 1];
#pragma unroll
            for (int j = 0; j < kD2; ++j) dY[j] = 0.0f;
            int64_t e = 0;
            float Y[kD2 > 0 ? kD2 : 1];
            float vx = 0.f, vy = 0.f, vz = 0.f;
            bool ok = live;
            if (live) {{
                e = perm ? perm[ee] : ee;
                const int64_t s = edge_src[e];
                if (s < 0 || s >= num_src) {{ if (u == 0) atomicExch(status, 2); ok = false; }}
                if (ok) {{
                    const float* xrow = node_x + s * kD1;
                    const float* wrow = w + e * kWn;
                    float* dwrow = grad_w + e * kWn;
                    if (IN2_MODE == 1) {{
                        vx = x2[e * 3]; vy = x2[e * 3 + 1]; vz = x2[e * 3 + 2];
                        e3b_sh_unit<kShLmax>(x2 + e * 3, Y);
                    }} else {{
                        const float* yrow = x2 + e * kD2;
#pragma unroll
                        for (int j = 0; j < kD2; ++j) Y[j] = yrow[j];
                    }}
#define E3B_STORE_DW(idx, val) dwrow[(idx)] = (val)
{_indent(bwd_body_nodx, 20)}
#undef E3B_STORE_DW
                }}
            }}
            e3b_group_reduce<kG, kD2>(dY, &s_dy[slot][0][0], u);
            if (ok) {{
                if (IN2_MODE == 1) {{
                    if (u == 0) {{
                        float gY[kD2 > 0 ? kD2 : 1];
#pragma unroll
                        for (int j = 0; j < kD2; ++j) {{
                            float v = 0.0f;
#pragma unroll
                            for (int q = 0; q < kWarpsPerGroup; ++q) v += s_dy[slot][q][j];
                            gY[j] = v;
                        }}
                        float gx, gy, gz;
                        e3b_sh_unit_bwd<kShLmax>(vx, vy, vz, gY, gx, gy, gz);
                        grad_x2[e * 3] = gx; grad_x2[e * 3 + 1] = gy; grad_x2[e * 3 + 2] = gz;
                    }}
                }} else {{
                    for (int j = u; j < kD2; j += kG) {{
                        float v = 0.0f;
                        for (int q = 0; q < kWarpsPerGroup; ++q) v += s_dy[slot][q][j];
                        grad_x2[e * kD2 + j] = v;
                    }}
                }}
            }}
            __syncthreads();
        }}
        __syncthreads();
    }}
}}

{v2_kernel}
}}  // namespace

// ================================================================= C ABI of the layout module
extern "C" int e3b_conv_select(int impl) {{ g_conv_impl = impl; return {1 if v2 else 0}; }}

extern "C" int e3b_layout_info(int32_t* dims) {{
    dims[0] = kD1; dims[1] = kD2; dims[2] = kDout; dims[3] = kWn; dims[4] = kShLmax; dims[5] = kG;
    return 0;
}}

extern "C" const char* e3b_layout_key(void) {{ return "{spec.key()}"; }}

extern "C" const char* e3b_layout_last_error(void) {{ return e3b_layout_error_buffer(); }}

extern "C" int e3b_uvu_fwd(const float* x1, const float* x2, const float* w, float* out, int64_t Z, int w_shared,
                           void* stream) {{
    if (Z < 0) return e3b_layout_fail(-1, "uvu_fwd: negative row count");
    if (Z == 0) return 0;
    if (!x1 || !x2 || !out || (kWn > 0 && !w)) return e3b_layout_fail(-1, "uvu_fwd: null pointer");
    const int64_t blocks = (Z + kRowsPerBlock - 1) / kRowsPerBlock;
    const unsigned grid = static_cast<unsigned>(blocks < 148LL * 64 ? blocks : 148LL * 64);
    uvu_fwd_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(x1, x2, w, out, Z, w_shared);
    return e3b_layout_check("uvu_fwd");
}}

extern "C" int e3b_uvu_bwd(const float* x1, const float* x2, const float* w, const float* grad_out, float* grad_x1,
                           float* grad_x2, float* grad_w, int64_t Z, int w_shared, void* stream) {{
    if (Z < 0) return e3b_layout_fail(-1, "uvu_bwd: negative row count");
    if (Z == 0) return 0;
    if (!x1 || !x2 || !grad_out || !grad_x1 || !grad_x2 || (kWn > 0 && (!w || !grad_w)))
        return e3b_layout_fail(-1, "uvu_bwd: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (w_shared && kWn > 0) {{
        cudaError_t err = cudaMemsetAsync(grad_w, 0, sizeof(float) * kWn, s);
        if (err != cudaSuccess) return e3b_layout_fail(-2, "uvu_bwd: memset: %s", cudaGetErrorString(err));
    }}
    const int64_t blocks = (Z + kRowsPerBlock - 1) / kRowsPerBlock;
    const unsigned grid = static_cast<unsigned>(blocks < 148LL * 64 ? blocks : 148LL * 64);
    uvu_bwd_kernel<<<grid, kThreads, 0, s>>>(x1, x2, w, grad_out, grad_x1, grad_x2, grad_w, Z, w_shared);
    return e3b_layout_check("uvu_bwd");
}}

extern "C" int e3b_conv_fwd(const float* node_x, const float* x2, int in2_mode, const int64_t* edge_src,
                            const int64_t* rowptr, const int64_t* perm, const float* w, float* out, int64_t num_nodes,
                            int64_t num_src, int64_t num_edges, float scale, int32_t* status, void* stream) {{
    if (num_nodes < 0 || num_edges < 0) return e3b_layout_fail(-1, "conv_fwd: negative size");
    if (num_nodes == 0) return 0;
    if (!rowptr || !out || !status || (num_edges > 0 && (!node_x || !x2 || !edge_src || (kWn > 0 && !w))))
        return e3b_layout_fail(-1, "conv_fwd: null pointer");
    if (in2_mode == 1 && kShLmax < 0) return e3b_layout_fail(-3, "conv_fwd: irreps_in2 is not Y^0..Y^L, pass rows instead");
    const int64_t blocks = (num_nodes + kRowsPerBlock - 1) / kRowsPerBlock;
    const unsigned grid = static_cast<unsigned>(blocks < 148LL * 64 ? blocks : 148LL * 64);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
{v2_launch}
    if (in2_mode == 1)
        conv_fwd_kernel<1><<<grid, kThreads, 0, s>>>(node_x, x2, edge_src, rowptr, perm, w, out, num_nodes, num_src, scale, status);
    else
        conv_fwd_kernel<0><<<grid, kThreads, 0, s>>>(node_x, x2, edge_src, rowptr, perm, w, out, num_nodes, num_src, scale, status);
    return e3b_layout_check("conv_fwd");
}}

extern "C" int e3b_conv_bwd(const float* node_x, const float* x2, int in2_mode, const int64_t* edge_src,
                            const int64_t* rowptr, const int64_t* perm, const float* w, const float* grad_out,
                            float* grad_w, float* grad_x2, int64_t num_nodes, int64_t num_src, int64_t num_edges,
                            float scale, int32_t* status, void* stream) {{
    if (num_nodes < 0 || num_edges < 0) return e3b_layout_fail(-1, "conv_bwd: negative size");
    if (num_nodes == 0 || num_edges == 0) return 0;
    if (!rowptr || !grad_out || !status || !node_x || !x2 || !edge_src || !grad_x2 || (kWn > 0 && (!w || !grad_w)))
        return e3b_layout_fail(-1, "conv_bwd: null pointer");
    if (in2_mode == 1 && kShLmax < 0) return e3b_layout_fail(-3, "conv_bwd: irreps_in2 is not Y^0..Y^L, pass rows instead");
    const int64_t blocks = (num_nodes + kRowsPerBlock - 1) / kRowsPerBlock;
    const unsigned grid = static_cast<unsigned>(blocks < 148LL * 64 ? blocks : 148LL * 64);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
{b2_launch}
    if (in2_mode == 1)
        conv_bwd_kernel<1><<<grid, kThreads, 0, s>>>(node_x, x2, edge_src, rowptr, perm, w, grad_out, grad_w, grad_x2, num_nodes, num_src, scale, status);
    else
        conv_bwd_kernel<0><<<grid, kThreads, 0, s>>>(node_x, x2, edge_src, rowptr, perm, w, grad_out, grad_w, grad_x2, num_nodes, num_src, scale, status);
    return e3b_layout_check("conv_bwd");
}}

// Gradient of e3b_conv_fwd w.r.t. the node features: grad_node_x [num_src, kD1] is overwritten.
extern "C" int e3b_conv_bwd_x(const float* x2, int in2_mode, const int64_t* edge_src, const int64_t* rowptr,
                              const int64_t* perm, const float* w, const float* grad_out, float* grad_node_x,
                              int64_t num_nodes, int64_t num_src, int64_t num_edges, float scale, int32_t* status,
                              void* stream) {{
    if (num_nodes < 0 || num_edges < 0 || num_src < 0) return e3b_layout_fail(-1, "conv_bwd_x: negative size");
    if (num_src == 0) return 0;
    if (!grad_node_x) return e3b_layout_fail(-1, "conv_bwd_x: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaMemsetAsync(grad_node_x, 0, sizeof(float) * kD1 * static_cast<size_t>(num_src), s);
    if (err != cudaSuccess) return e3b_layout_fail(-2, "conv_bwd_x: memset: %s", cudaGetErrorString(err));
    if (num_nodes == 0 || num_edges == 0) return 0;
    if (!rowptr || !grad_out || !status || !x2 || !edge_src || (kWn > 0 && !w)) return e3b_layout_fail(-1, "conv_bwd_x: null pointer");
    if (in2_mode == 1 && kShLmax < 0) return e3b_layout_fail(-3, "conv_bwd_x: irreps_in2 is not Y^0..Y^L, pass rows instead");
{x2_launch}
    const int64_t blocks = (num_nodes + kRowsPerBlock - 1) / kRowsPerBlock;
    const unsigned grid = static_cast<unsigned>(blocks < 148LL * 64 ? blocks : 148LL * 64);
    if (in2_mode == 1)
        conv_bwd_x_kernel<1><<<grid, kThreads, 0, s>>>(x2, edge_src, rowptr, perm, w, grad_out, grad_node_x, num_nodes, num_src, scale, status);
    else
        conv_bwd_x_kernel<0><<<grid, kThreads, 0, s>>>(x2, edge_src, rowptr, perm, w, grad_out, grad_node_x, num_nodes, num_src, scale, status);
    return e3b_layout_check("conv_bwd_x");
}}
"""
    return src
