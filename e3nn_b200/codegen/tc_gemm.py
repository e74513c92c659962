"""Generator of fp32-accurate tensor-core kernels for the weight-shared contractions of the path:
fully-connected ('uvw') tensor products and the per-irrep Linear (forward and its transpose).

Both are, per output irrep ("group"), a GEMM ``D[(z,k), n] = sum_K A[(z,k), K] * B[K, n]`` whose left
operand is produced on the fly from the input rows (Clebsch-Gordan contraction for 'uvw', a strided
copy for Linear) and whose right operand is the (scaled) weight matrix.

tcgen05 has no fp32 MMA; plain tf32 operands give ~1e-3 relative error.  The kernel therefore splits
both operands into ``hi = tf32(x)`` and ``lo = tf32(x - hi)`` and issues three ``kind::tf32`` MMAs per
k-step (``lo*hi + hi*lo + hi*hi``, fp32 accumulation in tensor memory): "3xTF32", 22-bit operands.
Measured on B200: 1e-5 .. 4e-5 x RMS (max-abs) on the 320-term contractions of this path, i.e. about
1000x better than plain tf32 but not inside the 1e-5 fp32 bound; a third piece (``hi + mid + lo``,
six MMAs) was measured to change nothing, so the remaining error is the accumulation in tensor
memory, not the operands.  ``precision = 1`` issues only ``hi*hi`` (the 2e-2 x RMS class).  The
strict fp32 mode of the modules therefore stays on the CUDA-core kernel (csrc/dense.cu).

Structure (persistent, one CTA per SM, a CTA serves one group):
  * a small preparation kernel writes, once per call, the weights of every group pre-scaled,
    pre-split (hi, lo) and pre-swizzled in chunks of 32 K, so that the main kernel fetches one
    chunk with a single ``cp.async.bulk`` copy per pipeline stage (``mbarrier`` complete_tx);
  * rows of a 128-row tile are (z, k) pairs, z-major: 128 // (2l+1) rows of z per tile;
  * 8 producer warps build A (hi, lo) for 32 consecutive K of the tile in the K-major 128-byte
    swizzled layout; lane = K index, every global load of a warp's rows is issued before first use;
  * one thread issues the MMAs; ``tcgen05.commit`` releases stages / publishes accumulators;
  * 4 epilogue warps read tensor memory (``tcgen05.ld``) and write the output rows while the next
    tile accumulates in the second TMEM buffer.
Every wait is bounded (mbarrier try_wait with an iteration limit, block-wide abort flag).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..o3._irreps import Irreps
from ..o3._spec import TPSpec
from ..o3._wigner import wigner_3j_numpy

SMEM_LIMIT = 227 * 1024
A_TILE = 128 * 128          # one 128 x 32 fp32 sub-tile
Y_BYTES = 8192
EPI_BYTES = 4 * 32 * 64 * 4   # 4 epilogue warps x (32 rows x 64 columns) fp32
PRODUCER_WARPS = 8          # default; GemmSpec.producer_warps selects 8 or 16 per module
SWAP_DIMS = (3, 5)          # 2l+1 for which the transposed Linear runs with swapped operands (see Group.swap)
PIECES = 2                  # tf32 pieces the stages have room for (hi, lo); 3 is supported by the code below


def _f(v: float) -> str:
    return f"{np.float32(v):.9e}f"


@dataclass
class Chunk:
    case: int          # producer case (one per distinct (l1,l2,l3,off2) code body)
    xoff: int          # offset of x1[., u0, 0] in the input row
    wbase: int         # B[kk, n] = scale * W[wbase + kk * sk + n * sn]
    sk: int
    sn: int
    scale: float
    # column blocks of equal width with their own weight slice and scale (several paths side by side in N);
    # None: one block, (wbase, scale)
    blocks: Optional[List[Tuple[int, float]]] = None


@dataclass
class Group:
    out_off: int
    n: int
    dim: int
    chunks: List[Chunk] = field(default_factory=list)
    cases: List[str] = field(default_factory=list)       # code of each producer case
    case_cost: List[int] = field(default_factory=list)
    case_d1: List[int] = field(default_factory=list)

    @property
    def zt(self) -> int:
        return 128 // self.dim

    has_y: bool = True
    aligned_out: bool = True   # output rows allow 16-byte stores
    plain: bool = False        # A is the input rows themselves (dense layer): 16-byte loads and stores
    # two MMAs per k-step in the split mode (a_hi x [b_hi | b_lo], a_lo x b_hi) instead of three; needs N <= 128
    # and twice the accumulator columns, pays for long contractions (the epilogue reads twice the columns); measured
    # neutral on the Linear groups (N = 64, K = 256-448: 3.05 against 3.07 ms), so only the transposed dense layer uses it
    wide_b: bool = False
    # Operands swapped in the MMA (rows of the accumulator = output channels, columns = the (z, k) rows of the
    # produced tile): a warp then stores one component of 32 consecutive channels of ONE row z per instruction
    # instead of touching 32 / (2l+1) rows.  For 2l+1 > 1 groups of transposed Linears whose width is a multiple of 128.
    swap: bool = False

    def resident_bytes(self) -> int:
        """Bytes of the prepared B operand when all of it stays in shared memory for the life of the CTA:
        groups with K <= 128 (at most four chunks), where re-fetching B for every row tile would move as
        many bytes as the output itself.  0 when B is streamed with the A chunks."""
        total = len(self.chunks) * PIECES * self.n * 128
        room = SMEM_LIMIT - 3072 - self.extra_bytes() - total
        return total if (0 < len(self.chunks) <= 4 and room >= 3 * PIECES * A_TILE) else 0

    def stage_bytes(self) -> int:
        return PIECES * A_TILE + (0 if self.resident_bytes() else PIECES * self.n * 128)

    def staged_epilogue(self) -> bool:
        """dim == 1 groups transpose their output through shared memory for fully coalesced stores."""
        return self.dim == 1 and self.n % 64 == 0 and self.aligned_out and not self.swap

    def extra_bytes(self) -> int:
        return (Y_BYTES if self.has_y else 0) + (EPI_BYTES if self.staged_epilogue() else 0)

    def nstage(self) -> int:
        return int(max(0, min(6, (SMEM_LIMIT - 3072 - self.extra_bytes() - self.resident_bytes()) // self.stage_bytes())))

    def smem_bytes(self) -> int:
        return self.resident_bytes() + self.nstage() * self.stage_bytes() + self.extra_bytes() + 1024 + 1024

    def work(self) -> int:
        # per 128-row tile: the producers' chunks plus the epilogue (tensor-memory loads and stores of N columns per
        # row; the dominant term of short-K groups)
        per_tile = sum(40 + self.case_cost[c.case] * max(1, -(-self.zt // PRODUCER_WARPS)) for c in self.chunks)
        per_tile += 4 * self.n
        return max(1, int(1000 * per_tile / self.zt))


@dataclass
class GemmSpec:
    d1: int
    d2: int
    dout: int
    groups: List[Group]
    key: str
    title: str
    zero_ranges: List[Tuple[int, int]] = field(default_factory=list)   # output columns no group writes
    # 8 producer warps (13 warps per CTA, 128 registers each) suit contractions bound by their output stores
    # (K <= 128); 16 (21 warps, 80 registers) hide the operand-load latency of long-K contractions
    producer_warps: int = 8
    # dense layers: the raw fp32 rows are the hi operand piece (the tensor core ignores the low 13 mantissa
    # bits), brought into the swizzled stage by 2-D tensor-map TMA copies issued by a dedicated warp
    tma_a: bool = False


# ------------------------------------------------------------------------------------------- front ends
def _uvw_case(l1: int, l2: int, l3: int, off2: int, pw: float) -> Tuple[str, int]:
    """Producer body for a 'uvw' path: vals[k] from xi[q][i] and the x2 row in shared memory (sy)."""
    c = wigner_3j_numpy(l1, l2, l3) * pw
    d2 = 2 * l2 + 1
    lines = [f"float yj[{d2}];", f"#pragma unroll\nfor (int j = 0; j < {d2}; ++j) yj[j] = syq[{off2} + j];"]
    for k in range(2 * l3 + 1):
        terms = []
        for i in range(2 * l1 + 1):
            inner = [(j, c[i, j, k]) for j in range(d2) if c[i, j, k] != 0.0]
            if inner:
                t = " + ".join(f"{_f(v)} * yj[{j}]" for j, v in inner)
                terms.append(f"({t}) * xi[q][{i}]")
        lines.append(f"vals[{k}] = {' + '.join(terms) if terms else '0.0f'};")
    cost = (2 * l1 + 1) + d2 + 2 * int((c != 0).sum()) + 6 * (2 * l3 + 1)
    return "\n".join(lines), cost


def uvw_gemm_spec(spec: TPSpec) -> Optional[GemmSpec]:
    """'uvw' paths with shared weights, x2 multiplicities 1, x1 multiplicities multiples of 32."""
    if not spec.shared_weights:
        return None
    live = spec.live_instructions()
    if not live or any(ins.connection_mode != "uvw" for _, ins in live):
        return None
    if spec.irreps_in2.dim > 16:   # the x2 rows of a tile are staged in Y_BYTES of shared memory
        return None
    o1, o2, oo = spec.irreps_in1.offsets(), spec.irreps_in2.offsets(), spec.irreps_out.offsets()
    woffs = spec.weight_offsets()
    groups: Dict[int, Group] = {}
    for n, ins in live:
        (m1, ir1), (m2, ir2), (mo, iro) = spec.irreps_in1[ins.i_in1], spec.irreps_in2[ins.i_in2], spec.irreps_out[ins.i_out]
        if m2 != 1 or m1 % 32 != 0 or mo % 16 != 0 or not (16 <= mo <= 256):
            return None
        g = groups.setdefault(ins.i_out, Group(oo[ins.i_out], mo, iro.dim))
        code, cost = _uvw_case(ir1.l, ir2.l, iro.l, o2[ins.i_in2], float(ins.path_weight))
        g.cases.append(code)
        g.case_cost.append(cost)
        g.case_d1.append(ir1.dim)
        case = len(g.cases) - 1
        for u0 in range(0, m1, 32):
            g.chunks.append(Chunk(case, o1[ins.i_in1] + u0 * ir1.dim, woffs[n] + u0 * mo, mo, 1, 1.0))
    out = [groups[k] for k in sorted(groups)]
    for g in out:
        g.has_y = True
        g.aligned_out = spec.irreps_out.dim % 4 == 0 and g.out_off % 4 == 0
    if any(g.nstage() < 2 for g in out):
        return None
    written = set(groups)
    zero = [(oo[i], mul * ir.dim) for i, (mul, ir) in enumerate(spec.irreps_out) if i not in written and mul * ir.dim > 0]
    return GemmSpec(spec.irreps_in1.dim, spec.irreps_in2.dim, spec.irreps_out.dim, out, spec.key(),
                    f"uvw {spec.irreps_in1} (x) {spec.irreps_in2} -> {spec.irreps_out}", zero, producer_warps=16)


def linear_gemm_spec(irreps_in: Irreps, irreps_out: Irreps, instructions, transpose: bool, key: str) -> Optional[GemmSpec]:
    """Linear (or its transpose: output cotangents -> input cotangents) as a GemmSpec."""
    oi, oo = irreps_in.offsets(), irreps_out.offsets()
    woff, offs = 0, []
    for ins in instructions:
        if ins.i_in == -1:
            offs.append(-1)
            continue
        offs.append(woff)
        woff += ins.path_shape[0] * ins.path_shape[1]
    src, dst = (irreps_out, irreps_in) if transpose else (irreps_in, irreps_out)
    so, do = (oo, oi) if transpose else (oi, oo)
    live = [(n, ins) for n, ins in enumerate(instructions) if ins.i_in != -1 and 0 not in ins.path_shape
            and irreps_in[ins.i_in].dim > 0 and irreps_out[ins.i_out].dim > 0]
    if not live:
        return None
    groups: Dict[int, Group] = {}
    for n, ins in live:
        t = ins.i_in if transpose else ins.i_out
        s = ins.i_out if transpose else ins.i_in
        mul_t, ir = dst[t]
        mul_s = src[s].mul
        if mul_s % 32 != 0 or mul_t % 16 != 0 or not (16 <= mul_t <= 256):
            return None
        g = groups.setdefault(t, Group(do[t], mul_t, ir.dim))
        if not g.cases:
            g.cases.append("#pragma unroll\n" + f"for (int k = 0; k < {ir.dim}; ++k) vals[k] = xi[q][k];")
            g.case_cost.append(ir.dim + 6 * ir.dim)
            g.case_d1.append(ir.dim)
        mul_in, mul_out = ins.path_shape
        for u0 in range(0, mul_s, 32):
            if transpose:   # K index = w (output channel of the layer), n = u: W[u, w] at off + u * mul_out + w
                g.chunks.append(Chunk(0, so[s] + u0 * ir.dim, offs[n] + u0, 1, mul_out, float(ins.path_weight)))
            else:           # K index = u, n = w
                g.chunks.append(Chunk(0, so[s] + u0 * ir.dim, offs[n] + u0 * mul_out, mul_out, 1, float(ins.path_weight)))
    out = [groups[k] for k in sorted(groups)]
    if transpose:
        # Neighbouring output slots fed by the same input block (the paths of one l in a convolution layout)
        # become one group with the paths side by side in N: the shared A operand is loaded, split and stored
        # once per group instead of once per path.
        merged: List[Group] = []
        for g in out:
            m = merged[-1] if merged else None
            width = len(m.chunks[0].blocks) if (m and m.chunks[0].blocks) else 1
            limit = 192 if g.dim == 1 else 256   # (32 KB of epilogue staging + a resident N = 256 operand: two stages)
            if (m is not None and m.dim == g.dim and m.n // width == g.n and m.n + g.n <= limit
                    and g.out_off == m.out_off + m.n * m.dim and len(m.chunks) == len(g.chunks)
                    and all(a.xoff == b.xoff and a.sk == b.sk and a.sn == b.sn for a, b in zip(m.chunks, g.chunks))):
                for a, b in zip(m.chunks, g.chunks):
                    a.blocks = (a.blocks or [(a.wbase, a.scale)]) + [(b.wbase, b.scale)]
                m.n += g.n
            else:
                merged.append(g)
        out = merged
    for g in out:
        g.has_y = False
        g.aligned_out = dst.dim % 4 == 0 and g.out_off % 4 == 0
        g.swap = transpose and g.dim in SWAP_DIMS and g.n % 128 == 0 and not g.staged_epilogue()
    if any(g.nstage() < 2 for g in out):
        return None
    zero = [(do[i], mul * ir.dim) for i, (mul, ir) in enumerate(dst) if i not in groups and mul * ir.dim > 0]
    return GemmSpec(src.dim, 0, dst.dim, out, key,
                    f"linear{'^T' if transpose else ''} {irreps_in} -> {irreps_out}", zero,
                    producer_warps=8 if transpose else 16)


def matmul_gemm_spec(k: int, n: int, transpose: bool, scale: float, key: str) -> Optional[GemmSpec]:
    """``out[z, :] = scale * x[z, :] @ W`` with ``W`` row-major ``[k, n]`` (or, transposed, ``g @ W^T``):
    the dense layers of the radial network.  Wide outputs are cut into column tiles of at most 256."""
    if transpose:
        if n % 32 != 0 or k % 16 != 0 or not (16 <= k <= 256):
            return None
        g = Group(0, k, 1)
        g.cases.append("vals[0] = xi[q][0];")
        g.case_cost.append(8)
        g.case_d1.append(1)
        for n0 in range(0, n, 32):
            g.chunks.append(Chunk(0, n0, n0, 1, n, scale))
        g.wide_b = k <= 128 and n >= 8 * k and PIECES == 2
        groups = [g]
        d_in, d_out = n, k
    else:
        if k % 32 != 0 or n % 16 != 0:
            return None
        groups = []
        col = 0
        while col < n:
            width = min(192 if k <= 128 else 256, n - col)
            g = Group(col, width, 1)
            g.cases.append("vals[0] = xi[q][0];")
            g.case_cost.append(8)
            g.case_d1.append(1)
            for k0 in range(0, k, 32):
                g.chunks.append(Chunk(0, k0, k0 * n + col, n, 1, scale))
            groups.append(g)
            col += width
        d_in, d_out = k, n
    for g in groups:
        g.has_y = False
        g.aligned_out = d_out % 4 == 0 and g.out_off % 4 == 0
        g.plain = d_in % 4 == 0     # rows can be moved 16 bytes at a time (and described by a tensor map)
    if any(g.nstage() < 2 for g in groups) or not all(g.plain for g in groups):
        return None
    return GemmSpec(d_in, 0, d_out, groups, key, f"matmul{'^T' if transpose else ''} [{k} x {n}] scale {scale!r}",
                    producer_warps=16 if transpose else 8, tma_a=True)


# ------------------------------------------------------------------------------------------- emission
def _indent(text: str, n: int) -> str:
    pad = " " * n
    return "\n".join(pad + line if line and not line.startswith("#pragma") else line for line in text.split("\n"))


def emit_module(gs: GemmSpec) -> str:
    d1, d2, dout = gs.d1, gs.d2, gs.dout
    PRODUCER_WARPS = gs.producer_warps
    assert PRODUCER_WARPS in (8, 16)
    smem_max = max(g.smem_bytes() for g in gs.groups)
    assert smem_max <= SMEM_LIMIT
    has_y = d2 > 0

    consts, funcs = [], []
    prep_off = 0
    prep_offsets = []
    for gi, g in enumerate(gs.groups):
        nch = len(g.chunks)
        prep_offsets.append(prep_off)
        prep_off += nch * PIECES * g.n * 128
        arr = lambda name, vals, typ="int": f"__constant__ {typ} {name}{gi}[{len(vals)}] = {{{', '.join(str(v) for v in vals)}}};"
        nblk = len(g.chunks[0].blocks) if g.chunks[0].blocks else 1
        assert all((len(c.blocks) if c.blocks else 1) == nblk for c in g.chunks) and g.n % nblk == 0
        cblocks = [c.blocks if c.blocks else [(c.wbase, c.scale)] for c in g.chunks]
        consts.append("\n".join([
            arr("kCase", [c.case for c in g.chunks]),
            arr("kXOff", [c.xoff for c in g.chunks]),
            arr("kCD1", [g.case_d1[c.case] for c in g.chunks]),
            arr("kWBase", [wb for blks in cblocks for wb, _ in blks]),
            arr("kSK", [c.sk for c in g.chunks]),
            arr("kSN", [c.sn for c in g.chunks]),
            arr("kScale", [_f(sc) for blks in cblocks for _, sc in blks], "float"),
        ]))
        qn = -(-g.zt // PRODUCER_WARPS)
        def load_code(ci: int, xi: str, xoff: str) -> str:
            dd = g.case_d1[ci]
            return f"""#pragma unroll
for (int q = 0; q < {qn}; ++q) {{{{
    const float* xr = xrow[q] + ({xoff} + lane * {dd});
#pragma unroll
    for (int i = 0; i < {dd}; ++i) {xi}[q][i] = xr[i];
}}}}""".replace("{{", "{").replace("}}", "}")

        def compute_code(ci: int, xi: str, stage: str) -> str:
            body = g.cases[ci].replace("xi[q]", f"{xi}[q]")
            ysrc = f"const float* syq = sy + q * {d2};" if has_y else ""
            return f"""#pragma unroll
for (int q = 0; q < {qn}; ++q) {{{{
    const int zl = pw + {PRODUCER_WARPS} * q;
    if (zl < ZT) {{{{
        {ysrc}
        float vals[DIM];
{_indent(body, 8)}
#pragma unroll
        for (int k = 0; k < DIM; ++k) {{{{
            const uint32_t off = soff[q * DIM + k];
            const float hi = tc::to_tf32(vals[k]);
            *reinterpret_cast<float*>({stage} + off) = hi;
            if (pieces > 1) {{{{
                const float rest = vals[k] - hi;          // exact in fp32
                const float mid = tc::to_tf32(rest);
                *reinterpret_cast<float*>({stage} + A_TILE + off) = mid;
                if (pieces > 2) *reinterpret_cast<float*>({stage} + 2 * A_TILE + off) = tc::to_tf32(rest - mid);
            }}}}
        }}}}
    }}}}
}}}}""".replace("{{", "{").replace("}}", "}")

        cases = []
        for ci, code in enumerate(g.cases):
            dd = g.case_d1[ci]
            cases.append(
                f"case {ci}: {{\n    float xi[{qn}][{dd}];\n{_indent(load_code(ci, 'xi', 'xoff'), 4)}\n"
                f"    asm volatile(\"\" ::: \"memory\");   // every load above is in flight before the first use below\n"
                f"{_indent(compute_code(ci, 'xi', 'stage'), 4)}\n    break; }}"
            )
        # chunk batching: groups with a single cheap case load two chunks' rows before converting either,
        # doubling the bytes a producer warp keeps in flight (these groups stream their A rows from HBM)
        batch = 2 if (len(g.cases) == 1 and nch % 2 == 0 and qn * g.case_d1[0] <= 16 and g.nstage() >= 4) else 1
        switch = "\n".join(cases)
        issue_b_body = lambda stage, bar, c: "" if g.resident_bytes() else f"""{{{{
    const uint32_t bar = tc::smem_u32({bar});
    const uint32_t bbytes = pieces * B_HALF;   // only the pieces this precision uses
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bbytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(tc::smem_u32({stage} + {PIECES} * A_TILE)), "l"(bsrc + static_cast<size_t>({c}) * {PIECES} * B_HALF),
                   "r"(bbytes), "r"(bar) : "memory");
}}}}""".replace("{{", "{").replace("}}", "}")
        issue_b = lambda stage, bar, c: "" if g.resident_bytes() else "if (pw == 0 && lane == 0) " + issue_b_body(stage, bar, c)
        if batch == 1:
            PRODUCER_LOOP = f"""            for (int c = 0; c < NCHUNK; ++c, ++it) {{
                {{
                    // the input values of the chunk two ahead (of this tile, or of the CTA's next tile) are requested
                    // into L2 now: no registers are held, and the loads that follow find them closer
                    const bool same = c + 2 < NCHUNK;
                    const int cn = same ? c + 2 : (c + 2 - NCHUNK < NCHUNK ? c + 2 - NCHUNK : NCHUNK - 1);
                    const int64_t shift_rows = same ? 0 : static_cast<int64_t>(nctas) * ZT;
                    if (z0 + shift_rows < Z) {{
                        const int poff = kXOff{gi}[cn] + lane * kCD1{gi}[cn];
#pragma unroll
                        for (int q = 0; q < {qn}; ++q) {{
                            const int zl = pw + {PRODUCER_WARPS} * q;
                            int64_t z = z0 + shift_rows + (zl < ZT ? zl : 0);
                            if (z >= Z) z = Z - 1;
                            asm volatile("prefetch.global.L2 [%0];" ::"l"(x1 + z * {d1} + poff));
                        }}
                    }}
                }}
                const int s = it % NSTAGE;
                const uint32_t ph = (it / NSTAGE) & 1;
                if (!tc::mbar_wait(&bar_empty[s], ph ^ 1u, abort_flag)) {{ ok = false; break; }}
                uint8_t* stage = sS + s * STAGE_BYTES;
{_indent(issue_b('stage', '&bar_full[s]', 'c'), 16)}
                const int xoff = kXOff{gi}[c];
                switch (kCase{gi}[c]) {{
{_indent(switch, 16)}
                }}
                tc::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&bar_full[s]);"""
        else:
            dd = g.case_d1[0]
            # software pipeline over chunk pairs: the loads of the next pair are issued (into registers) before
            # this pair is converted, so a warp's load latency overlaps its own conversion work and barrier waits
            PRODUCER_LOOP = f"""            float xa[{qn}][{dd}], xb[{qn}][{dd}], na[{qn}][{dd}], nb[{qn}][{dd}];
{_indent(load_code(0, 'xa', f'kXOff{gi}[0]'), 12)}
{_indent(load_code(0, 'xb', f'kXOff{gi}[1]'), 12)}
            for (int c = 0; c < NCHUNK; c += 2, it += 2) {{
                if (c + 2 < NCHUNK) {{
{_indent(load_code(0, 'na', f'kXOff{gi}[c + 2]'), 20)}
{_indent(load_code(0, 'nb', f'kXOff{gi}[c + 3]'), 20)}
                }}
                asm volatile("" ::: "memory");   // the next pair's loads are in flight before anything below
                const int s0 = it % NSTAGE, s1 = (it + 1) % NSTAGE;
                const uint32_t ph0 = (it / NSTAGE) & 1, ph1 = ((it + 1) / NSTAGE) & 1;
                if (!tc::mbar_wait(&bar_empty[s0], ph0 ^ 1u, abort_flag)) {{ ok = false; break; }}
                if (!tc::mbar_wait(&bar_empty[s1], ph1 ^ 1u, abort_flag)) {{ ok = false; break; }}
                uint8_t* stage0 = sS + s0 * STAGE_BYTES;
                uint8_t* stage1 = sS + s1 * STAGE_BYTES;
{_indent(issue_b('stage0', '&bar_full[s0]', 'c'), 16)}
{_indent(issue_b('stage1', '&bar_full[s1]', '(c + 1)'), 16)}
{_indent(compute_code(0, 'xa', 'stage0'), 16)}
                tc::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&bar_full[s0]);
{_indent(compute_code(0, 'xb', 'stage1'), 16)}
                tc::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&bar_full[s1]);
#pragma unroll
                for (int q = 0; q < {qn}; ++q)
#pragma unroll
                    for (int i = 0; i < {dd}; ++i) {{ xa[q][i] = na[q][i]; xb[q][i] = nb[q][i]; }}"""
        y_load = f"""
            __syncwarp();
            for (int idx = lane; idx < {qn} * {d2}; idx += 32) {{   // x2 rows of this warp's z -> shared memory
                const int zl = pw + {PRODUCER_WARPS} * (idx / {d2});
                int64_t z = z0 + (zl < ZT ? zl : 0);
                if (z >= Z) z = Z - 1;
                sy[idx] = x2[z * {d2} + idx % {d2}];
            }}
            __syncwarp();""" if has_y else ""
        if g.plain and gs.tma_a:
            assert g.dim == 1 and g.zt == 128 and 128 % (4 * PRODUCER_WARPS) == 0 and not has_y
            RPW = 128 // PRODUCER_WARPS
            NJ = RPW // 4
            PRODUCER_BLOCK = f"""        // The stage's hi tile is the raw fp32 data, written by a tensor-map TMA copy (issued by the TMA warp).
        // A lane owns 16 bytes (4 consecutive K) of {NJ} rows: it reads them back, forms lo = x - trunc(x) rounded
        // to tf32 and stores the lo tile.  With one piece per operand there is nothing to convert.
        uint32_t po[{NJ}];
        const int pc4 = lane & 7;
#pragma unroll
        for (int j = 0; j < {NJ}; ++j) {{
            const int r = pw * {RPW} + 4 * j + (lane >> 3);
            po[j] = (r >> 3) * 1024 + (r & 7) * 128 + ((pc4 ^ (r & 7)) << 4);
        }}
        for (int64_t t = cta; t < tiles && ok; t += nctas) {{
            for (int c = 0; c < NCHUNK; ++c, ++it) {{
                const int s = it % NSTAGE;
                const uint32_t ph = (it / NSTAGE) & 1;
                if (!tc::mbar_wait(&bar_raw[s], ph, abort_flag)) {{ ok = false; break; }}
                uint8_t* stage = sS + s * STAGE_BYTES;
                if (pieces > 1) {{
#pragma unroll
                    for (int j = 0; j < {NJ}; ++j) {{
                        const float4 v = *reinterpret_cast<const float4*>(stage + po[j]);
                        *reinterpret_cast<float4*>(stage + A_TILE + po[j]) = tc::lo_piece4(v);
                    }}
                    tc::fence_proxy_async_smem();
                }}
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&bar_full[s]);
            }}
        }}
"""
        else:
            PRODUCER_BLOCK = f"""        uint32_t soff[{qn} * DIM];          // swizzled byte offsets of this thread's elements in an A sub-tile
#pragma unroll
        for (int q = 0; q < {qn}; ++q)
#pragma unroll
            for (int k = 0; k < DIM; ++k) soff[q * DIM + k] = tc::sw128_offset((pw + {PRODUCER_WARPS} * q) * DIM + k, lane);
        for (int64_t t = cta; t < tiles && ok; t += nctas) {{
            const int64_t z0 = t * ZT;
            const float* xrow[{qn}];          // input rows of this warp's z (rows past the end read the last row)
#pragma unroll
            for (int q = 0; q < {qn}; ++q) {{
                const int zl = pw + {PRODUCER_WARPS} * q;
                int64_t z = z0 + (zl < ZT ? zl : 0);
                if (z >= Z) z = Z - 1;
                xrow[q] = x1 + z * {d1};
            }}{y_load}
{PRODUCER_LOOP}
            }}
        }}
"""
        # gate applied to the 16 values a thread holds for row z (Linear followed by Gate): the table entry of a
        # channel (column of its component 0) gives kind, destination, activation and gate slot
        gated_store = """if (ep.tbl != nullptr) {
                        const int4 e0 = __ldg(reinterpret_cast<const int4*>(ep.tbl) + OUT_OFF + w0 * DIM);
                        const int4 e15 = __ldg(reinterpret_cast<const int4*>(ep.tbl) + OUT_OFF + (w0 + 15) * DIM);
                        const float* grow = ep.gates + z * ep.n_slots + e0.w;
                        if (e0.x == 1 && e15.x == 1 && e15.y == e0.y + 15 * DIM && e15.w == e0.w + 15 &&
                            (reinterpret_cast<uintptr_t>(grow) & 15u) == 0) {
                            // 16 consecutive gated channels with consecutive gates and destinations (the layout a Gate
                            // produces inside one irreps block): four 16-byte gate loads, no per-channel table reads
                            float4 gq[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) gq[q] = __ldg(reinterpret_cast<const float4*>(grow) + q);
                            float* dstp = ep.final_out + z * ep.dout_final + e0.y + kq;
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                dstp[(4 * q) * DIM] = __uint_as_float(r[4 * q]) * gq[q].x;
                                dstp[(4 * q + 1) * DIM] = __uint_as_float(r[4 * q + 1]) * gq[q].y;
                                dstp[(4 * q + 2) * DIM] = __uint_as_float(r[4 * q + 2]) * gq[q].z;
                                dstp[(4 * q + 3) * DIM] = __uint_as_float(r[4 * q + 3]) * gq[q].w;
                            }
                        } else {
#pragma unroll 1
                            for (int j = 0; j < 16; ++j) {
                                const int c = OUT_OFF + (w0 + j) * DIM;
                                const int4 e = __ldg(reinterpret_cast<const int4*>(ep.tbl) + c);
                                const float v = __uint_as_float(r[j]);
                                if (e.x == 1) ep.final_out[z * ep.dout_final + e.y + kq] = v * __ldg(ep.gates + z * ep.n_slots + e.w);
                                else if (e.x == 0) ep.final_out[z * ep.dout_final + e.y] = __ldg(ep.cst + c) * tc::gate_act(e.z, v);
                                else if (e.x == 2) ep.gates[z * ep.n_slots + e.w] = __ldg(ep.cst + c) * tc::gate_act(e.z, v);
                            }
                        }
                    } else """
        if g.dim == 1 and dout % 4 == 0 and g.out_off % 4 == 0:
            store = gated_store + """{
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        reinterpret_cast<float4*>(orow + w0)[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                                             __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                    }"""
        else:
            store = gated_store + """{
#pragma unroll
                    for (int j = 0; j < 16; ++j) orow[(w0 + j) * DIM + kq] = __uint_as_float(r[j]);
                    }"""
        if g.staged_epilogue():
            EPILOGUE = f"""            // 64 columns at a time: registers -> this warp's staging tile (16-byte chunks XOR-swizzled by row,
            // conflict free) -> read back two rows per instruction -> fully coalesced 256-byte row segments
            float* se = sE + warp * (32 * 64);
            for (int wb = 0; wb < N; wb += 64) {{{{
                float4* mine = reinterpret_cast<float4*>(se + lane * 64);
                const int sw = lane & 15;
#pragma unroll
                for (int h = 0; h < 2; ++h) {{{{
                    uint32_t r0[16], r1[16];
                    tc::tmem_ld16(tbase + wb + 32 * h, r0); tc::tmem_ld16(tbase + wb + 32 * h + 16, r1);
                    if (nparts == 1) tc::tmem_ld_wait();
                    for (int p = 1; p < nparts; ++p) {{{{   // further partial accumulators: summed here in fp32
                        uint32_t q0[16], q1[16];
                        const uint32_t po = part_off(p);
                        tc::tmem_ld16(tbase + po + wb + 32 * h, q0); tc::tmem_ld16(tbase + po + wb + 32 * h + 16, q1);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) {{{{
                            r0[j] = __float_as_uint(__uint_as_float(r0[j]) + __uint_as_float(q0[j]));
                            r1[j] = __float_as_uint(__uint_as_float(r1[j]) + __uint_as_float(q1[j]));
                        }}}}
                    }}}}
#pragma unroll
                    for (int c = 0; c < 4; ++c) {{{{
                        mine[(8 * h + c) ^ sw] = make_float4(__uint_as_float(r0[4 * c]), __uint_as_float(r0[4 * c + 1]), __uint_as_float(r0[4 * c + 2]), __uint_as_float(r0[4 * c + 3]));
                        mine[(8 * h + c + 4) ^ sw] = make_float4(__uint_as_float(r1[4 * c]), __uint_as_float(r1[4 * c + 1]), __uint_as_float(r1[4 * c + 2]), __uint_as_float(r1[4 * c + 3]));
                    }}}}
                }}}}
                __syncwarp();
                const int half = lane >> 4, cc = lane & 15;
                if (ep.tbl != nullptr) {{{{
                    // Gate on the scalar irreps: this lane's four columns keep their table entries for the 32 rows
                    int4 e[4];
                    float ec[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {{{{
                        const int c = OUT_OFF + wb + 4 * cc + q;
                        e[q] = __ldg(reinterpret_cast<const int4*>(ep.tbl) + c);
                        ec[q] = __ldg(ep.cst + c);
                    }}}}
                    // four columns of one kind with consecutive, 16-byte aligned destinations leave as one store
                    const bool same = e[0].x == e[1].x && e[0].x == e[2].x && e[0].x == e[3].x && e[0].z == e[1].z &&
                                      e[0].z == e[2].z && e[0].z == e[3].z;
                    const bool vec_s = same && e[0].x == 0 && e[1].y == e[0].y + 1 && e[2].y == e[0].y + 2 && e[3].y == e[0].y + 3 &&
                                       (e[0].y & 3) == 0 && (ep.dout_final & 3) == 0;
                    const bool vec_g = same && e[0].x == 2 && e[1].w == e[0].w + 1 && e[2].w == e[0].w + 2 && e[3].w == e[0].w + 3 &&
                                       (e[0].w & 3) == 0 && (ep.n_slots & 3) == 0;
#pragma unroll 4
                    for (int rr = 0; rr < 32; rr += 2) {{{{
                        const int rl = rr + half;
                        const float4 v = reinterpret_cast<const float4*>(se + rl * 64)[cc ^ (rl & 15)];
                        const int64_t zr = t * ZT + warp * 32 + rl;
                        if (zr >= Z) continue;
                        const float vv[4] = {{{{v.x, v.y, v.z, v.w}}}};
                        float a[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) a[q] = ec[q] * tc::gate_act(e[q].z, vv[q]);
                        if (vec_s) {{{{
                            *reinterpret_cast<float4*>(ep.final_out + zr * ep.dout_final + e[0].y) = make_float4(a[0], a[1], a[2], a[3]);
                        }}}} else if (vec_g) {{{{
                            *reinterpret_cast<float4*>(ep.gates + zr * ep.n_slots + e[0].w) = make_float4(a[0], a[1], a[2], a[3]);
                        }}}} else {{{{
#pragma unroll
                            for (int q = 0; q < 4; ++q) {{{{
                                if (e[q].x == 0) ep.final_out[zr * ep.dout_final + e[q].y] = a[q];
                                else if (e[q].x == 2) ep.gates[zr * ep.n_slots + e[q].w] = a[q];
                            }}}}
                        }}}}
                    }}}}
                }}}} else {{{{
#pragma unroll 4
                for (int rr = 0; rr < 32; rr += 2) {{{{
                    const int rl = rr + half;
                    const float4 v = reinterpret_cast<const float4*>(se + rl * 64)[cc ^ (rl & 15)];
                    const int64_t zr = t * ZT + warp * 32 + rl;
                    if (zr < Z) reinterpret_cast<float4*>(out + zr * {dout} + OUT_OFF + wb)[cc] = v;
                }}}}
                }}}}
                __syncwarp();
            }}}}""".replace("{{", "{").replace("}}", "}")
        elif g.swap:
            ncol = g.zt * g.dim          # live columns: the (z, k) rows of the produced tile
            blocks = []
            for c0 in range(0, ncol, 16):
                st = []
                for j in range(min(16, ncol - c0)):
                    zq, kq = divmod(c0 + j, g.dim)
                    st.append(f"                    if (z0 + {zq} < Z) orow_n[{zq}ll * {dout} + {kq}] = __uint_as_float(ra[{j}]);")
                blocks.append("\n".join([
                    "                {",
                    f"                    tc::tmem_ld16(tb + {c0}, ra);",
                    "                    if (nparts == 1) tc::tmem_ld_wait();",
                    "                    for (int p = 1; p < nparts; ++p) {",
                    f"                        tc::tmem_ld16(tb + part_off(p) + {c0}, rb);",
                    "                        tc::tmem_ld_wait();",
                    "#pragma unroll",
                    "                        for (int j = 0; j < 16; ++j) ra[j] = __float_as_uint(__uint_as_float(ra[j]) + __uint_as_float(rb[j]));",
                    "                    }",
                ] + st + ["                }"]))
            EPILOGUE = "\n".join([
                "            // swapped accumulator: lane = output channel n of this 128-channel tile, columns = (z, k) rows of the",
                "            // produced tile; for a fixed column the warp writes component k of 32 consecutive channels of row z",
                "            uint32_t ra[16], rb[16];",
                "            const int64_t z0 = t * ZT;",
                "            for (int m = 0; m < N / 128; ++m) {",
                "                const int n = m * 128 + warp * 32 + lane;",
                f"                float* orow_n = out + z0 * {dout} + OUT_OFF + n * DIM;",
                "                const uint32_t tb = tbase + m * 128;",
            ] + blocks + ["            }"])
        else:
            EPILOGUE = f"""            // 16 columns per tcgen05.ld; the next load is in flight while the previous block is stored
            // (a register block is only read after the wait that follows its load)
            auto store16 = [&](const uint32_t (&r)[16], int w0) {{{{
                if (valid) {{{{
{store}
                }}}}
            }}}};
            uint32_t ra[16], rb[16];
            for (int w0 = 0; w0 < N; w0 += 16) {{{{
                tc::tmem_ld16(tbase + w0, ra);
                if (nparts == 1) tc::tmem_ld_wait();
                for (int p = 1; p < nparts; ++p) {{{{
                    tc::tmem_ld16(tbase + part_off(p) + w0, rb);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) ra[j] = __float_as_uint(__uint_as_float(ra[j]) + __uint_as_float(rb[j]));
                }}}}
                store16(ra, w0);
            }}}}""".replace("{{", "{").replace("}}", "}")
        ACC_WAIT = "            if (!tc::mbar_wait(&bar_acc_full[b], bph, abort_flag)) break;"
        if g.plain and gs.tma_a:
            TMA_ROLE = f"""    if (warp == kMmaWarp + 1 && lane == 0) {{
        // ================= TMA issue (single thread): raw A tiles (and the streamed B chunks) as far ahead as the
        // ring allows; completion of a tile is signalled on bar_raw, which the producer warps wait on
        uint32_t it = 0;
        bool ok = true;
        for (int64_t t = cta; t < tiles && ok; t += nctas) {{
            for (int c = 0; c < NCHUNK; ++c, ++it) {{
                const int s = it % NSTAGE;
                const uint32_t ph = (it / NSTAGE) & 1;
                if (!tc::mbar_wait(&bar_empty[s], ph ^ 1u, abort_flag)) {{ ok = false; break; }}
                uint8_t* stage = sS + s * STAGE_BYTES;
                tc::tma_load_2d(stage, tmap, kXOff{gi}[c], static_cast<int32_t>(t * ZT), &bar_raw[s], A_TILE);
{_indent(issue_b_body('stage', '&bar_full[s]', 'c'), 16)}
            }}
        }}
    }}"""
        else:
            TMA_ROLE = ""
        funcs.append(f"""
// ---------------------------------------------------------------- group {gi}: N = {g.n}, 2l+1 = {g.dim}, K = {32 * nch}
__device__ __forceinline__ void run_group_{gi}(const float* __restrict__ x1, const float* __restrict__ x2,
        const uint8_t* __restrict__ bprep, float* __restrict__ out, int64_t Z, int cta, int nctas, uint8_t* smem,
        int* status, int pieces, const CUtensorMap* tmap, const GateEpilogue& ep) {{
    constexpr int N = {g.n}, DIM = {g.dim}, ZT = {g.zt}, NCHUNK = {nch}, NSTAGE = {g.nstage()}, NBUF = 2;
    // partial accumulators per buffer: even / odd k-steps accumulate in different TMEM columns, which halves
    // the length of each dependent MMA chain (and of the fp32 accumulation error); summed in the epilogue
    constexpr bool WIDE = {'true' if g.wide_b else 'false'};   // split mode with two MMAs per k-step (issue_chunk_wide)
    constexpr int ACCW = WIDE ? 2 * N : N;          // columns of one partial accumulator
    constexpr int NACC = {(2 if 8 * g.n <= 512 else 1) if g.wide_b else (2 if 4 * g.n <= 512 else 1)};
    static_assert(NBUF * NACC * ACCW <= 512, "accumulators exceed tensor memory");
    constexpr int OUT_OFF = {g.out_off};
    constexpr uint32_t A_TILE = {A_TILE}, B_HALF = N * 128, STAGE_BYTES = {g.stage_bytes()};
    constexpr uint32_t RESIDENT_BYTES = {g.resident_bytes()};   // > 0: the whole prepared B stays in shared memory
    constexpr uint32_t IDESC = tc::idesc_tf32_m128(N);
    constexpr uint32_t IDESC_WIDE = tc::idesc_tf32_m128(WIDE ? 2 * N : N);
    constexpr bool SWAP = {'true' if g.swap else 'false'};      // operands swapped: accumulator rows = output channels, columns = tile rows
    constexpr uint32_t IDESC_SWAP = tc::idesc_tf32_m128(128);
    // the epilogue sums `nparts` column blocks of width N: the partial accumulators, and in the two-MMA split
    // mode the two halves of each
    const int nsub = (WIDE && pieces == 2) ? 2 : 1;
    const int nparts = NACC * nsub;
    auto part_off = [&](int p) {{ return (p / nsub) * ACCW + (p % nsub) * N; }};
    uint8_t* sB = smem;
    uint8_t* sS = smem + RESIDENT_BYTES;
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(sS + NSTAGE * STAGE_BYTES);
    uint64_t* bar_empty = bar_full + NSTAGE;
    uint64_t* bar_acc_full = bar_empty + NSTAGE;
    uint64_t* bar_acc_empty = bar_acc_full + NBUF;
    uint64_t* bar_b = bar_acc_empty + NBUF;
    uint64_t* bar_raw = bar_b + 1;            // [NSTAGE] completion of the TMA copy of a stage's raw A tile
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_raw + NSTAGE);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* sY = reinterpret_cast<float*>(sS + NSTAGE * STAGE_BYTES + 1024);
    float* sE = sY + {(Y_BYTES if g.has_y else 0) // 4};   // epilogue staging (only used by staged epilogues)
    const uint8_t* bsrc = bprep + {prep_offsets[gi]};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {{
        *abort_flag = 0;
        for (int s = 0; s < NSTAGE; ++s) {{ tc::mbar_init(&bar_full[s], kProducerWarps); tc::mbar_init(&bar_empty[s], 1); }}
        for (int b = 0; b < NBUF; ++b) {{ tc::mbar_init(&bar_acc_full[b], 1); tc::mbar_init(&bar_acc_empty[b], kEpilogueWarps); }}
        tc::mbar_init(bar_b, 1);
        for (int s = 0; s < NSTAGE; ++s) tc::mbar_init(&bar_raw[s], 1);
        tc::mbar_init_fence();
    }}
    if (warp == kMmaWarp) tc::tmem_alloc(tmem_slot, kTmemCols);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const int64_t tiles = (Z + ZT - 1) / ZT;

    if (warp < kEpilogueWarps) {{
        // ================= epilogue: tensor memory -> registers -> global
        int tile_i = 0;
        const int row = warp * 32 + lane;
        const int zq = row / DIM, kq = row - zq * DIM;
        for (int64_t t = cta; t < tiles; t += nctas, ++tile_i) {{
            const int b = tile_i % NBUF;
            const uint32_t bph = (tile_i / NBUF) & 1;
{ACC_WAIT}
            tc::tc_fence_after_sync();
            const int64_t z = t * ZT + zq;
            const bool valid = zq < ZT && z < Z;
            float* orow = out + z * {dout} + OUT_OFF;
            const uint32_t tbase = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + b * (NACC * ACCW);
{EPILOGUE}
            tc::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&bar_acc_empty[b]);
        }}
    }} else if (warp < kEpilogueWarps + kProducerWarps) {{
        // ================= producers: A (hi, lo) chunks; warp 0 also fetches the prepared B chunk
        const int pw = warp - kEpilogueWarps;
        float* sy = sY + pw * {qn * max(d2, 1)};
        uint32_t it = 0;
        bool ok = true;
        if (RESIDENT_BYTES > 0 && pw == 0 && lane == 0 && cta < tiles) {{
            // the group's whole prepared B: one bulk copy per chunk, one barrier for all of them
            const uint32_t bar = tc::smem_u32(bar_b);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(RESIDENT_BYTES) : "memory");
            for (int c = 0; c < NCHUNK; ++c)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(tc::smem_u32(sB + c * {PIECES} * B_HALF)), "l"(bsrc + static_cast<size_t>(c) * {PIECES} * B_HALF),
                               "r"({PIECES} * B_HALF), "r"(bar) : "memory");
        }}
{PRODUCER_BLOCK}
    }} else if (warp == kMmaWarp && lane == 0) {{
        // ================= MMA issue (single thread)
        uint32_t it = 0;
        int tile_i = 0;
        bool ok = true;
        if (RESIDENT_BYTES > 0 && cta < tiles) ok = tc::mbar_wait(bar_b, 0, abort_flag, 2000000u);
        const uint64_t bdesc_resident = tc::smem_desc_k_sw128(tc::smem_u32(sB));
        for (int64_t t = cta; t < tiles && ok; t += nctas, ++tile_i) {{
            const int b = tile_i % NBUF;
            const uint32_t bph = (tile_i / NBUF) & 1;
            if (!tc::mbar_wait(&bar_acc_empty[b], bph ^ 1u, abort_flag)) break;
            tc::tc_fence_after_sync();
            const uint32_t d_base = tmem_base + b * (NACC * ACCW);
            for (int c = 0; c < NCHUNK; ++c, ++it) {{
                const int s = it % NSTAGE;
                const uint32_t ph = (it / NSTAGE) & 1;
                if (!tc::mbar_wait(&bar_full[s], ph, abort_flag)) {{ ok = false; break; }}
                tc::tc_fence_after_sync();
                // descriptors differ from the stage's base descriptor only in the address field (bytes >> 4):
                // everything below is compile-time offsets added to two 64-bit values, fully unrolled
                const uint64_t adesc = tc::smem_desc_k_sw128(tc::smem_u32(sS + s * STAGE_BYTES));
                const uint64_t bdesc = RESIDENT_BYTES > 0 ? bdesc_resident + static_cast<uint64_t>(c) * (({PIECES} * B_HALF) >> 4)
                                                          : adesc + (({PIECES} * A_TILE) >> 4);
                if constexpr (SWAP) {{
                    // M = 128 output channels of the weights, N = the 128 rows of the produced tile
#pragma unroll
                    for (int m = 0; m < N / 128; ++m) {{
                        const uint64_t wdesc = bdesc + static_cast<uint64_t>((m * 128 * 128) >> 4);
                        if (pieces == 1) tc::issue_chunk<1, 128, NACC, B_HALF, A_TILE, ACCW>(d_base + m * 128, wdesc, adesc, IDESC_SWAP, c > 0);
                        else if (pieces == 2) tc::issue_chunk<2, 128, NACC, B_HALF, A_TILE, ACCW>(d_base + m * 128, wdesc, adesc, IDESC_SWAP, c > 0);
                        else tc::issue_chunk<3, 128, NACC, B_HALF, A_TILE, ACCW>(d_base + m * 128, wdesc, adesc, IDESC_SWAP, c > 0);
                    }}
                }} else
                if (pieces == 1) tc::issue_chunk<1, N, NACC, A_TILE, B_HALF, ACCW>(d_base, adesc, bdesc, IDESC, c > 0);
                else if (WIDE && pieces == 2) tc::issue_chunk_wide<N, NACC, A_TILE, B_HALF>(d_base, adesc, bdesc, IDESC, IDESC_WIDE, c > 0);
                else if (pieces == 2) tc::issue_chunk<2, N, NACC, A_TILE, B_HALF, ACCW>(d_base, adesc, bdesc, IDESC, c > 0);
                else tc::issue_chunk<3, N, NACC, A_TILE, B_HALF, ACCW>(d_base, adesc, bdesc, IDESC, c > 0);
                tc::mma_commit(&bar_empty[s]);
            }}
            if (ok) tc::mma_commit(&bar_acc_full[b]);
        }}
    }}
{TMA_ROLE}
    tc::tc_fence_before_sync();
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicExch(status, 3);
    if (warp == kMmaWarp) tc::tmem_dealloc(tmem_base, kTmemCols);
}}

// weights of group {gi} -> scaled, split into tf32 (hi, lo), K-major 128-byte swizzled chunks of 32 K
__device__ __forceinline__ void prep_group_{gi}(const float* __restrict__ W, uint8_t* __restrict__ bprep, int idx) {{
    constexpr int N = {g.n}, NCHUNK = {nch};
    if (idx >= NCHUNK * 32 * N) return;
    const int c = idx / (32 * N), rem = idx - c * 32 * N;
    const int kk = rem / N, n = rem - kk * N;   // n fastest: coalesced when sn == 1
    constexpr int NBLK = {len(g.chunks[0].blocks) if g.chunks[0].blocks else 1}, BW = N / NBLK;   // column blocks with their own weight slice
    const int blk = n / BW, nn = n - blk * BW;
    const float v = kScale{gi}[c * NBLK + blk] * W[kWBase{gi}[c * NBLK + blk] + kk * kSK{gi}[c] + nn * kSN{gi}[c]];
    const float hi = tc::to_tf32(v);
    const float rest = v - hi;
    const float mid = tc::to_tf32(rest);
    uint8_t* dst = bprep + {prep_offsets[gi]} + static_cast<size_t>(c) * {PIECES} * N * 128 + tc::sw128_offset(n, kk);
    *reinterpret_cast<float*>(dst) = hi;
    *reinterpret_cast<float*>(dst + N * 128) = mid;
    {'*reinterpret_cast<float*>(dst + 2 * N * 128) = tc::to_tf32(rest - mid);' if PIECES >= 3 else ''}
}}
""")

    ng = len(gs.groups)
    dispatch = "\n".join(
        f"    {'else ' if gi else ''}if (blockIdx.x < cta_end{gi}) run_group_{gi}(x1, x2, bprep, out, Z, blockIdx.x - cta_begin{gi}, cta_end{gi} - cta_begin{gi}, smem, status, pieces, &tmap_a, ep);"
        for gi in range(ng))
    bounds = "\n".join(
        f"    const int cta_begin{gi} = {'0' if gi == 0 else f'cta_end{gi-1}'}, cta_end{gi} = cta_begin{gi} + split.n[{gi}];" for gi in range(ng))
    prep_max = max(len(g.chunks) * 32 * g.n for g in gs.groups)
    prep_dispatch = "\n".join(f"    {'else ' if gi else ''}if (blockIdx.y == {gi}) prep_group_{gi}(W, bprep, idx);" for gi in range(ng))
    zero_fill = "\n".join(
        f"    {{ cudaError_t e = cudaMemset2DAsync(out + {off}, {dout} * sizeof(float), 0, {n} * sizeof(float), Z, s); "
        f"if (e != cudaSuccess) return e3b_layout_fail(-2, \"tc_gemm: zero fill: %s\", cudaGetErrorString(e)); }}"
        for off, n in gs.zero_ranges)
    return f"""// Generated by e3nn_b200/codegen/tc_gemm.py -- do not edit.
// {gs.title}, key {gs.key}
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstring>
#include "layout_common.cuh"
#include "tc_common.cuh"

namespace {{

constexpr int kEpilogueWarps = 4;
constexpr int kProducerWarps = {PRODUCER_WARPS};
constexpr int kMmaWarp = kEpilogueWarps + kProducerWarps;
constexpr int kThreads = (kMmaWarp + 1 + {1 if gs.tma_a else 0}) * 32;   // + the TMA warp of dense-layer modules
constexpr int kTmemCols = 512;
constexpr int kGroups = {ng};
constexpr int kSmemBytes = {smem_max};
constexpr long long kPrepBytes = {prep_off};

struct CtaSplit {{ int n[kGroups]; }};

// Gate applied in the epilogue (a Linear followed by Gate, e3nn/nn/_gate.py:127-144).  tbl[4 c ..] = {{kind,
// destination column, activation, gate slot}} and cst[c] per column c of the Linear's output row: kind 0 scalar:
// final[z, dst] = cst * act(v); kind 2 gate: gates[z, slot] = cst * act(v); kind 1 gated component k of a channel
// whose component 0 is column c: final[z, dst + k] = v * gates[z, slot]; kind 3: unused.  tbl == nullptr: plain store.
struct GateEpilogue {{
    const int32_t* tbl;
    const float* cst;
    float* gates;
    float* final_out;
    int n_slots, dout_final;
}};

{chr(10).join(consts)}
{''.join(funcs)}

__global__ void __launch_bounds__(kThreads, 1) tc_gemm_kernel(const float* __restrict__ x1, const float* __restrict__ x2,
        const uint8_t* __restrict__ bprep, float* __restrict__ out, int64_t Z, CtaSplit split, int* status, int pieces,
        const __grid_constant__ CUtensorMap tmap_a, const GateEpilogue ep) {{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
{bounds}
{dispatch}
}}

__global__ void tc_gemm_prep_kernel(const float* __restrict__ W, uint8_t* __restrict__ bprep) {{
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
{prep_dispatch}
}}

}}  // namespace

extern "C" int e3b_layout_info(int32_t* dims) {{
    dims[0] = {d1}; dims[1] = {d2}; dims[2] = {dout}; dims[3] = 0; dims[4] = -1; dims[5] = kThreads;
    return 0;
}}
extern "C" const char* e3b_layout_key(void) {{ return "{gs.key}"; }}
extern "C" const char* e3b_layout_last_error(void) {{ return e3b_layout_error_buffer(); }}
extern "C" long long e3b_tc_gemm_scratch_bytes(void) {{ return kPrepBytes; }}

static const int kGroupWork[kGroups] = {{{', '.join(str(g.work()) for g in gs.groups)}}};
static const int kGroupDim[kGroups] = {{{', '.join(str(g.dim) for g in gs.groups)}}};   // 2l+1 of each output group

static int tc_gemm_launch(const float* x1, const float* x2, const float* weight, float* out, int64_t Z, int precision,
                          void* scratch, const int* cta_split, int32_t* status, cudaStream_t s, const GateEpilogue& ep,
                          int pass /* 0: every group; 1: groups of scalars only; 2: the other groups */, bool prepare) {{
    CtaSplit split;
    int used = 0;
    bool any = false;
    for (int g = 0; g < kGroups; ++g) any = any || pass == 0 || (pass == 1) == (kGroupDim[g] == 1);
    if (!any) return 0;
    if (cta_split) {{
        for (int g = 0; g < kGroups; ++g) {{ split.n[g] = cta_split[g] < 1 ? 1 : cta_split[g]; used += split.n[g]; }}
    }} else {{
        const int num_ctas = 148 < kGroups ? kGroups : 148;
        long total = 0;
        for (int g = 0; g < kGroups; ++g) {{
            const bool on = pass == 0 || (pass == 1) == (kGroupDim[g] == 1);
            total += on ? kGroupWork[g] : 0;
        }}
        int on_groups = 0;
        for (int g = 0; g < kGroups; ++g) {{
            const bool on = pass == 0 || (pass == 1) == (kGroupDim[g] == 1);
            int n = on ? static_cast<int>((static_cast<long>(num_ctas) * kGroupWork[g]) / total) : 0;
            if (on && n < 1) n = 1;
            split.n[g] = n;
            used += n;
            on_groups += on ? 1 : 0;
        }}
        for (int g = kGroups - 1; used < num_ctas; g = (g + kGroups - 1) % kGroups)
            if (split.n[g] > 0) {{ split.n[g]++; used++; }}
        while (used > num_ctas && used > on_groups) {{
            int big = 0;
            for (int g = 1; g < kGroups; ++g) if (split.n[g] > split.n[big]) big = g;
            split.n[big]--; used--;
        }}
    }}
    if (prepare)
        tc_gemm_prep_kernel<<<dim3(({prep_max} + 255) / 256, kGroups), 256, 0, s>>>(weight, static_cast<uint8_t*>(scratch));
    cudaError_t err = cudaFuncSetAttribute(tc_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (err != cudaSuccess) return e3b_layout_fail(-2, "tc_gemm: smem attribute: %s", cudaGetErrorString(err));
    CUtensorMap tmap;
    std::memset(&tmap, 0, sizeof(tmap));
    if ({'true' if gs.tma_a else 'false'}) {{
        // x1 as a [Z, {d1}] fp32 matrix, boxes of 128 rows x 32 columns, 128-byte swizzle: the layout the MMA reads
        const int rc = tc::encode_tensor_map_2d(&tmap, x1, {d1}, Z, 32, 128);
        if (rc != 0) return e3b_layout_fail(-2, "tc_gemm: cuTensorMapEncodeTiled failed (%d)", rc);
    }}
    tc_gemm_kernel<<<used, kThreads, kSmemBytes, s>>>(x1, x2, static_cast<const uint8_t*>(scratch), out, Z, split, status,
                                                       precision, tmap, ep);
    return e3b_layout_check("tc_gemm");
}}

static int tc_gemm_check_args(const float* x1, const float* x2, const float* weight, const float* out, int64_t Z,
                              int precision, const void* scratch, const int32_t* status) {{
    if (Z < 0) return e3b_layout_fail(-1, "tc_gemm: negative row count");
    if (!x1 || !weight || !out || !status || !scratch || ({d2} > 0 && !x2)) return e3b_layout_fail(-1, "tc_gemm: null pointer");
    if (reinterpret_cast<uintptr_t>(out) % 16 != 0 || reinterpret_cast<uintptr_t>(scratch) % 16 != 0)
        return e3b_layout_fail(-1, "tc_gemm: out and scratch must be 16-byte aligned");
    if (precision < 1 || precision > {PIECES}) return e3b_layout_fail(-1, "tc_gemm: precision must be between 1 and {PIECES}");
    if ({'true' if any(g.plain for g in gs.groups) else 'false'} && reinterpret_cast<uintptr_t>(x1) % 16 != 0)
        return e3b_layout_fail(-1, "tc_gemm: x1 must be 16-byte aligned");
    return 0;
}}

// precision = number of tf32 pieces per operand: 1 = plain tf32 (1 MMA per step, ~1e-3 relative),
// 2 = hi/lo split (3 MMAs, 22-bit operands, ~2e-5 x RMS); 3 (hi/mid/lo, 6 MMAs) only if the module was
// generated with room for three pieces.
// scratch: e3b_tc_gemm_scratch_bytes() bytes of device memory, 16-byte aligned (prepared weights).
// cta_split: optional host array of kGroups CTA counts (NULL: proportional to the estimated work).
extern "C" int e3b_tc_gemm_fwd(const float* x1, const float* x2, const float* weight, float* out, int64_t Z,
                               int precision, void* scratch, const int* cta_split, int32_t* status, void* stream) {{
    if (Z == 0) return 0;
    if (int rc = tc_gemm_check_args(x1, x2, weight, out, Z, precision, scratch, status)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
{zero_fill}
    const GateEpilogue none{{nullptr, nullptr, nullptr, nullptr, 0, 0}};
    return tc_gemm_launch(x1, x2, weight, out, Z, precision, scratch, cta_split, status, s, none, 0, true);
}}

// The same contraction with Gate as its epilogue (only meaningful for a Linear whose output row is a Gate's input
// row): gate_table [dout, 4] int32 and gate_const [dout] describe the columns of that row as in GateEpilogue above,
// gates [Z, n_slots] receives the activated gate scalars, out [Z, dout_final] the Gate's output row; the row of
// {dout} columns itself is never written.  Two launches on `stream`: the scalar irreps (plain scalars and gates),
// then the gated irreps, which read the gates of their rows.
extern "C" int e3b_tc_gemm_fwd_gate(const float* x1, const float* weight, const int32_t* gate_table, const float* gate_const,
                                    float* gates, int n_slots, float* out, int dout_final, int64_t Z, int precision,
                                    void* scratch, int32_t* status, void* stream) {{
    if (Z == 0) return 0;
    if ({d2} > 0) return e3b_layout_fail(-3, "tc_gemm_fwd_gate: only layouts without a second operand (Linear)");
    if ({'true' if any(g.swap for g in gs.groups) else 'false'}) return e3b_layout_fail(-3, "tc_gemm_fwd_gate: this module has groups with swapped operands, which have no gate epilogue");
    if (int rc = tc_gemm_check_args(x1, nullptr, weight, out, Z, precision, scratch, status)) return rc;
    if (!gate_table || !gate_const || (n_slots > 0 && !gates) || n_slots < 0 || dout_final <= 0)
        return e3b_layout_fail(-1, "tc_gemm_fwd_gate: bad gate arguments");
    if (reinterpret_cast<uintptr_t>(gate_table) % 16 != 0) return e3b_layout_fail(-1, "tc_gemm_fwd_gate: gate_table must be 16-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const GateEpilogue ep{{gate_table, gate_const, gates, out, n_slots, dout_final}};
    if (int rc = tc_gemm_launch(x1, nullptr, weight, out, Z, precision, scratch, nullptr, status, s, ep, 1, true)) return rc;
    return tc_gemm_launch(x1, nullptr, weight, out, Z, precision, scratch, nullptr, status, s, ep, 2, false);
}}
"""
