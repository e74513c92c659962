"""Host-side construction of "dense plans" for ``e3b_dense_fwd`` (layout in csrc/dense.cu).

A plan lists, per output irrep, the (path, u, v) triples that are contracted against the
shared weights, and for every path the Clebsch-Gordan non-zeros (with the path coefficient
folded in) that turn a pair of input rows into the left operand of that contraction.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np

from ._irreps import Irreps
from ._wigner import wigner_3j_numpy

MAGIC = 0x65336250


def _f2i(v: float) -> int:
    return int(np.float32(v).view(np.int32))


class _Builder:
    def __init__(self, d1: int, d2: int, dout: int):
        self.d1, self.d2, self.dout = d1, d2, dout
        self.groups: List[List[int]] = []
        self.kent: List[int] = []
        self.paths: List[List[Tuple[int, int]]] = []   # per path, per k: (cg_start, cg_count)
        self.cg: List[int] = []
        self.max_k = 0

    def add_path(self, per_k: Sequence[Sequence[Tuple[int, int, float]]]) -> int:
        entry = []
        for triples in per_k:
            start = len(self.cg) // 3
            for i, j, c in triples:
                self.cg += [i, j, _f2i(c)]
            entry.append((start, len(triples)))
        self.paths.append(entry)
        return len(self.paths) - 1

    def add_group(self, out_off: int, mul_out: int, dim3: int, kents: Sequence[Tuple[int, int, int, int]], w_stride: int = 1):
        start = len(self.kent) // 4
        for k in kents:
            self.kent += list(k)
        self.groups.append([out_off, mul_out, dim3, len(kents), start, w_stride])
        self.max_k = max(self.max_k, len(kents))

    def finish(self) -> np.ndarray:
        header = 12
        off_groups = header
        off_kent = off_groups + 6 * len(self.groups)
        off_pathk = off_kent + len(self.kent)
        n_paths = len(self.paths)
        pathk_words: List[int] = []
        dir_words = []
        base = off_pathk + n_paths
        for entry in self.paths:
            dir_words.append(base + len(pathk_words))
            for s, c in entry:
                pathk_words += [s, c]
        off_cg = base + len(pathk_words)
        total = off_cg + len(self.cg)
        words = [MAGIC, self.d1, self.d2, self.dout, len(self.groups), n_paths, total,
                 off_groups, off_kent, off_pathk, off_cg, self.max_k]
        for g in self.groups:
            words += g
        words += self.kent + dir_words + pathk_words + self.cg
        assert len(words) == total
        return np.asarray(words, dtype=np.int64).astype(np.int32)


def uvw_plan(spec, instruction_ids: Optional[Sequence[int]] = None) -> Tuple[np.ndarray, List[int]]:
    """Plan of the 'uvw' paths of a `TPSpec`.  Returns (plan words, output irreps written)."""
    i1, i2, io = spec.irreps_in1, spec.irreps_in2, spec.irreps_out
    o1, o2, oo = i1.offsets(), i2.offsets(), io.offsets()
    woffs = spec.weight_offsets()
    b = _Builder(i1.dim, i2.dim, io.dim)
    live = [(n, ins) for n, ins in spec.live_instructions() if ins.connection_mode == "uvw"]
    if instruction_ids is not None:
        live = [(n, ins) for n, ins in live if n in set(instruction_ids)]
    written = sorted({ins.i_out for _, ins in live})
    for out_idx in written:
        kents = []
        mul_out, ir_out = io[out_idx]
        for n, ins in live:
            if ins.i_out != out_idx:
                continue
            (m1, ir1), (m2, ir2) = i1[ins.i_in1], i2[ins.i_in2]
            c = wigner_3j_numpy(ir1.l, ir2.l, ir_out.l) * ins.path_weight
            per_k = []
            for k in range(ir_out.dim):
                per_k.append([(i, j, float(c[i, j, k])) for i in range(ir1.dim) for j in range(ir2.dim) if c[i, j, k] != 0.0])
            pid = b.add_path(per_k)
            for u in range(m1):
                for v in range(m2):
                    kents.append((pid, o1[ins.i_in1] + u * ir1.dim, o2[ins.i_in2] + v * ir2.dim,
                                  woffs[n] + (u * m2 + v) * mul_out))
        b.add_group(oo[out_idx], mul_out, ir_out.dim, kents, 1)
    return b.finish(), written


def linear_plan(irreps_in: Irreps, irreps_out: Irreps, instructions, transpose: bool = False) -> Tuple[np.ndarray, List[int]]:
    """Plan of a Linear (weight instructions only).  ``transpose``: the map from output
    cotangents back to input cotangents (same weights, read with a stride); a transposed plan may hold
    several groups for one target and must be run with ``accumulate`` on zeroed rows."""
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
    b = _Builder(src.dim, 0, dst.dim)
    live = [(n, ins) for n, ins in enumerate(instructions) if ins.i_in != -1 and 0 not in ins.path_shape
            and irreps_in[ins.i_in].dim > 0 and irreps_out[ins.i_out].dim > 0]
    targets = sorted({(ins.i_in if transpose else ins.i_out) for _, ins in live})
    for t in targets:
        mul_t, ir = dst[t]
        # a group reads W with one stride: forward 1; transposed the output multiplicity of the path, so the
        # paths out of one input irrep are grouped by it (the caller accumulates the groups of a target)
        by_stride = {}
        for n, ins in live:
            if (ins.i_in if transpose else ins.i_out) != t:
                continue
            s = ins.i_out if transpose else ins.i_in
            mul_s = src[s].mul
            pid = b.add_path([[(k, 0, float(ins.path_weight))] for k in range(ir.dim)])
            mul_in, mul_out = ins.path_shape
            kents = by_stride.setdefault(mul_out if transpose else 1, [])
            for q in range(mul_s):
                # forward: W[u=q, w] contiguous in w; transpose: W[u, w=q] strided by mul_out in u
                wbase = offs[n] + (q if transpose else q * mul_out)
                kents.append((pid, so[s] + q * ir.dim, -1, wbase))
        for stride, kents in by_stride.items():
            b.add_group(do[t], mul_t, ir.dim, kents, stride)
    return b.finish(), targets
