"""Layout specifications: the compile-time description a kernel is generated from.

A ``TPSpec`` is the normalised form of a tensor product: the three irreps layouts and
the instruction list with the final per-path coefficient, computed exactly as
``e3nn/o3/_tensor_product/_tensor_product.py:236-324`` does.  A ``LinearSpec`` is the
same for ``e3nn/o3/_linear.py:133-187``.  Both are pure host-side metadata.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass
from math import prod, sqrt
from typing import List, NamedTuple, Optional, Sequence, Tuple

from ._irreps import Irreps

ALL_MODES = ("uvw", "uvu", "uvv", "uuw", "uuu", "uvuv", "uvu<v", "u<vw")
SUPPORTED_MODES = ALL_MODES


class Instruction(NamedTuple):
    """Same fields as ``e3nn/o3/_tensor_product/_instruction.py:4-11``."""

    i_in1: int
    i_in2: int
    i_out: int
    connection_mode: str
    has_weight: bool
    path_weight: float
    path_shape: tuple


class LinearInstruction(NamedTuple):
    """Same fields as ``e3nn/o3/_linear.py:14-18``; ``i_in == -1`` marks a bias."""

    i_in: int
    i_out: int
    path_shape: tuple
    path_weight: float


def _path_shape(mode: str, m1: int, m2: int, mo: int) -> tuple:
    return {
        "uvw": (m1, m2, mo),
        "uvu": (m1, m2),
        "uvv": (m1, m2),
        "uuw": (m1, mo),
        "uuu": (m1,),
        "uvuv": (m1, m2),
        "uvu<v": (m1 * (m2 - 1) // 2,),
        "u<vw": (m1 * (m2 - 1) // 2, mo),
    }[mode]


def _num_elements(mode: str, m1: int, m2: int) -> int:
    return {
        "uvw": m1 * m2,
        "uvu": m2,
        "uvv": m1,
        "uuw": m1,
        "uuu": 1,
        "uvuv": 1,
        "uvu<v": 1,
        "u<vw": m1 * (m2 - 1) // 2,
    }[mode]


def normalize_tp_instructions(
    irreps_in1: Irreps,
    irreps_in2: Irreps,
    irreps_out: Irreps,
    instructions: Sequence[tuple],
    in1_var: Optional[Sequence[float]] = None,
    in2_var: Optional[Sequence[float]] = None,
    out_var: Optional[Sequence[float]] = None,
    irrep_normalization: str = "component",
    path_normalization: str = "element",
) -> List[Instruction]:
    """Instruction tuples ``(i1, i2, iout, mode, has_weight[, path_weight])`` -> `Instruction`
    with ``path_weight`` replaced by the final coefficient ``sqrt(alpha)``."""
    assert irrep_normalization in ["component", "norm", "none"]
    assert path_normalization in ["element", "path", "none"]
    raw = [tuple(x) if len(x) == 6 else tuple(x) + (1.0,) for x in instructions]
    raw = [
        Instruction(
            i1, i2, io, mode, hw, pw,
            _path_shape(mode, irreps_in1[i1].mul, irreps_in2[i2].mul, irreps_out[io].mul),
        )
        for (i1, i2, io, mode, hw, pw) in raw
    ]
    in1_var = [1.0] * len(irreps_in1) if in1_var is None else [float(v) for v in in1_var]
    in2_var = [1.0] * len(irreps_in2) if in2_var is None else [float(v) for v in in2_var]
    out_var = [1.0] * len(irreps_out) if out_var is None else [float(v) for v in out_var]
    assert len(in1_var) == len(irreps_in1), "Len of ir1_var must be equal to len(irreps_in1)"
    assert len(in2_var) == len(irreps_in2), "Len of ir2_var must be equal to len(irreps_in2)"
    assert len(out_var) == len(irreps_out), "Len of out_var must be equal to len(irreps_out)"

    def nel(ins: Instruction) -> int:
        return _num_elements(ins.connection_mode, irreps_in1[ins.i_in1].mul, irreps_in2[ins.i_in2].mul)

    out: List[Instruction] = []
    for ins in raw:
        a, b, c = irreps_in1[ins.i_in1], irreps_in2[ins.i_in2], irreps_out[ins.i_out]
        assert a.ir.p * b.ir.p == c.ir.p
        assert abs(a.ir.l - b.ir.l) <= c.ir.l <= a.ir.l + b.ir.l
        assert ins.connection_mode in ALL_MODES
        if irrep_normalization == "component":
            alpha = c.ir.dim
        elif irrep_normalization == "norm":
            alpha = a.ir.dim * b.ir.dim
        else:
            alpha = 1
        if path_normalization == "element":
            x = sum(in1_var[i.i_in1] * in2_var[i.i_in2] * nel(i) for i in raw if i.i_out == ins.i_out)
        elif path_normalization == "path":
            x = in1_var[ins.i_in1] * in2_var[ins.i_in2] * nel(ins)
            x *= len([i for i in raw if i.i_out == ins.i_out])
        else:
            x = 1
        if x > 0.0:
            alpha /= x
        alpha *= out_var[ins.i_out]
        alpha *= ins.path_weight
        out.append(ins._replace(path_weight=sqrt(alpha)))
    return out


@dataclass(frozen=True)
class TPSpec:
    irreps_in1: Irreps
    irreps_in2: Irreps
    irreps_out: Irreps
    instructions: Tuple[Instruction, ...]
    shared_weights: bool

    @property
    def weight_numel(self) -> int:
        return sum(prod(i.path_shape) for i in self.instructions if i.has_weight)

    def weight_offsets(self) -> List[int]:
        """Start of every instruction's block in the flat weight vector (-1: no weight)."""
        out, off = [], 0
        for ins in self.instructions:
            if ins.has_weight:
                out.append(off)
                off += prod(ins.path_shape)
            else:
                out.append(-1)
        return out

    def modes(self) -> set:
        return {i.connection_mode for i in self.instructions}

    def live_instructions(self) -> List[Tuple[int, Instruction]]:
        """Instructions that contribute (no zero-dim operand), with their index."""
        out = []
        for n, ins in enumerate(self.instructions):
            if (
                self.irreps_in1[ins.i_in1].dim == 0
                or self.irreps_in2[ins.i_in2].dim == 0
                or self.irreps_out[ins.i_out].dim == 0
            ):
                continue
            out.append((n, ins))
        return out

    def key(self) -> str:
        """Stable hash of everything a generated kernel depends on (computed once: the spec is immutable after
        construction and the key is looked up on every forward call)."""
        cached = self.__dict__.get("_key")
        if cached is not None:
            return cached
        blob = json.dumps(
            {
                "in1": str(self.irreps_in1),
                "in2": str(self.irreps_in2),
                "out": str(self.irreps_out),
                "ins": [
                    [i.i_in1, i.i_in2, i.i_out, i.connection_mode, bool(i.has_weight), repr(float(i.path_weight))]
                    for i in self.instructions
                ],
                "shared": bool(self.shared_weights),
            },
            sort_keys=True,
        )
        self.__dict__["_key"] = hashlib.sha1(blob.encode()).hexdigest()[:16]
        return self.__dict__["_key"]


def normalize_linear_instructions(
    irreps_in: Irreps,
    irreps_out: Irreps,
    instructions: Optional[Sequence[Tuple[int, int]]],
    biases,
    f_in: Optional[int] = None,
    path_normalization: str = "element",
) -> List[LinearInstruction]:
    assert path_normalization in ["element", "path"]
    if instructions is None:
        instructions = [
            (i_in, i_out)
            for i_in, (_, ir_in) in enumerate(irreps_in)
            for i_out, (_, ir_out) in enumerate(irreps_out)
            if ir_in == ir_out
        ]
    raw = [LinearInstruction(i, o, (irreps_in[i].mul, irreps_out[o].mul), 1.0) for i, o in instructions]

    def fan(ins: LinearInstruction) -> float:
        x = sum(
            irreps_in[i.i_in if path_normalization == "element" else ins.i_in].mul
            for i in raw
            if i.i_out == ins.i_out
        )
        if f_in is not None:
            x *= f_in
        return 1.0 if x == 0 else x

    out = [ins._replace(path_weight=fan(ins) ** (-0.5)) for ins in raw]
    for ins in out:
        if not ins.i_in < len(irreps_in):
            raise IndexError(f"{ins.i_in} is not a valid index for irreps_in")
        if not ins.i_out < len(irreps_out):
            raise IndexError(f"{ins.i_out} is not a valid index for irreps_out")
        if not (ins.i_in == -1 or irreps_in[ins.i_in].ir == irreps_out[ins.i_out].ir):
            raise ValueError(f"{ins.i_in} and {ins.i_out} do not have the same irrep")
    if biases is None:
        biases = len(irreps_out) * (False,)
    if isinstance(biases, bool):
        biases = [biases and ir.is_scalar() for _, ir in irreps_out]
    assert len(biases) == len(irreps_out)
    assert all(ir.is_scalar() or (not b) for b, (_, ir) in zip(biases, irreps_out))
    out += [
        LinearInstruction(-1, i_out, (mul_ir.dim,), 1.0)
        for i_out, (bias, mul_ir) in enumerate(zip(biases, irreps_out))
        if bias
    ]
    return out
