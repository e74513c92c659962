"""Scalar activation on rows of irreps features, with the reference's constructor and attributes
(``e3nn/nn/_activation.py:9-111``).

``Activation(irreps_in, acts)``: block ``b`` of ``irreps_in`` is passed through ``acts[b]`` rescaled to unit second
moment (``e3nn/math/_normalize_activation.py:9-57``), or copied when ``acts[b]`` is ``None``; an activation on a
non-scalar block is an error, an odd scalar takes the parity of its activation (``_activation.py:39-57``).  The
reference narrows, applies and concatenates block by block; here the row is read once and written once by the
same elementwise kernels that serve ``Gate`` (``e3b_gate_fwd`` / ``e3b_gate_bwd`` with no gated columns).
"""
from __future__ import annotations

import torch

from .. import _lib
from ..o3 import Irreps
from ._fc import normalize2mom_constant
from ._gate import _ACT_CODE, _GateFunction, _act_name, _activation_irreps


class Activation(torch.nn.Module):
    def __init__(self, irreps_in, acts) -> None:
        super().__init__()
        irreps_in = Irreps(irreps_in)
        if len(irreps_in) != len(acts):
            raise ValueError(f"Irreps in and number of activation functions does not match: {len(acts), (irreps_in, acts)}")
        names = [_act_name(a) for a in acts]
        self.irreps_in = irreps_in
        self.irreps_out = _activation_irreps(irreps_in, names)
        self.acts = list(acts)
        out_tbl, out_cst, in_tbl, in_cst = [], [], [], []
        col = 0
        for (mul, ir), name in zip(irreps_in, names):
            cst = normalize2mom_constant(name) if name is not None else 1.0
            for _ in range(mul * ir.dim):
                out_tbl.append([col, -1, _ACT_CODE[name]])
                out_cst.append(cst)
                in_tbl.append([0, col, 1, 0, _ACT_CODE[name]])
                in_cst.append(cst)
                col += 1
        self.register_buffer("_out_tbl", torch.tensor(out_tbl, dtype=torch.int32).reshape(-1, 3), persistent=False)
        self.register_buffer("_out_cst", torch.tensor(out_cst, dtype=torch.float32), persistent=False)
        self.register_buffer("_in_tbl", torch.tensor(in_tbl, dtype=torch.int32).reshape(-1, 5), persistent=False)
        self.register_buffer("_in_cst", torch.tensor(in_cst, dtype=torch.float32), persistent=False)

    def __repr__(self) -> str:
        acts = "".join(["x" if a is not None else " " for a in self.acts])
        return f"{self.__class__.__name__} [{acts}] ({self.irreps_in} -> {self.irreps_out})"

    def forward(self, features: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if not features.is_cuda:
            raise NotImplementedError("Activation runs on CUDA tensors only")
        if dim not in (-1, features.dim() - 1):
            raise NotImplementedError("Activation acts on the last dimension")
        torch._assert(features.shape[-1] == self.irreps_in.dim, "Incorrect last dimension for features")
        if self.irreps_in.dim == 0:
            return torch.zeros_like(features)
        lead = features.shape[:-1]
        x = features.reshape(-1, self.irreps_in.dim).to(torch.float32).contiguous()
        for name in ("_out_tbl", "_in_tbl"):
            _lib.require_operand(getattr(self, name), x, f"Activation.{name} (move the module with .to(device))", None, torch.int32)
        if x.shape[0] == 0:
            return features.new_zeros(*lead, self.irreps_out.dim)
        out = _GateFunction.apply(x, self._out_tbl, self._out_cst, self._in_tbl, self._in_cst, self.irreps_out.dim)
        return out.reshape(*lead, self.irreps_out.dim)
