"""``Gate`` applied as the epilogue of the ``Linear`` that feeds it.

Every model of the reference runs ``Linear`` -> ``Gate`` back to back (``e3nn/nn/models/gate_points_2101.py:275-293``):
the Linear writes a ``[rows, gate.irreps_in.dim]`` row which the Gate reads again at once.  ``LinearGate(lin, gate)``
evaluates the pair with ``e3b_tc_gemm_fwd_gate`` (tensor-core Linear, ``math_mode='tf32x3' | 'tf32'``) or
``e3b_dense_fwd_gate`` (fp32 Linear): the gate is applied where the Linear's result is still in registers, the
scalar irreps (plain scalars and gates) first, the gated irreps after them; only the activated gate scalars make a
round trip through memory.  The result equals ``gate(lin(x))``.

The fused kernels are forward passes.  When a gradient is required (the Gate's gradient needs the Linear's output
row), with biases, or for Linear outputs no path writes, the two modules run one after the other.

``fuse``: ``True`` runs the fused kernels whenever they apply, ``False`` never, ``"auto"`` (default) only where they
are the faster choice.  Today that is nowhere: the fused pair moves 46 % fewer bytes, but both Linear kernels are
bound by their epilogues (strided 4-byte stores of the 2l+1 > 1 irreps; the fp32 kernel by its arithmetic), the
gate adds loads to exactly that part, and the scalar irreps must run as a launch of their own before the gated
ones: 7.7 ms fused against 4.1 + 2.0 ms on 1,048,576 rows of ``64x0e+64x1o+64x2e+64x3o`` (tensor cores), 28.9 against
24.5 + 2.0 ms (fp32).
"""
from __future__ import annotations

import torch

from .. import _lib
from ..o3._linear import Linear
from ._gate import Gate


class LinearGate(torch.nn.Module):
    def __init__(self, lin: Linear, gate: Gate, fuse="auto") -> None:
        super().__init__()
        if fuse not in (True, False, "auto"):
            raise ValueError('fuse must be True, False or "auto"')
        self.fuse = fuse
        if lin.irreps_out.simplify() != gate.irreps_in.simplify() or lin.irreps_out.dim != gate.irreps_in.dim:
            raise ValueError(f"lin.irreps_out = {lin.irreps_out} does not match gate.irreps_in = {gate.irreps_in}")
        self.lin, self.gate = lin, gate
        self.irreps_in, self.irreps_out = lin.irreps_in, gate.irreps_out
        in_tbl = gate._in_tbl.reshape(-1, 5).tolist()
        slot_of, n_slots = {}, 0
        for c, (kind, _, _, _, _) in enumerate(in_tbl):
            if kind == 2:
                slot_of[c] = n_slots
                n_slots += 1
        tbl = []
        for c, (kind, first_out, _, partner, act) in enumerate(in_tbl):
            if kind == 0:
                tbl.append([0, first_out, act, 0])
            elif kind == 1:
                tbl.append([1, first_out, act, slot_of[partner]])
            elif kind == 2:
                tbl.append([2, 0, act, slot_of[c]])
            else:
                tbl.append([3, 0, 3, 0])
        self.n_slots = n_slots
        self.register_buffer("_fuse_tbl", torch.tensor(tbl, dtype=torch.int32).reshape(-1, 4), persistent=False)
        self.register_buffer("_fuse_cst", gate._in_cst.detach().clone().float(), persistent=False)

    def fusable(self, features: torch.Tensor) -> bool:
        lin = self.lin
        needs_grad = torch.is_grad_enabled() and (features.requires_grad or any(p.requires_grad for p in lin.parameters()))
        return (not needs_grad and lin.internal_weights and lin.bias_numel == 0 and not lin._unwritten
                and lin.weight_numel > 0 and features.dtype == torch.float32
                and (lin._precision == 0 or lin._tc_fwd is not None))

    def forward(self, features: torch.Tensor) -> torch.Tensor:
        if not features.is_cuda:
            raise NotImplementedError("LinearGate runs on CUDA tensors only")
        if self.fuse is not True or not self.fusable(features):
            return self.gate(self.lin(features))
        lin = self.lin
        torch._assert(features.shape[-1] == lin.irreps_in.dim, "Incorrect last dimension for features")
        lead = features.shape[:-1]
        x = features.reshape(-1, lin.irreps_in.dim).contiguous()
        rows, dev = x.shape[0], x.device
        if rows == 0:
            return features.new_zeros(*lead, self.irreps_out.dim)
        _lib.require_operand(lin.weight, x, "weight", lin.weight_numel)
        _lib.require_operand(self._fuse_tbl, x, "LinearGate tables (move the module with .to(device))", None, torch.int32)
        _lib.poll_status(dev)
        out = torch.empty(rows, self.irreps_out.dim, dtype=torch.float32, device=dev)
        gates = torch.empty(rows, max(self.n_slots, 1), dtype=torch.float32, device=dev)
        if lin._precision > 0:
            _lib.tc_gemm_module(lin._tc_fwd).run_gate(x, lin.weight.detach().reshape(-1).contiguous(), self._fuse_tbl,
                                                      self._fuse_cst, gates, out, lin._precision)
            return out.reshape(*lead, self.irreps_out.dim)
        with torch.cuda.device(dev), _lib.nvtx_range("e3b_dense_fwd_gate"):
            rc = _lib.core().e3b_dense_fwd_gate(lin._plan_host.ctypes.data, _lib._ptr(lin._plan_on(dev, False)), _lib._ptr(x),
                                                _lib._ptr(lin.weight.detach().reshape(-1).contiguous()), _lib._ptr(self._fuse_tbl),
                                                _lib._ptr(self._fuse_cst), _lib._ptr(gates), self.n_slots, _lib._ptr(out),
                                                self.irreps_out.dim, rows, _lib.stream_ptr())
        _lib.check(rc, "e3b_dense_fwd_gate")
        return out.reshape(*lead, self.irreps_out.dim)

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}({self.lin.irreps_in} -> {self.gate.irreps_in} -> {self.irreps_out})"
