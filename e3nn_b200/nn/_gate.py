"""Gate non-linearity with the reference's constructor and attributes (``e3nn/nn/_gate.py:35-144``).

``Gate(irreps_scalars, act_scalars, irreps_gates, act_gates, irreps_gated)``: the input rows are laid out
as ``irreps_in`` = the sorted, simplified sum of the three irreps (``_Sortcut``, ``_gate.py:12-32``); scalars
go through their activations rescaled to unit second moment (``e3nn/nn/_activation.py:34``,
``e3nn/math/_normalize_activation.py:9-57``), every gated channel is multiplied by its activated gate (the
``ElementwiseTensorProduct`` of ``_gate.py:116`` reduces to that for scalar gates), the output is
``act(scalars) + gated``.  Odd scalars take the parity of their activation (``_activation.py:39-57``).
One elementwise kernel per direction (``e3b_gate_fwd`` / ``e3b_gate_bwd``) driven by host-built tables.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch

from .. import _lib
from ..o3 import Irreps
from ._fc import normalize2mom_constant

_ACT_CODE = {"silu": 0, "tanh": 1, "relu": 2, None: 3, "sigmoid": 4, "abs": 5}
_ACT_PARITY = {"silu": 0, "tanh": -1, "relu": 0, "sigmoid": 0, "abs": 1}     # parity of the function itself


def _act_name(act: Optional[Callable]) -> Optional[str]:
    if act is None:
        return None
    name = getattr(act, "__name__", None)
    if name not in _ACT_CODE:
        raise NotImplementedError(f"Gate supports silu, tanh, relu, sigmoid and abs activations, got {act!r}")
    return name


def _activation_irreps(irreps: Irreps, acts: Sequence[Optional[str]]) -> Irreps:
    """Output irreps of ``Activation(irreps, acts)`` (``e3nn/nn/_activation.py:36-60``)."""
    if len(irreps) != len(acts):
        raise ValueError(f"Irreps in and number of activation functions does not match: {len(acts), (irreps, acts)}")
    out = []
    for (mul, ir), act in zip(irreps, acts):
        if act is None:
            out.append((mul, ir))
            continue
        if ir.l != 0:
            raise ValueError("Activation: cannot apply an activation function to a non-scalar input.")
        p_out = _ACT_PARITY[act] if ir.p == -1 else ir.p
        if p_out == 0:
            raise ValueError("Activation: the parity is violated! The input scalar is odd but the activation is neither "
                             "even nor odd.")
        out.append((mul, (0, p_out)))
    return Irreps(out)


def channel_tables(out_tbl: torch.Tensor, out_cst: torch.Tensor):
    """Per-channel form of the per-output-column table: runs of output columns that read consecutive input columns
    and share one gate column become one entry {first input column, count, gate column, activation, first output
    column}; scalars are runs of one.  Returns ``(int32 [n, 5], float32 [n])`` host tensors."""
    rows, csts = [], []
    tbl, cst = out_tbl.reshape(-1, 3).tolist(), out_cst.tolist()
    j = 0
    while j < len(tbl):
        src, gate, act = tbl[j]
        n = 1
        if gate >= 0:
            while j + n < len(tbl) and tbl[j + n][1] == gate and tbl[j + n][0] == src + n:
                n += 1
        rows.append([src, n, gate, act, j])
        csts.append(cst[j])
        j += n
    return torch.tensor(rows, dtype=torch.int32).reshape(-1, 5), torch.tensor(csts, dtype=torch.float32)


class _GateFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_tbl, out_cst, in_tbl, in_cst, dout, ch_tbl=None, ch_cst=None):
        rows, din = x.shape
        out = torch.empty(rows, dout, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            if ch_tbl is not None:
                rc = _lib.core().e3b_gate_fwd_channels(_lib._ptr(x), _lib._ptr(ch_tbl), _lib._ptr(ch_cst), _lib._ptr(out), rows,
                                                       din, dout, ch_tbl.shape[0], _lib.stream_ptr())
            else:
                rc = _lib.core().e3b_gate_fwd(_lib._ptr(x), _lib._ptr(out_tbl), _lib._ptr(out_cst), _lib._ptr(out), rows, din,
                                              dout, _lib.stream_ptr())
        _lib.check(rc, "e3b_gate_fwd")
        ctx.save_for_backward(x, in_tbl, in_cst)
        ctx.dout = dout
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out):
        x, in_tbl, in_cst = ctx.saved_tensors
        rows, din = x.shape
        gx = torch.empty_like(x)
        with torch.cuda.device(x.device):
            rc = _lib.core().e3b_gate_bwd(_lib._ptr(x), _lib._ptr(grad_out.contiguous()), _lib._ptr(in_tbl), _lib._ptr(in_cst),
                                          _lib._ptr(gx), rows, din, ctx.dout, _lib.stream_ptr())
        _lib.check(rc, "e3b_gate_bwd")
        return gx, None, None, None, None, None, None, None


class Gate(torch.nn.Module):
    def __init__(self, irreps_scalars, act_scalars, irreps_gates, act_gates, irreps_gated) -> None:
        super().__init__()
        irreps_scalars, irreps_gates, irreps_gated = Irreps(irreps_scalars), Irreps(irreps_gates), Irreps(irreps_gated)
        if len(irreps_gates) > 0 and irreps_gates.lmax > 0:
            raise ValueError(f"Gate scalars must be scalars, instead got irreps_gates = {irreps_gates}")
        if len(irreps_scalars) > 0 and irreps_scalars.lmax > 0:
            raise ValueError(f"Scalars must be scalars, instead got irreps_scalars = {irreps_scalars}")
        if irreps_gates.num_irreps != irreps_gated.num_irreps:
            raise ValueError(f"There are {irreps_gated.num_irreps} irreps in irreps_gated, but a different number "
                             f"({irreps_gates.num_irreps}) of gate scalars in irreps_gates")
        names_s = [_act_name(a) for a in act_scalars]
        names_g = [_act_name(a) for a in act_gates]
        out_scalars = _activation_irreps(irreps_scalars, names_s)
        out_gates = _activation_irreps(irreps_gates, names_g)

        # input layout: the three irreps concatenated, sorted (stable) and simplified (_Sortcut)
        pieces = [irreps_scalars.simplify(), irreps_gates.simplify(), irreps_gated.simplify()]
        self.irreps_scalars, self.irreps_gates, self.irreps_gated = pieces
        # activations are given per block of the un-simplified irreps: expand them to one entry per channel first
        chan_act_s = [n for (mul, _), n in zip(irreps_scalars, names_s) for _ in range(mul)]
        chan_act_g = [n for (mul, _), n in zip(irreps_gates, names_g) for _ in range(mul)]
        chan_par_g = [ir.p for (mul, ir) in out_gates for _ in range(mul)]
        cat = Irreps(list(pieces[0]) + list(pieces[1]) + list(pieces[2]))
        srt, p, _ = cat.sort()
        self.irreps_in = srt.simplify()
        off_sorted = srt.offsets()
        # column of the first element of block b of `cat` inside the sorted input row
        col_of = [off_sorted[p[b]] for b in range(len(cat))]
        n_s, n_g = len(pieces[0]), len(pieces[1])

        scal_cols = [col_of[b] + u for b in range(n_s) for u in range(pieces[0][b].mul)]
        gate_cols = [col_of[n_s + b] + u for b in range(n_g) for u in range(pieces[1][b].mul)]
        assert len(scal_cols) == len(chan_act_s) and len(gate_cols) == len(chan_act_g)

        out_tbl, out_cst = [], []
        din = self.irreps_in.dim
        in_tbl = [[3, 0, 0, 0, 3] for _ in range(din)]
        in_cst = [0.0] * din
        for col, name in zip(scal_cols, chan_act_s):
            cst = normalize2mom_constant(name) if name is not None else 1.0
            in_tbl[col] = [0, len(out_tbl), 1, 0, _ACT_CODE[name]]
            in_cst[col] = cst
            out_tbl.append([col, -1, _ACT_CODE[name]])
            out_cst.append(cst)
        gated_out = []
        g = 0
        for b, (mul, ir) in enumerate(pieces[2]):
            base = col_of[n_s + n_g + b]
            for u in range(mul):
                name, gcol = chan_act_g[g], gate_cols[g]
                cst = normalize2mom_constant(name) if name is not None else 1.0
                in_tbl[gcol] = [2, len(out_tbl), ir.dim, base + u * ir.dim, _ACT_CODE[name]]
                in_cst[gcol] = cst
                for m in range(ir.dim):
                    c = base + u * ir.dim + m
                    in_tbl[c] = [1, len(out_tbl), 1, gcol, _ACT_CODE[name]]
                    in_cst[c] = cst
                    out_tbl.append([c, gcol, _ACT_CODE[name]])
                    out_cst.append(cst)
                g += 1
            # parity of a gated block times the parity of its (activated) gates; the reference requires the gates of
            # one block to share it (ElementwiseTensorProduct pairs whole blocks after matching multiplicities)
            pg = chan_par_g[g - 1] if mul > 0 else 1
            gated_out.append((mul, (ir.l, ir.p * pg)))
        self.irreps_out = Irreps(list(out_scalars) + gated_out)
        self.register_buffer("_out_tbl", torch.tensor(out_tbl, dtype=torch.int32).reshape(-1, 3), persistent=False)
        self.register_buffer("_out_cst", torch.tensor(out_cst, dtype=torch.float32), persistent=False)
        self.register_buffer("_in_tbl", torch.tensor(in_tbl, dtype=torch.int32).reshape(-1, 5), persistent=False)
        self.register_buffer("_in_cst", torch.tensor(in_cst, dtype=torch.float32), persistent=False)
        ch_tbl, ch_cst = channel_tables(self._out_tbl, self._out_cst)
        self.register_buffer("_ch_tbl", ch_tbl, persistent=False)
        self.register_buffer("_ch_cst", ch_cst, persistent=False)

    def __repr__(self) -> str:
        return f"{self.__class__.__name__} ({self.irreps_in} -> {self.irreps_out})"

    def forward(self, features: torch.Tensor) -> torch.Tensor:
        if not features.is_cuda:
            raise NotImplementedError("Gate runs on CUDA tensors only")
        torch._assert(features.shape[-1] == self.irreps_in.dim, "Incorrect last dimension for features")
        lead = features.shape[:-1]
        x = features.reshape(-1, self.irreps_in.dim).to(torch.float32).contiguous()
        for name in ("_out_tbl", "_in_tbl", "_ch_tbl"):
            _lib.require_operand(getattr(self, name), x, f"Gate.{name} (move the module with .to(device))", None, torch.int32)
        for name in ("_out_cst", "_in_cst", "_ch_cst"):
            _lib.require_operand(getattr(self, name), x, f"Gate.{name} (move the module with .to(device))")
        out = _GateFunction.apply(x, self._out_tbl, self._out_cst, self._in_tbl, self._in_cst, self.irreps_out.dim,
                                  self._ch_tbl if self._ch_tbl.shape[0] > 0 else None, self._ch_cst)
        return out.reshape(*lead, self.irreps_out.dim)
