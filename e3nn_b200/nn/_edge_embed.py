"""Edge embedding (edge vectors, Bessel basis, first radial layer) as one kernel per direction.

Host side of ``e3b_radial_embed_fwd`` / ``e3b_radial_embed_bwd``.  Mirrors
``edge_vec = pos[src] - pos[dst] + shift`` (``e3nn/nn/models/gate_points_2101.py:328``),
``e3nn.math.bessel`` (``e3nn/math/_bessel.py:6-37``) and the first layer of ``FullyConnectedNet``
(``e3nn/nn/_fc.py:38-48``).  Differentiable with respect to the positions only.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib

_ACT = {"silu": 0, "tanh": 1, "relu": 2, None: 3}
# "bessel" = e3nn.math.bessel; the others = soft_one_hot_linspace(..., basis=<name>) ("soft_bessel" = its basis="bessel")
_BASIS = {"bessel": 0, "gaussian": 1, "cosine": 2, "smooth_finite": 3, "fourier": 4, "soft_bessel": 5}
_ENVELOPE = {None: 0, "smooth_cutoff": 1}


class _EdgeEmbedFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pos, edge_src, edge_dst, shift, w0, spec, w_scale, act_scale, act):
        E, N = edge_src.numel(), pos.shape[0]
        nb, hidden = w0.shape
        edge_vec = torch.empty(E, 3, dtype=torch.float32, device=pos.device)
        h = torch.empty(E, hidden, dtype=torch.float32, device=pos.device)
        status = _lib.status_word(pos.device)
        with torch.cuda.device(pos.device), _lib.nvtx_range("e3b_radial_embed_fwd"):
            rc = _lib.core().e3b_radial_embed_fwd(
                _lib._ptr(pos), _lib._ptr(edge_src), _lib._ptr(edge_dst), _lib._ptr(shift) if shift is not None else None,
                _lib._ptr(w0), E, N, nb, hidden, *spec, w_scale, act_scale, act, _lib._ptr(edge_vec), _lib._ptr(h),
                _lib._ptr(status), _lib.stream_ptr())
        _lib.check(rc, "e3b_radial_embed_fwd")
        _lib.status_after_launch(pos.device)
        ctx.save_for_backward(pos, edge_src, edge_dst, shift if shift is not None else torch.empty(0), w0)
        ctx.meta = (shift is not None, spec, w_scale, act_scale, act)
        return edge_vec, h

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_vec, grad_h):
        pos, edge_src, edge_dst, shift, w0 = ctx.saved_tensors
        has_shift, spec, w_scale, act_scale, act = ctx.meta
        if ctx.needs_input_grad[4]:
            raise NotImplementedError("the fused edge embedding has no gradient w.r.t. the first-layer weights")
        E, N = edge_src.numel(), pos.shape[0]
        nb, hidden = w0.shape
        grad_pos = torch.zeros_like(pos)
        if grad_h is None:
            grad_h = torch.zeros(E, hidden, dtype=torch.float32, device=pos.device)
        status = _lib.status_word(pos.device)
        with torch.cuda.device(pos.device), _lib.nvtx_range("e3b_radial_embed_bwd"):
            rc = _lib.core().e3b_radial_embed_bwd(
                _lib._ptr(pos), _lib._ptr(edge_src), _lib._ptr(edge_dst), _lib._ptr(shift) if has_shift else None,
                _lib._ptr(w0), _lib._ptr(grad_h.contiguous()), _lib._ptr(grad_vec.contiguous()) if grad_vec is not None else None,
                E, N, nb, hidden, *spec, w_scale, act_scale, act, _lib._ptr(grad_pos), _lib._ptr(status), _lib.stream_ptr())
        _lib.check(rc, "e3b_radial_embed_bwd")
        _lib.status_after_launch(pos.device)
        return grad_pos, None, None, None, None, None, None, None, None


def edge_embed(pos: torch.Tensor, edge_src: torch.Tensor, edge_dst: torch.Tensor, shift: Optional[torch.Tensor],
               w0: torch.Tensor, r_max: float, w_scale: float, act_scale: float, act: Optional[str],
               check_indices: bool = False, basis: str = "bessel", cutoff: bool = True, start: float = 0.0,
               basis_scale: float = 1.0, envelope: Optional[str] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(edge_vec [E,3], h [E,hidden])`` with ``h = env(r) * act_scale * act(w_scale * B(r) @ w0)``, ``r = |edge_vec|``.

    ``basis="bessel"``: ``B = e3nn.math.bessel(r, num_basis, r_max)``; ``"gaussian" | "cosine" | "smooth_finite" |
    "fourier" | "soft_bessel"``: ``B = basis_scale * soft_one_hot_linspace(r, start, r_max, num_basis, basis, cutoff)``
    (``e3nn/math/_soft_one_hot_linspace.py``; ``"soft_bessel"`` is its ``basis="bessel"``).  ``envelope="smooth_cutoff"``
    multiplies ``h`` by ``smooth_cutoff(r / r_max)`` (``gate_points_2101.py:136-141``).

    ``w0`` is ``[num_basis <= 16, hidden in {32, 64, 96, 128}]``.  With ``check_indices`` the device status word
    is read back (a synchronisation) and an index outside the node range raises ``IndexError``.
    """
    if not pos.is_cuda:
        raise NotImplementedError("edge_embed runs on CUDA tensors only")
    _lib.require_same_device(pos, edge_src, edge_dst, shift, w0)
    _lib.poll_status(pos.device)
    if act not in _ACT:
        raise NotImplementedError(f"edge_embed: unsupported activation {act!r}")
    if pos.dtype != torch.float32 or w0.dtype != torch.float32:
        raise NotImplementedError("edge_embed computes in float32")
    if edge_src.dtype != torch.int64 or edge_dst.dtype != torch.int64:
        raise TypeError("edge_src and edge_dst must be int64")
    if basis not in _BASIS:
        raise ValueError(f'basis="{basis}" is not a valid entry')
    if envelope not in _ENVELOPE:
        raise ValueError(f"unknown envelope {envelope!r}")
    nb, hidden = w0.shape
    if nb > 16 or hidden not in (32, 64, 96, 128):
        raise NotImplementedError("edge_embed: num_basis <= 16 and hidden in {32, 64, 96, 128}")
    spec = (_BASIS[basis], int(bool(cutoff)), _ENVELOPE[envelope], float(start), float(r_max), float(basis_scale))
    shift_c = shift.contiguous().float() if shift is not None else None
    vec, h = _EdgeEmbedFunction.apply(pos.contiguous(), edge_src.contiguous(), edge_dst.contiguous(), shift_c,
                                      w0.detach().contiguous() if not w0.requires_grad else w0.contiguous(),
                                      spec, float(w_scale), float(act_scale), _ACT[act])
    if check_indices:
        _lib.check_status(pos.device, "edge_embed")
    return vec, h
