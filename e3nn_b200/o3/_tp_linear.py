"""A fully connected tensor product followed by an ``o3.Linear``, evaluated as ONE tensor product.

The reference runs the two modules one after the other (``e3nn/o3/_tensor_product/_codegen.py:148-165`` then
``e3nn/o3/_linear.py:445-450``), which writes and re-reads the intermediate ``[rows, irreps_mid.dim]`` tensor.  Both
maps are linear in that intermediate and the Linear only mixes the channels of one irrep, so their composition is
again a 'uvw' product with the weights

    W'_{p,b}[u, v, w'] = c_ab * sum_w W_p[u, v, w] L_ab[w, w']        (path p into slot a, Linear path a -> b)

(``c_ab`` the Linear's path normalisation).  Forming ``W'`` costs ``sum_p mul1 * mul2 * mul_a * mul_b`` multiply-adds
per call (4.5 MFLOP for ``128x0e+64x1o+32x2e``), independent of the number of rows; the product kernel then
produces the Linear's output directly and the intermediate never exists.  Exact in real arithmetic; in floating
point the rounding of the intermediate is replaced by the rounding of ``W'``.

``W'`` is formed with differentiable torch operations on the two weight tensors, so gradients reach both modules'
parameters through the product's weight gradient; gradients w.r.t. the operands come from the product.
"""
from __future__ import annotations

from typing import List

import torch

from ._linear import Linear
from ._tensor_product import TensorProduct


class TensorProductLinear(torch.nn.Module):
    """``lin(tp(x, y))`` for a weight-shared 'uvw' ``tp`` and a bias-free, weight-shared ``lin``, as one product.

    ``tp`` and ``lin`` stay the owners of their parameters (``state_dict`` keys ``tp.weight``, ``lin.weight``, as when
    the two modules are held side by side)."""

    def __init__(self, tp: TensorProduct, lin: Linear, math_mode: str = None):
        super().__init__()
        if not isinstance(tp, TensorProduct) or not isinstance(lin, Linear):
            raise TypeError("TensorProductLinear(tp, lin) takes a TensorProduct and a Linear")
        if lin.irreps_in != tp.irreps_out:
            raise ValueError(f"lin.irreps_in = {lin.irreps_in} does not match tp.irreps_out = {tp.irreps_out}")
        if not (tp.shared_weights and tp.internal_weights and lin.shared_weights and lin.internal_weights):
            raise NotImplementedError("TensorProductLinear needs internal, shared weights in both modules")
        if lin.bias_numel > 0:
            raise NotImplementedError("TensorProductLinear does not take a Linear with biases")
        if any(ins.connection_mode != "uvw" or not ins.has_weight for ins in tp.instructions):
            raise NotImplementedError("TensorProductLinear needs a TensorProduct made of weighted 'uvw' paths")
        self.tp, self.lin = tp, lin
        self.irreps_in1, self.irreps_in2, self.irreps_out = tp.irreps_in1, tp.irreps_in2, lin.irreps_out
        # composed instruction list: one path per (product path p into slot a, Linear path a -> b)
        instr: List[tuple] = []
        self._pairs: List[tuple] = []
        for n, ins in enumerate(tp.instructions):
            for m, lins in enumerate(lin.instructions):
                if lins.i_in == ins.i_out and 0 not in lins.path_shape and 0 not in ins.path_shape:
                    # the composed path keeps the product's coefficient; 'none' normalisations take its square
                    instr.append((ins.i_in1, ins.i_in2, lins.i_out, "uvw", True, float(ins.path_weight) ** 2))
                    self._pairs.append((n, m, float(lins.path_weight)))
        self.fused = TensorProduct(tp.irreps_in1, tp.irreps_in2, lin.irreps_out, instr, irrep_normalization="none",
                                   path_normalization="none", internal_weights=False, shared_weights=True,
                                   math_mode=math_mode if math_mode is not None else tp.math_mode)

    def composed_weight(self) -> torch.Tensor:
        """``W'`` in the instruction order of the fused product (differentiable w.r.t. both weight tensors).

        Without autograd (inference) the result is kept until one of the two weight tensors is modified in place
        or replaced (their version counters and storage are compared), so repeated calls do no weight arithmetic."""
        tw, lw = self.tp.weight, self.lin.weight
        track = torch.is_grad_enabled() and (tw.requires_grad or lw.requires_grad)
        key = (tw.data_ptr(), tw._version, lw.data_ptr(), lw._version, tw.device)
        if not track and getattr(self, "_cache_key", None) == key:
            return self._cache
        w = self._compose()
        if not track:
            self._cache_key, self._cache = key, w.detach()
        return w

    def _compose(self) -> torch.Tensor:
        tp_views = list(self.tp.weight_views())
        lin_views = list(self.lin.weight_views())
        parts = []
        for n, m, c in self._pairs:
            w = tp_views[n]                                   # [u, v, w]
            parts.append((w.reshape(-1, w.shape[-1]) @ (lin_views[m] * c)).reshape(-1))
        return torch.cat(parts) if parts else self.tp.weight.new_zeros(0)

    def forward(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        return self.fused(x, y, self.composed_weight())

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}({self.tp.irreps_in1} x {self.tp.irreps_in2} -> {self.tp.irreps_out} -> {self.irreps_out})"
