"""Radial network that produces the per-edge 'uvu' weights (adjacent to the hot path).

``FullyConnectedNet`` mirrors ``e3nn/nn/_fc.py:52-88`` (weights ``layer{i}.weight`` of shape
``[h_in, h_out]`` ~ N(0,1), every layer divided by sqrt(h_in), hidden layers followed by the
activation rescaled to unit second moment, ``e3nn/math/_normalize_activation.py:9-57``) and ``bessel``
mirrors ``e3nn/math/_bessel.py:6-37``.  With ``math_mode='tf32x3'`` the layers whose widths fit
(h_in % 32 == 0, h_out % 16 == 0: the 64 -> weight_numel layer) run on the tcgen05 kernel of
``codegen/tc_gemm.py`` with hi/lo-split tf32 operands, forward and input gradient; other layers and
``math_mode='fp32'`` are plain dense GEMMs left to cuBLAS through ``torch.matmul`` in fp32.  The
elementwise parts are torch operators.
"""
from __future__ import annotations

import hashlib
import math
from functools import lru_cache
from typing import Callable, List, Optional

import torch

from .. import _lib
from ..codegen import tc_gemm


@lru_cache(maxsize=None)
def normalize2mom_constant(name: str = "silu") -> float:
    """<f(z)^2>^{-1/2} for z ~ N(0,1), estimated exactly like the reference: 1e6 samples, seed 0, fp64."""
    f = {"silu": torch.nn.functional.silu, "tanh": torch.tanh, "relu": torch.relu, "sigmoid": torch.sigmoid,
         "abs": torch.abs}[name]
    gen = torch.Generator(device="cpu").manual_seed(0)
    z = torch.randn(1_000_000, generator=gen, dtype=torch.float64)
    return f(z).pow(2).mean().pow(-0.5).item()


def bessel(x: torch.Tensor, n: int, x_max: float = 1.0) -> torch.Tensor:
    """Bessel radial basis ``sqrt(2/c) sin(k pi x / c) / x``, k = 1..n; shape ``[..., n]``."""
    assert isinstance(n, int)
    x = x[..., None]
    k = torch.arange(1, n + 1, dtype=x.dtype, device=x.device)
    x_nonzero = torch.where(x == 0.0, torch.ones_like(x), x)
    return math.sqrt(2.0 / x_max) * torch.where(
        x == 0, k * math.pi / x_max, torch.sin(k * math.pi / x_max * x_nonzero) / x_nonzero
    )


class _ScaledMatmul(torch.autograd.Function):
    """``scale * x @ W`` on the tensor cores (hi/lo-split tf32 operands).  The gradient w.r.t. ``x`` is the
    transposed module; the gradient w.r.t. ``W`` (``scale * x^T g``, a plain [h_in, rows] x [rows, h_out] product
    needed only in training) is a library fp32 GEMM."""

    @staticmethod
    def forward(ctx, x, weight, fwd_spec, bwd_spec, scale):
        out = torch.empty(x.shape[0], weight.shape[1], dtype=torch.float32, device=x.device)
        _lib.tc_gemm_module(fwd_spec).run(x, None, weight, out, 2)
        ctx.save_for_backward(weight, x if weight.requires_grad else None)
        ctx.bwd_spec, ctx.scale = bwd_spec, scale
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out):
        weight, x = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = torch.empty(grad_out.shape[0], weight.shape[0], dtype=torch.float32, device=grad_out.device)
            _lib.tc_gemm_module(ctx.bwd_spec).run(grad_out, None, weight, gx, 2)
        if ctx.needs_input_grad[1]:
            gw = (x.t() @ grad_out) * ctx.scale
        return gx, gw, None, None, None


class _Layer(torch.nn.Module):
    def __init__(self, h_in: int, h_out: int, act: Optional[Callable], cst: float, var_in: float, var_out: float,
                 math_mode: str = "fp32"):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.randn(h_in, h_out))
        self.act, self.cst = act, cst
        self.h_in, self.h_out, self.var_in, self.var_out = h_in, h_out, var_in, var_out
        self.math_mode = math_mode
        self._tc = None

    def _scale(self) -> float:
        if self.act is not None:
            return 1.0 / (self.h_in * self.var_in) ** 0.5
        return 1.0 / (self.h_in * self.var_in / self.var_out) ** 0.5

    def _tc_specs(self):
        if self._tc is None:
            s = self._scale()
            tag = f"mm{self.h_in}x{self.h_out}s{hashlib.sha1(repr(s).encode()).hexdigest()[:10]}"
            self._tc = (tc_gemm.matmul_gemm_spec(self.h_in, self.h_out, False, s, tag + "f"),
                        tc_gemm.matmul_gemm_spec(self.h_in, self.h_out, True, s, tag + "t"))
        return self._tc

    def _matmul(self, x: torch.Tensor) -> torch.Tensor:
        use_tc = self.math_mode == "tf32x3" and x.is_cuda and x.dtype == torch.float32 and x.dim() == 2
        if use_tc:
            fwd, bwd = self._tc_specs()
            if fwd is not None and bwd is not None:
                _lib.require_operand(self.weight, x, "layer weight", self.h_in * self.h_out)
                torch._assert(x.shape[1] == self.h_in, "Incorrect last dimension for the layer input")
                return _ScaledMatmul.apply(x.contiguous(), self.weight, fwd, bwd, self._scale())
        return x @ (self.weight * self._scale())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self._matmul(x)
        if self.act is not None:
            return self.act(x) * (self.cst * self.var_out ** 0.5)
        return x


class FullyConnectedNet(torch.nn.Sequential):
    """``FullyConnectedNet(hs, act)`` with the reference's parameter names (``layer0.weight`` ...)."""

    def __init__(self, hs: List[int], act=None, variance_in: int = 1, variance_out: int = 1, out_act: bool = False,
                 math_mode: str = "fp32"):
        super().__init__()
        assert math_mode in ("fp32", "tf32x3")
        self.hs = list(hs)
        cst = 1.0
        if act is not None:
            name = getattr(act, "__name__", None)
            if name not in ("silu", "tanh", "relu"):
                raise NotImplementedError("FullyConnectedNet supports silu, tanh and relu activations")
            cst = normalize2mom_constant(name)
            if abs(cst - 1) < 1e-4:
                cst = 1.0
        var_in = variance_in
        for i, (h1, h2) in enumerate(zip(self.hs, self.hs[1:])):
            last = i == len(self.hs) - 2
            var_out = variance_out if last else 1
            a = act if (not last or out_act) else None
            setattr(self, f"layer{i}", _Layer(h1, h2, a, cst, var_in, var_out, math_mode))
            var_in = var_out

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}{self.hs}"
