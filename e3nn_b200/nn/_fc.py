"""Radial network that produces the per-edge 'uvu' weights (adjacent to the hot path).

``FullyConnectedNet`` mirrors ``e3nn/nn/_fc.py:52-88`` (weights ``layer{i}.weight`` of shape
``[h_in, h_out]`` ~ N(0,1), every layer divided by sqrt(h_in), hidden layers followed by the
activation rescaled to unit second moment, ``e3nn/math/_normalize_activation.py:9-57``) and ``bessel``
mirrors ``e3nn/math/_bessel.py:6-37``.  The two matrix products are plain dense GEMMs and are left to
cuBLAS through ``torch.matmul`` in fp32; the elementwise parts are torch operators.  Nothing here is
a hand-written kernel yet: fusing this network into the convolution kernel is the next step for the
full interaction block.
"""
from __future__ import annotations

import math
from functools import lru_cache
from typing import Callable, List, Optional

import torch


@lru_cache(maxsize=None)
def normalize2mom_constant(name: str = "silu") -> float:
    """<f(z)^2>^{-1/2} for z ~ N(0,1), estimated exactly like the reference: 1e6 samples, seed 0, fp64."""
    f = {"silu": torch.nn.functional.silu, "tanh": torch.tanh, "relu": torch.relu}[name]
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


class _Layer(torch.nn.Module):
    def __init__(self, h_in: int, h_out: int, act: Optional[Callable], cst: float, var_in: float, var_out: float):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.randn(h_in, h_out))
        self.act, self.cst = act, cst
        self.h_in, self.h_out, self.var_in, self.var_out = h_in, h_out, var_in, var_out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.act is not None:
            x = x @ (self.weight / (self.h_in * self.var_in) ** 0.5)
            return self.act(x) * (self.cst * self.var_out ** 0.5)
        return x @ (self.weight / (self.h_in * self.var_in / self.var_out) ** 0.5)


class FullyConnectedNet(torch.nn.Sequential):
    """``FullyConnectedNet(hs, act)`` with the reference's parameter names (``layer0.weight`` ...)."""

    def __init__(self, hs: List[int], act=None, variance_in: int = 1, variance_out: int = 1, out_act: bool = False):
        super().__init__()
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
            setattr(self, f"layer{i}", _Layer(h1, h2, a, cst, var_in, var_out))
            var_in = var_out

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}{self.hs}"
