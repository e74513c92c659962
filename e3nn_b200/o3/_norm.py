"""Drop-in ``Norm``: the Euclidean norm of every irrep channel (``e3nn/o3/_norm.py:9-75``).

The squared norm of a channel is its 'uuu' product with itself into ``0e``; with a path weight of ``2l+1`` the
coefficient (3j symbol ``delta / sqrt(2l+1)``, 'component' normalisation of a scalar output: 1) comes out as exactly
``sum_m x_m^2``.  The products run on the kernels of `TensorProduct`; the square root is one elementwise operation.
"""
from __future__ import annotations

import torch

from ._irreps import Irreps
from ._tensor_product import TensorProduct


class Norm(torch.nn.Module):
    def __init__(self, irreps_in, squared: bool = False) -> None:
        super().__init__()
        irreps_in = Irreps(irreps_in).simplify()
        scalars = Irreps([(mul, "0e") for mul, _ in irreps_in])
        paths = [(n, n, n, "uuu", False, ir.dim) for n, (_, ir) in enumerate(irreps_in)]
        self.tp = TensorProduct(irreps_in, irreps_in, scalars, paths, irrep_normalization="component")
        self.irreps_in = irreps_in
        self.irreps_out = scalars.simplify()
        self.squared = squared

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}({self.irreps_in})"

    def forward(self, features: torch.Tensor) -> torch.Tensor:
        """``[..., irreps_in.dim] -> [..., number of channels]``."""
        out = self.tp(features, features)
        if self.squared:
            return out
        # the clamp keeps the gradient of the square root finite at rounding-level negative values
        return out.relu().sqrt()
