"""Drop-in ``SphericalHarmonics`` / ``spherical_harmonics`` backed by the sm_100a kernel.

Same constructor, attributes, error behaviour and call signature as
``e3nn/o3/_spherical_harmonics.py:15-190``.  The arithmetic runs in ``e3b_sh_fwd`` /
``e3b_sh_bwd`` (fp32, CUDA only).
"""
from __future__ import annotations

from typing import Any, List, Union

import torch

from .. import _lib
from ._irreps import Irreps

_NORM_CODE = {"component": 0, "integral": 1, "norm": 2}


class _SHFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, lmax: int, normalize: bool, code: int):
        n = x.shape[0]
        out = torch.empty(n, (lmax + 1) ** 2, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device), _lib.nvtx_range("e3b_sh_fwd"):
            rc = _lib.core().e3b_sh_fwd(_lib._ptr(x), _lib._ptr(out), n, lmax, int(normalize), code, _lib.stream_ptr())
        _lib.check(rc, "e3b_sh_fwd")
        ctx.save_for_backward(x)
        ctx.args = (lmax, normalize, code)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out: torch.Tensor):
        (x,) = ctx.saved_tensors
        lmax, normalize, code = ctx.args
        grad_out = grad_out.contiguous()
        gx = torch.empty_like(x)
        with torch.cuda.device(x.device):
            rc = _lib.core().e3b_sh_bwd(_lib._ptr(x), _lib._ptr(grad_out), _lib._ptr(gx), x.shape[0], lmax,
                                        int(normalize), code, _lib.stream_ptr())
        _lib.check(rc, "e3b_sh_bwd")
        return gx, None, None, None


class SphericalHarmonics(torch.nn.Module):
    """Module version of `spherical_harmonics`; parameters as in the reference."""

    def __init__(
        self,
        irreps_out: Union[int, List[int], str, Irreps],
        normalize: bool,
        normalization: str = "integral",
        irreps_in: Any = None,
    ) -> None:
        super().__init__()
        self.normalize = normalize
        self.normalization = normalization
        assert normalization in ["integral", "component", "norm"]

        if isinstance(irreps_out, str):
            irreps_out = Irreps(irreps_out)
        if isinstance(irreps_out, Irreps) and irreps_in is None:
            for mul, (l, p) in irreps_out:
                if l % 2 == 1 and p == 1:
                    irreps_in = Irreps("1e")
        if irreps_in is None:
            irreps_in = Irreps("1o")
        irreps_in = Irreps(irreps_in)
        if irreps_in not in (Irreps("1x1o"), Irreps("1x1e")):
            raise ValueError(
                "irreps_in for SphericalHarmonics must be either a vector (`1x1o`) or a pseudovector (`1x1e`), "
                f"not `{irreps_in}`"
            )
        self.irreps_in = irreps_in
        input_p = irreps_in[0].ir.p

        if isinstance(irreps_out, Irreps):
            ls = []
            for mul, (l, p) in irreps_out:
                if p != input_p**l:
                    raise ValueError(
                        f"irreps_out `{irreps_out}` passed to SphericalHarmonics asked for an output of l = {l} with "
                        f"parity p = {p}, which is inconsistent with the input parity {input_p} — the output parity "
                        f"should have been p = {input_p**l}"
                    )
                ls.extend([l] * mul)
        elif isinstance(irreps_out, int):
            ls = [irreps_out]
        else:
            ls = list(irreps_out)

        self.irreps_out = Irreps([(1, (l, input_p**l)) for l in ls]).simplify()
        self._ls_list = ls
        self._lmax = max(ls)
        self._is_range_lmax = ls == list(range(max(ls) + 1))
        if self._lmax > 12:
            raise NotImplementedError(
                "spherical_harmonics maximum l implemented is 12, send us an email to ask for more"
            )

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        _lib.require_cuda(x)
        if x.dtype != torch.float32:
            raise TypeError(f"e3nn_b200 spherical harmonics are fp32 only, got {x.dtype}")
        assert x.shape[-1] == 3
        lead = x.shape[:-1]
        flat = x.reshape(-1, 3).contiguous()
        sh = _SHFunction.apply(flat, self._lmax, self.normalize, _NORM_CODE[self.normalization])
        if not self._is_range_lmax:
            sh = torch.cat([sh[:, l * l : (l + 1) * (l + 1)] for l in self._ls_list], dim=-1)
        return sh.reshape(*lead, sh.shape[-1])

    def extra_repr(self) -> str:
        return f"{self._ls_list}, normalize={self.normalize}, normalization={self.normalization}"


def spherical_harmonics(
    l: Union[int, List[int], str, Irreps], x: torch.Tensor, normalize: bool, normalization: str = "integral"
) -> torch.Tensor:
    """``e3nn.o3.spherical_harmonics`` (``_spherical_harmonics.py:115-190``) on the GPU."""
    return SphericalHarmonics(l, normalize, normalization)(x)
