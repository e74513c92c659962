"""Irrep / Irreps bookkeeping for the O(3) hot path (host side only).

Mirrors the public behaviour of ``e3nn/o3/_irreps.py`` (``Irrep`` :14-264,
``_MulIr`` :267-298, ``Irreps`` :301-806) as far as the tensor-product, linear and
spherical-harmonics modules need it: parsing of strings such as ``"32x0e + 16x1o"``,
dimensions, slices, sort / simplify, random tensors and the selection rule of
``Irrep * Irrep``.  Nothing in here touches the GPU; the kernels only ever see the
flat offsets derived from these objects.
"""
from __future__ import annotations

import collections
import itertools
import re
from typing import Iterable, Iterator, List, Tuple, Union

import torch

_IRREP_RE = re.compile(r"^\s*(\d+)\s*([eoy])\s*$")


class Irrep(tuple):
    """One irreducible representation of O(3): degree ``l`` and parity ``p`` (+1 / -1).

    Ordering is the plain ``(l, p)`` tuple ordering, which is what the reference's
    ``Irreps.sort`` relies on (``e3nn/o3/_irreps.py:587-614``).
    """

    __slots__ = ()

    def __new__(cls, l, p=None):
        if p is None:
            if isinstance(l, Irrep):
                return l
            if isinstance(l, MulIr):
                return l.ir
            if isinstance(l, str):
                m = _IRREP_RE.match(l)
                if m is None:
                    raise ValueError(f'unable to convert string "{l}" into an Irrep')
                deg = int(m.group(1))
                par = {"e": 1, "o": -1, "y": (-1) ** deg}[m.group(2)]
                l, p = deg, par
            elif isinstance(l, tuple):
                l, p = l
        if not isinstance(l, int) or isinstance(l, bool) or l < 0:
            raise ValueError(f"l must be positive integer, got {l}")
        if p not in (-1, 1):
            raise ValueError(f"parity must be on of (-1, 1), got {p}")
        return tuple.__new__(cls, (l, p))

    @property
    def l(self) -> int:  # noqa: E743
        return self[0]

    @property
    def p(self) -> int:
        return self[1]

    @property
    def dim(self) -> int:
        return 2 * self[0] + 1

    def is_scalar(self) -> bool:
        return self[0] == 0 and self[1] == 1

    def __repr__(self) -> str:
        return f"{self[0]}{'e' if self[1] == 1 else 'o'}"

    @classmethod
    def iterator(cls, lmax=None) -> Iterator["Irrep"]:
        """0e, 0o, 1o, 1e, 2e, 2o, ... (natural parity first)."""
        for l in itertools.count():
            yield Irrep(l, (-1) ** l)
            yield Irrep(l, -((-1) ** l))
            if l == lmax:
                break

    def __mul__(self, other) -> Iterator["Irrep"]:
        """Selection rule: |l1-l2| <= l <= l1+l2 with parity p1*p2."""
        other = Irrep(other)
        for l in range(abs(self.l - other.l), self.l + other.l + 1):
            yield Irrep(l, self.p * other.p)

    def __rmul__(self, mul) -> "Irreps":
        assert isinstance(mul, int)
        return Irreps([(mul, self)])

    def __add__(self, other) -> "Irreps":
        return Irreps(self) + Irreps(other)

    def D_from_angles(self, alpha, beta, gamma, k=None) -> torch.Tensor:
        from ._wigner import wigner_D

        if k is None:
            k = torch.zeros_like(alpha)
        alpha, beta, gamma, k = torch.broadcast_tensors(alpha, beta, gamma, k)
        return wigner_D(self.l, alpha, beta, gamma) * self.p ** k[..., None, None]

    def D_from_matrix(self, R) -> torch.Tensor:
        from ._rotation import matrix_to_angles

        d = torch.det(R).sign()
        R = d[..., None, None] * R
        k = (1 - d) / 2
        return self.D_from_angles(*matrix_to_angles(R), k)

    def count(self, _value):
        raise NotImplementedError

    def index(self, _value):
        raise NotImplementedError

    def __contains__(self, _object):
        raise NotImplementedError

    def __len__(self):
        raise NotImplementedError


class MulIr(tuple):
    """A multiplicity paired with an `Irrep`; unpacks as ``mul, ir``."""

    __slots__ = ()

    def __new__(cls, mul, ir=None):
        if ir is None:
            mul, ir = mul
        assert isinstance(mul, int)
        return tuple.__new__(cls, (mul, Irrep(ir)))

    @property
    def mul(self) -> int:
        return self[0]

    @property
    def ir(self) -> Irrep:
        return self[1]

    @property
    def dim(self) -> int:
        return self[0] * self[1].dim

    def __repr__(self) -> str:
        return f"{self[0]}x{self[1]}"

    def count(self, _value):
        raise NotImplementedError

    def index(self, _value):
        raise NotImplementedError


_MulIr = MulIr  # name used by the reference


def _parse_irreps_string(text: str) -> List[MulIr]:
    out: List[MulIr] = []
    if text.strip() == "":
        return out
    for term in text.split("+"):
        if "x" in term:
            mul_s, ir_s = term.split("x")
            mul = int(mul_s)
        else:
            mul, ir_s = 1, term
        if mul < 0:
            raise ValueError
        out.append(MulIr(mul, Irrep(ir_s)))
    return out


class Irreps(tuple):
    """Direct sum of irreps with multiplicities, e.g. ``Irreps("64x0e+64x1o")``.

    Feature vectors are laid out irrep after irrep; inside one entry the layout is
    ``[mul, 2l+1]`` row-major (``e3nn/o3/_tensor_product/_codegen.py:79-94``).
    """

    __slots__ = ()
    _is_e3nn_irreps = True

    def __new__(cls, irreps=None):
        if isinstance(irreps, Irreps):
            return tuple.__new__(cls, irreps)
        out: List[MulIr] = []
        if irreps is None:
            pass
        elif isinstance(irreps, Irrep):
            out.append(MulIr(1, irreps))
        elif isinstance(irreps, MulIr):
            out.append(irreps)
        elif isinstance(irreps, str):
            try:
                out = _parse_irreps_string(irreps)
            except Exception:
                raise ValueError(f'Unable to convert string "{irreps}" into an Irreps')
        else:
            for item in irreps:
                mul, ir = None, None
                if isinstance(item, str):
                    mul, ir = 1, Irrep(item)
                elif isinstance(item, Irrep):
                    mul, ir = 1, item
                elif isinstance(item, MulIr):
                    mul, ir = item
                elif len(item) == 2:
                    mul, ir = item
                    ir = Irrep(ir)
                if not (isinstance(mul, int) and mul >= 0 and ir is not None):
                    raise ValueError(f'Unable to interpret "{item}" as an irrep.')
                out.append(MulIr(mul, ir))
        return tuple.__new__(cls, out)

    @staticmethod
    def spherical_harmonics(lmax: int, p: int = -1) -> "Irreps":
        return Irreps([(1, (l, p**l)) for l in range(lmax + 1)])

    def slices(self) -> List[slice]:
        out, start = [], 0
        for mul_ir in self:
            out.append(slice(start, start + mul_ir.dim))
            start += mul_ir.dim
        return out

    def offsets(self) -> List[int]:
        """Start column of every entry in the flat feature vector."""
        return [s.start for s in self.slices()]

    def randn(self, *size: int, normalization: str = "component", requires_grad: bool = False, dtype=None, device=None):
        di = size.index(-1)
        lsize, rsize = size[:di], size[di + 1 :]
        if normalization == "component":
            return torch.randn(*lsize, self.dim, *rsize, requires_grad=requires_grad, dtype=dtype, device=device)
        if normalization == "norm":
            x = torch.zeros(*lsize, self.dim, *rsize, requires_grad=requires_grad, dtype=dtype, device=device)
            with torch.no_grad():
                for s, (mul, ir) in zip(self.slices(), self):
                    r = torch.randn(*lsize, mul, ir.dim, *rsize, dtype=dtype, device=device)
                    r.div_(r.norm(2, dim=di + 1, keepdim=True))
                    x.narrow(di, s.start, mul * ir.dim).copy_(r.reshape(*lsize, -1, *rsize))
            return x
        raise ValueError("Normalization needs to be 'norm' or 'component'")

    def __getitem__(self, i):
        x = tuple.__getitem__(self, i)
        if isinstance(i, slice):
            return Irreps(x)
        return x

    def __contains__(self, ir) -> bool:
        ir = Irrep(ir)
        return any(ir == other for _, other in self)

    def count(self, ir) -> int:
        ir = Irrep(ir)
        return sum(mul for mul, other in self if other == ir)

    def index(self, _object):
        raise NotImplementedError

    def __add__(self, irreps) -> "Irreps":
        return Irreps(tuple.__add__(self, Irreps(irreps)))

    def __mul__(self, other) -> "Irreps":
        if isinstance(other, Irreps):
            raise NotImplementedError("Use o3.TensorProduct for this, see the documentation")
        return Irreps(tuple.__mul__(self, other))

    def __rmul__(self, other) -> "Irreps":
        return Irreps(tuple.__rmul__(self, other))

    def simplify(self) -> "Irreps":
        """Merge *adjacent* equal irreps and drop zero multiplicities (no sorting)."""
        out: List[Tuple[int, Irrep]] = []
        for mul, ir in self:
            if out and out[-1][1] == ir:
                out[-1] = (out[-1][0] + mul, ir)
            elif mul > 0:
                out.append((mul, ir))
        return Irreps(out)

    def remove_zero_multiplicities(self) -> "Irreps":
        return Irreps([(mul, ir) for mul, ir in self if mul > 0])

    def sort(self):
        """Stable sort by (l, p).  Returns ``(irreps, p, inv)`` with ``p[old] = new``."""
        Ret = collections.namedtuple("sort", ["irreps", "p", "inv"])
        keyed = sorted((ir, i, mul) for i, (mul, ir) in enumerate(self))
        inv = tuple(i for _, i, _ in keyed)
        p = [0] * len(inv)
        for new, old in enumerate(inv):
            p[old] = new
        return Ret(Irreps([(mul, ir) for ir, _, mul in keyed]), tuple(p), inv)

    def regroup(self) -> "Irreps":
        return self.sort().irreps.simplify()

    @property
    def dim(self) -> int:
        return sum(mul * ir.dim for mul, ir in self)

    @property
    def num_irreps(self) -> int:
        return sum(mul for mul, _ in self)

    @property
    def ls(self) -> List[int]:
        return [l for mul, (l, _) in self for _ in range(mul)]

    @property
    def lmax(self) -> int:
        if len(self) == 0:
            raise ValueError("Cannot get lmax of empty Irreps")
        return max(self.ls)

    def __repr__(self) -> str:
        return "+".join(f"{mul_ir}" for mul_ir in self)

    def D_from_angles(self, alpha, beta, gamma, k=None) -> torch.Tensor:
        return _direct_sum(*[ir.D_from_angles(alpha, beta, gamma, k) for mul, ir in self for _ in range(mul)])

    def D_from_matrix(self, R) -> torch.Tensor:
        from ._rotation import matrix_to_angles

        d = torch.det(R).sign()
        R = d[..., None, None] * R
        k = (1 - d) / 2
        return self.D_from_angles(*matrix_to_angles(R), k)


def _direct_sum(*matrices: torch.Tensor) -> torch.Tensor:
    """Block-diagonal stack over the last two dims (batch dims must agree)."""
    if len(matrices) == 0:
        return torch.zeros(0, 0)
    lead = matrices[0].shape[:-2]
    n = sum(m.shape[-1] for m in matrices)
    out = matrices[0].new_zeros(*lead, n, n)
    i = 0
    for m in matrices:
        d = m.shape[-1]
        out[..., i : i + d, i : i + d] = m
        i += d
    return out
