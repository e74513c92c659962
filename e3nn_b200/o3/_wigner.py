"""Clebsch-Gordan constants in the real basis, and Wigner D matrices.

``wigner_3j(l1, l2, l3)`` returns the same tensor as ``e3nn.o3.wigner_3j``
(``e3nn/o3/_wigner.py:102-164``): the SU(2) Clebsch-Gordan coefficients
(Condon-Shortley phases) rotated into the real spherical-harmonics basis with the
``(-i)^l`` phase of ``change_basis_real_to_complex`` (``_wigner.py:30-51``) and scaled
to unit Frobenius norm.  The SU(2) coefficients are evaluated here with Racah's
closed form using exact integer arithmetic; the reference uses an equivalent closed
form (``_wigner.py:234-286``).  These tensors are only ever *constants*: they are
baked into the generated CUDA kernels as immediates and never live on the GPU.

``wigner_D`` follows ``_wigner.py:62-99`` (Y-X-Y Euler angles through the matrix
exponential of the real so(3) generators) and is used by the equivariance tests only.
"""
from __future__ import annotations

import functools
from fractions import Fraction
from math import factorial

import numpy as np
import torch


def _su2_cg_coefficient(j1: int, m1: int, j2: int, m2: int, j3: int, m3: int) -> float:
    """<j1 m1; j2 m2 | j3 m3> for integer spins (Racah's formula)."""
    if m3 != m1 + m2 or not (abs(j1 - j2) <= j3 <= j1 + j2):
        return 0.0
    if abs(m1) > j1 or abs(m2) > j2 or abs(m3) > j3:
        return 0.0
    f = factorial
    pref = Fraction(
        (2 * j3 + 1) * f(j3 + j1 - j2) * f(j3 - j1 + j2) * f(j1 + j2 - j3),
        f(j1 + j2 + j3 + 1),
    ) * (f(j3 + m3) * f(j3 - m3) * f(j1 - m1) * f(j1 + m1) * f(j2 - m2) * f(j2 + m2))
    total = Fraction(0)
    for k in range(0, j1 + j2 - j3 + 1):
        args = (k, j1 + j2 - j3 - k, j1 - m1 - k, j2 + m2 - k, j3 - j2 + m1 + k, j3 - j1 - m2 + k)
        if min(args) < 0:
            continue
        den = 1
        for a in args:
            den *= f(a)
        total += Fraction((-1) ** k, den)
    # both factors are exact rationals; only the final square root is rounded
    return float(total) * float(pref) ** 0.5


def _su2_cg(j1: int, j2: int, j3: int) -> np.ndarray:
    out = np.zeros((2 * j1 + 1, 2 * j2 + 1, 2 * j3 + 1), dtype=np.float64)
    for m1 in range(-j1, j1 + 1):
        for m2 in range(-j2, j2 + 1):
            m3 = m1 + m2
            if abs(m3) <= j3:
                out[j1 + m1, j2 + m2, j3 + m3] = _su2_cg_coefficient(j1, m1, j2, m2, j3, m3)
    return out


def _real_to_complex(l: int) -> np.ndarray:
    """Unitary Q with rows = complex index m, columns = real index (``_wigner.py:30-41``)."""
    q = np.zeros((2 * l + 1, 2 * l + 1), dtype=np.complex128)
    s = 1.0 / np.sqrt(2.0)
    for m in range(-l, 0):
        q[l + m, l - m] = s
        q[l + m, l + m] = -1j * s
    q[l, l] = 1.0
    for m in range(1, l + 1):
        q[l + m, l + m] = (-1) ** m * s
        q[l + m, l - m] = 1j * (-1) ** m * s
    return (-1j) ** l * q


@functools.lru_cache(maxsize=None)
def _so3_cg(l1: int, l2: int, l3: int) -> np.ndarray:
    q1, q2, q3 = _real_to_complex(l1), _real_to_complex(l2), _real_to_complex(l3)
    c = _su2_cg(l1, l2, l3).astype(np.complex128)
    c = np.einsum("ij,kl,nm,ikn->jlm", q1, q2, np.conj(q3), c)
    assert np.abs(c.imag).max() < 1e-9
    c = np.ascontiguousarray(c.real)
    c /= np.linalg.norm(c)
    c[np.abs(c) < 1e-14] = 0.0
    c.setflags(write=False)
    return c


def wigner_3j_numpy(l1: int, l2: int, l3: int) -> np.ndarray:
    """fp64 ``[2l1+1, 2l2+1, 2l3+1]`` array (read-only, cached)."""
    assert isinstance(l1, int) and isinstance(l2, int) and isinstance(l3, int)
    assert abs(l2 - l3) <= l1 <= l2 + l3
    return _so3_cg(l1, l2, l3)


def wigner_3j(l1: int, l2: int, l3: int, dtype=None, device=None) -> torch.Tensor:
    """Same values and layout as ``e3nn.o3.wigner_3j`` (``_wigner.py:102-147``)."""
    c = torch.from_numpy(wigner_3j_numpy(l1, l2, l3).copy())
    if dtype is None:
        dtype = torch.get_default_dtype()
    return c.to(dtype=dtype, device=device).contiguous()


# ---------------------------------------------------------------------------------------
# Wigner D (tests only)
# ---------------------------------------------------------------------------------------
def _su2_generators(j: int) -> np.ndarray:
    m = np.arange(-j, j)
    raising = np.diag(-np.sqrt(j * (j + 1) - m * (m + 1)), k=-1).astype(np.complex128)
    m = np.arange(-j + 1, j + 1)
    lowering = np.diag(np.sqrt(j * (j + 1) - m * (m - 1)), k=1).astype(np.complex128)
    m = np.arange(-j, j + 1)
    return np.stack([0.5 * (raising + lowering), np.diag(1j * m), -0.5j * (raising - lowering)], axis=0)


@functools.lru_cache(maxsize=None)
def _so3_generators(l: int) -> np.ndarray:
    x = _su2_generators(l)
    q = _real_to_complex(l)
    x = np.conj(q.T) @ x @ q
    assert np.abs(x.imag).max() < 1e-9
    return np.ascontiguousarray(x.real)


def so3_generators(l: int) -> torch.Tensor:
    return torch.from_numpy(_so3_generators(l).copy()).to(torch.get_default_dtype())


def wigner_D(l: int, alpha: torch.Tensor, beta: torch.Tensor, gamma: torch.Tensor) -> torch.Tensor:
    """D^l(alpha, beta, gamma), Y-X-Y convention, shape ``(..., 2l+1, 2l+1)``."""
    alpha, beta, gamma = torch.broadcast_tensors(alpha, beta, gamma)
    two_pi = 2 * torch.pi
    alpha = alpha[..., None, None] % two_pi
    beta = beta[..., None, None] % two_pi
    gamma = gamma[..., None, None] % two_pi
    X = torch.from_numpy(_so3_generators(l).copy()).to(dtype=alpha.dtype, device=alpha.device)
    return torch.matrix_exp(alpha * X[1]) @ torch.matrix_exp(beta * X[0]) @ torch.matrix_exp(gamma * X[1])
