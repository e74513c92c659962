"""Generator of straight-line CUDA device code for real spherical harmonics.

The polynomials are those of ``e3nn/o3/_spherical_harmonics.py:193-249`` for l <= 3
(written out in closed form there) and, for larger l, the recurrence the reference's
own generator used (``e3nn/o3/_spherical_harmonics_generator.py:57-65``):

    Y^{l+1}_k  =  s_l * sum_{a,i} C^{(l+1,1,l)}_{k a i}  r_a  Y^l_i ,

with ``s_l > 0`` chosen so that ``|Y^{l+1}(0,1,0)| = sqrt(2l+3)`` ('component'
normalisation).  The backward code is reverse-mode differentiation of the same
recurrence for every l >= 1 (for l <= 3 the closed forms are the same polynomials).

Output: a header with, for every L in 0..LMAX,

    __device__ void e3b_sh_fwd_<L>(float x, float y, float z, float* Y);
    __device__ void e3b_sh_bwd_<L>(float x, float y, float z, const float* Y, float* g,
                                   float& gx, float& gy, float& gz);

``Y`` / ``g`` hold (L+1)^2 values, l-major.  All indices are compile-time constants so
the arrays live in registers once the caller's loops are unrolled.
"""
from __future__ import annotations

import math
from functools import lru_cache
from typing import Dict, List, Tuple

import numpy as np

from ..o3._wigner import wigner_3j_numpy

LMAX_SUPPORTED = 12


def _f(v: float) -> str:
    """fp32 literal with enough digits to round-trip."""
    return f"{np.float32(v):.9e}f"


@lru_cache(maxsize=None)
def recurrence_terms(l: int) -> Tuple[Tuple[int, int, int, float], ...]:
    """Terms (k, a, i, coef) with Y^{l+1}_k += coef * r_a * Y^l_i (coef includes s_l)."""
    c = wigner_3j_numpy(l + 1, 1, l)
    pole = np.array([0.0, 1.0, 0.0])
    y_pole = _eval_fp64(l, pole)[l * l :]
    nxt = np.einsum("kai,a,i->k", c, pole, y_pole)
    s = math.sqrt(2 * l + 3) / np.linalg.norm(nxt)
    out = []
    for k in range(2 * l + 3):
        for a in range(3):
            for i in range(2 * l + 1):
                if c[k, a, i] != 0.0:
                    out.append((k, a, i, float(s * c[k, a, i])))
    return tuple(out)


def _eval_fp64(lmax: int, r: np.ndarray) -> np.ndarray:
    """Reference evaluation of the recurrence in fp64 (host; used for s_l and tests)."""
    y = [1.0]
    if lmax >= 1:
        y += [math.sqrt(3.0) * r[0], math.sqrt(3.0) * r[1], math.sqrt(3.0) * r[2]]
    for l in range(1, lmax):
        prev = y[l * l :]
        nxt = [0.0] * (2 * l + 3)
        for k, a, i, coef in recurrence_terms(l):
            nxt[k] += coef * r[a] * prev[i]
        y += nxt
    return np.array(y)


def _closed_forms_upto3(lmax: int) -> List[str]:
    lines = ["Y[0] = 1.0f;"]
    if lmax >= 1:
        s3 = _f(math.sqrt(3.0))
        lines += [f"Y[1] = {s3} * x;", f"Y[2] = {s3} * y;", f"Y[3] = {s3} * z;"]
    if lmax >= 2:
        s15, s5 = _f(math.sqrt(15.0)), _f(math.sqrt(5.0))
        lines += [
            "const float y2 = y * y;",
            "const float x2z2 = x * x + z * z;",
            f"Y[4] = {s15} * x * z;",
            f"Y[5] = {s15} * x * y;",
            f"Y[6] = {s5} * (y2 - 0.5f * x2z2);",
            f"Y[7] = {s15} * y * z;",
            f"Y[8] = {_f(0.5 * math.sqrt(15.0))} * (z * z - x * x);",
        ]
    if lmax >= 3:
        a, b, s7 = _f(math.sqrt(42.0) / 6.0), _f(math.sqrt(168.0) / 8.0), _f(math.sqrt(7.0))
        lines += [
            f"Y[9] = {a} * (Y[4] * z + Y[8] * x);",
            f"Y[10] = {s7} * Y[4] * y;",
            f"Y[11] = {b} * (4.0f * y2 - x2z2) * x;",
            f"Y[12] = {_f(0.5 * math.sqrt(7.0))} * y * (2.0f * y2 - 3.0f * x2z2);",
            f"Y[13] = {b} * z * (4.0f * y2 - x2z2);",
            f"Y[14] = {s7} * Y[8] * y;",
            f"Y[15] = {a} * (Y[8] * z - Y[4] * x);",
        ]
    return lines


def _recurrence_fwd_lines(l: int) -> List[str]:
    """Y block l+1 from block l, grouped as x*(..) + y*(..) + z*(..)."""
    base_prev, base_next = l * l, (l + 1) * (l + 1)
    by_k: Dict[int, Dict[int, List[Tuple[int, float]]]] = {}
    for k, a, i, coef in recurrence_terms(l):
        by_k.setdefault(k, {}).setdefault(a, []).append((i, coef))
    lines = []
    for k in range(2 * l + 3):
        parts = []
        for a, name in enumerate("xyz"):
            terms = by_k.get(k, {}).get(a)
            if not terms:
                continue
            inner = " + ".join(f"{_f(c)} * Y[{base_prev + i}]" for i, c in terms)
            parts.append(f"{name} * ({inner})")
        lines.append(f"Y[{base_next + k}] = " + (" + ".join(parts) if parts else "0.0f") + ";")
    return lines


def emit_fwd(lmax: int) -> str:
    body = _closed_forms_upto3(min(lmax, 3))
    for l in range(3, lmax):
        body += _recurrence_fwd_lines(l)
    text = "\n    ".join(body)
    return (
        f"__device__ __forceinline__ void e3b_sh_fwd_{lmax}(float x, float y, float z, float* __restrict__ Y) {{\n"
        f"    {text}\n}}\n"
    )


def emit_bwd(lmax: int) -> str:
    """g (cotangent of Y, modified in place) -> (gx, gy, gz); Y must hold the forward values."""
    lines = ["gx = 0.0f; gy = 0.0f; gz = 0.0f;"]
    for l in range(lmax - 1, 0, -1):
        base_prev, base_next = l * l, (l + 1) * (l + 1)
        # group by (k): t = g[next+k]; then gr_a += coef*t*Y_i ; g_i += coef*t*r_a
        by_k: Dict[int, List[Tuple[int, int, float]]] = {}
        for k, a, i, coef in recurrence_terms(l):
            by_k.setdefault(k, []).append((a, i, coef))
        lines.append("{")
        for k, terms in sorted(by_k.items()):
            lines.append(f"  const float t{k} = g[{base_next + k}];")
            for a, i, coef in terms:
                r = "xyz"[a]
                lines.append(f"  g{r} = fmaf({_f(coef)} * t{k}, Y[{base_prev + i}], g{r});")
                lines.append(f"  g[{base_prev + i}] = fmaf({_f(coef)} * t{k}, {r}, g[{base_prev + i}]);")
        lines.append("}")
    if lmax >= 1:
        s3 = _f(math.sqrt(3.0))
        lines += [f"gx = fmaf({s3}, g[1], gx);", f"gy = fmaf({s3}, g[2], gy);", f"gz = fmaf({s3}, g[3], gz);"]
    text = "\n    ".join(lines)
    return (
        f"__device__ __forceinline__ void e3b_sh_bwd_{lmax}(float x, float y, float z, const float* __restrict__ Y,\n"
        f"        float* __restrict__ g, float& gx, float& gy, float& gz) {{\n"
        f"    {text}\n}}\n"
    )


def emit_header(lmax_limit: int = LMAX_SUPPORTED) -> str:
    parts = [
        "// Generated by e3nn_b200/codegen/sh.py -- do not edit.\n"
        "// Real spherical harmonics, 'component' normalisation, l-major layout.\n"
        "#pragma once\n"
    ]
    for lmax in range(lmax_limit + 1):
        parts.append(emit_fwd(lmax))
        parts.append(emit_bwd(lmax))
    # compile-time dispatchers
    parts.append("template <int L> __device__ __forceinline__ void e3b_sh_fwd(float x, float y, float z, float* Y);\n")
    parts.append(
        "template <int L> __device__ __forceinline__ void e3b_sh_bwd(float x, float y, float z, const float* Y,\n"
        "        float* g, float& gx, float& gy, float& gz);\n"
    )
    for lmax in range(lmax_limit + 1):
        parts.append(
            f"template <> __device__ __forceinline__ void e3b_sh_fwd<{lmax}>(float x, float y, float z, float* Y) "
            f"{{ e3b_sh_fwd_{lmax}(x, y, z, Y); }}\n"
            f"template <> __device__ __forceinline__ void e3b_sh_bwd<{lmax}>(float x, float y, float z, const float* Y,\n"
            f"        float* g, float& gx, float& gy, float& gz) {{ e3b_sh_bwd_{lmax}(x, y, z, Y, g, gx, gy, gz); }}\n"
        )
    return "\n".join(parts)
