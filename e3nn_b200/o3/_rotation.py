"""Minimal rotation helpers (Y-X-Y Euler angles) used by the equivariance tests.

Conventions follow ``e3nn/o3/_rotation.py``: ``angles_to_matrix`` (:362-382) is
``R_y(alpha) R_x(beta) R_y(gamma)``, ``xyz_to_angles`` (:672-700) measures ``beta`` from
the +y axis, ``matrix_to_angles`` (:385-409) inverts ``angles_to_matrix``.
"""
from __future__ import annotations

import math

import torch


def matrix_x(angle: torch.Tensor) -> torch.Tensor:
    c, s = angle.cos(), angle.sin()
    o, z = torch.ones_like(angle), torch.zeros_like(angle)
    return torch.stack([torch.stack([o, z, z], -1), torch.stack([z, c, -s], -1), torch.stack([z, s, c], -1)], -2)


def matrix_y(angle: torch.Tensor) -> torch.Tensor:
    c, s = angle.cos(), angle.sin()
    o, z = torch.ones_like(angle), torch.zeros_like(angle)
    return torch.stack([torch.stack([c, z, s], -1), torch.stack([z, o, z], -1), torch.stack([-s, z, c], -1)], -2)


def angles_to_matrix(alpha, beta, gamma) -> torch.Tensor:
    alpha, beta, gamma = torch.broadcast_tensors(alpha, beta, gamma)
    return matrix_y(alpha) @ matrix_x(beta) @ matrix_y(gamma)


def xyz_to_angles(xyz):
    xyz = torch.nn.functional.normalize(xyz, p=2.0, dim=-1).clamp(-1, 1)
    return torch.atan2(xyz[..., 0], xyz[..., 2]), torch.acos(xyz[..., 1])


def matrix_to_angles(R):
    assert torch.allclose(torch.det(R), R.new_tensor(1))
    a, b = xyz_to_angles(R @ R.new_tensor([0.0, 1.0, 0.0]))
    R = angles_to_matrix(a, b, torch.zeros_like(a)).transpose(-1, -2) @ R
    return a, b, torch.atan2(R[..., 0, 2], R[..., 0, 0])


def rand_angles(*shape, dtype=None, device=None):
    alpha = 2 * math.pi * torch.rand(shape, dtype=dtype, device=device)
    gamma = 2 * math.pi * torch.rand(shape, dtype=dtype, device=device)
    beta = torch.rand(shape, dtype=dtype, device=device).mul(2).sub(1).acos()
    return alpha, beta, gamma


def rand_matrix(*shape, dtype=None, device=None) -> torch.Tensor:
    """Uniformly random proper rotations, shape ``(*shape, 3, 3)``."""
    return angles_to_matrix(*rand_angles(*shape, dtype=dtype, device=device))
