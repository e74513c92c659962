"""One NequIP-style interaction block: the caller of the hot path, assembled from its kernels.

Mirrors the data flow of ``e3nn/nn/models/v2106/points_convolution.py:99-113`` restricted to the steps
on the accelerated path (no self-connection / node attributes):

    edge_vec = pos[src] - pos[dst] + shift                       (gate_points_2101.py:328 sign convention)
    w        = FullyConnectedNet([num_basis, hidden, weight_numel], silu)(bessel(|edge_vec|))
    mid      = scatter(tp(x[src], Y(edge_vec), w), dst) / sqrt(num_neighbors)     -> e3b_conv_fwd
    out      = Linear(mid)                                                         -> e3b_dense_fwd

Gradients w.r.t. the positions flow through ``e3b_conv_bwd`` (per-edge weight and edge-vector
cotangents, spherical harmonics included) and the transposed Linear plan; torch autograd connects
them through the radial network.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib, layouts
from ..message_passing import conv_uvu
from ..o3 import Irreps, Linear
from ._edge_embed import edge_embed
from ._fc import FullyConnectedNet, bessel


def radius_graph_pbc(pos: torch.Tensor, box: float, cutoff: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Neighbour list of a periodic cubic box, both directions, sorted by destination then source.

    Returns ``edge_src, edge_dst, shift`` with ``edge_vec = pos[src] - pos[dst] + shift``
    (``gate_points_2101.py:328``).  CUDA positions with ``box >= 3 * cutoff`` use the device cell list
    (``e3b_neighbor_count`` / ``e3b_neighbor_fill``; ``neighbor_list_pbc`` also returns the CSR row pointers);
    host positions use a k-d tree (scipy), which is also the checker of the device builder in the tests.
    """
    if pos.is_cuda and box >= 3.0 * cutoff:
        src, dst, shift, _ = neighbor_list_pbc(pos, box, cutoff)
        return src, dst, shift
    return _radius_graph_pbc_host(pos, box, cutoff)


def neighbor_list_pbc(pos: torch.Tensor, box: float, cutoff: float, rows: Optional[Tuple[int, int]] = None):
    """Device cell list: ``edge_src, edge_dst, shift, rowptr`` (edges sorted by destination, then source).

    ``rows=(n0, n1)``: only the edges whose destination lies in ``[n0, n1)`` (the shard of a rank that owns those
    rows); ``rowptr`` is then the CSR of the range, starting at 0, while ``edge_src`` / ``edge_dst`` keep global atom
    numbers.  All atoms are binned in either case; only the rows of the range are walked."""
    from .. import _lib

    if not pos.is_cuda:
        raise NotImplementedError("neighbor_list_pbc runs on CUDA tensors only (use radius_graph_pbc for host positions)")
    if box < 3.0 * cutoff:
        raise NotImplementedError("the cell list needs box >= 3 * cutoff")
    pos32 = pos.detach().to(torch.float32).contiguous()
    n, dev = pos32.shape[0], pos32.device
    core = _lib.core()
    nbytes = core.e3b_neighbor_scratch_bytes(n, float(box), float(cutoff))
    scratch = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=dev)
    n0, n1 = (0, n) if rows is None else (int(rows[0]), int(rows[1]))
    if not (0 <= n0 <= n1 <= n):
        raise IndexError(f"rows {rows} outside [0, {n}]")
    rowptr = torch.empty(n1 - n0 + 1, dtype=torch.int64, device=dev)
    with torch.cuda.device(dev):
        rc = core.e3b_neighbor_count_rows(_lib._ptr(pos32), n, float(box), float(cutoff), _lib._ptr(scratch), scratch.numel(),
                                          n0, n1, _lib._ptr(rowptr), _lib.stream_ptr())
        _lib.check(rc, "e3b_neighbor_count_rows")
        num_edges = int(rowptr[n1 - n0].item())       # the one synchronisation: the caller allocates the edge arrays
        src = torch.empty(num_edges, dtype=torch.int64, device=dev)
        dst = torch.empty(num_edges, dtype=torch.int64, device=dev)
        shift = torch.empty(num_edges, 3, dtype=torch.float32, device=dev)
        if num_edges > 0:
            rc = core.e3b_neighbor_fill_rows(_lib._ptr(pos32), n, float(box), float(cutoff), _lib._ptr(scratch), scratch.numel(),
                                             n0, n1, _lib._ptr(rowptr), _lib._ptr(src), _lib._ptr(dst), _lib._ptr(shift),
                                             _lib.stream_ptr())
            _lib.check(rc, "e3b_neighbor_fill_rows")
    return src, dst, shift.to(pos.dtype), rowptr


def _radius_graph_pbc_host(pos: torch.Tensor, box: float, cutoff: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    import numpy as np
    from scipy.spatial import cKDTree

    p = pos.detach().cpu().double().numpy() % box
    tree = cKDTree(p, boxsize=box)
    pairs = tree.query_pairs(cutoff, output_type="ndarray")
    src = np.concatenate([pairs[:, 0], pairs[:, 1]])
    dst = np.concatenate([pairs[:, 1], pairs[:, 0]])
    order = np.lexsort((src, dst))
    src, dst = src[order], dst[order]
    d = p[src] - p[dst]
    shift = -box * np.round(d / box)
    # positions may lie outside [0, box): express the shift relative to the given coordinates
    raw = pos.detach().cpu().double().numpy()
    shift = (p[src] - raw[src]) - (p[dst] - raw[dst]) + shift
    dev = pos.device
    return (torch.from_numpy(src).to(dev), torch.from_numpy(dst).to(dev),
            torch.from_numpy(shift).to(device=dev, dtype=pos.dtype))


class InteractionBlock(torch.nn.Module):
    def __init__(self, irreps_node, lmax: int, num_basis: int = 8, hidden: int = 64, r_max: float = 5.0,
                 num_neighbors: float = 1.0, irreps_out=None, linear_math_mode: str = "tf32x3",
                 radial_math_mode: str = "tf32x3"):
        super().__init__()
        self.irreps_node = Irreps(irreps_node)
        self.irreps_sh = Irreps.spherical_harmonics(lmax)
        self.irreps_out = Irreps(irreps_out) if irreps_out is not None else self.irreps_node
        self.tp = layouts.conv_tensor_product(self.irreps_node, self.irreps_sh, self.irreps_out)
        self.fc = FullyConnectedNet([num_basis, hidden, self.tp.weight_numel], torch.nn.functional.silu,
                                    math_mode=radial_math_mode)
        self.lin = Linear(self.tp.irreps_out, self.irreps_out, math_mode=linear_math_mode)
        self.num_basis, self.r_max, self.num_neighbors = num_basis, r_max, num_neighbors
        # SMs the radial layer leaves free while a feature transfer overlaps it (forward(before_conv=...)); 0: none
        self.overlap_reserved_sms = 0

    def edge_weights(self, edge_vec: torch.Tensor) -> torch.Tensor:
        # the basis sin(k pi r / c) / r is evaluated in fp64 (8 values per edge, negligible cost): in fp32
        # the argument reduction of sin alone costs about one digit of the 1e-5 error budget
        basis = bessel(edge_vec.double().norm(dim=-1), self.num_basis, self.r_max).to(edge_vec.dtype)
        return self.fc(basis)

    def forward(self, pos: torch.Tensor, node_features: torch.Tensor, edge_src: torch.Tensor, edge_dst: torch.Tensor,
                rowptr: torch.Tensor, shift: Optional[torch.Tensor] = None, before_conv=None,
                phase_mark=None) -> torch.Tensor:
        """``edge_*`` must be sorted by destination and ``rowptr`` their CSR (`e3nn_b200.csr_from_dst`).

        ``before_conv``: optional callable run right before the convolution, the first step that reads
        ``node_features`` (a sharded caller passes the ``wait`` of its asynchronous feature all-gather, which then
        overlaps the edge embedding and the radial network).
        ``phase_mark``: optional callable ``phase_mark(name)`` called on the launching stream at the phase
        boundaries of the step (forward: after the radial network, after ``before_conv``, after the convolution,
        after the Linear; backward, through tensor hooks: after the transposed Linear, after the convolution
        gradient, after the transposed radial layer), e.g. to record CUDA events."""
        layer0 = self.fc.layer0
        fused = (pos.is_cuda and pos.dtype == torch.float32 and len(self.fc.hs) == 3 and self.num_basis <= 16
                 and self.fc.hs[1] in (32, 64, 96, 128) and not (torch.is_grad_enabled() and layer0.weight.requires_grad))
        if fused:
            # vectors, Bessel basis and the first radial layer in one kernel (and one for their gradient)
            act = getattr(layer0.act, "__name__", None) if layer0.act is not None else None
            edge_vec, h = edge_embed(pos, edge_src, edge_dst, shift, layer0.weight, self.r_max, layer0._scale(),
                                     layer0.cst * layer0.var_out ** 0.5, act)
            # a transfer in flight (before_conv is its wait) runs a kernel of its own: leave it some SMs
            limit = 148 - self.overlap_reserved_sms if (before_conv is not None and self.overlap_reserved_sms > 0) else None
            with _lib.tc_gemm_cta_limit(limit):
                w = self.fc.layer1(h)
        else:
            edge_vec = pos[edge_src] - pos[edge_dst]
            if shift is not None:
                edge_vec = edge_vec + shift
            w = self.edge_weights(edge_vec)
        mark = phase_mark if phase_mark is not None else (lambda name: None)
        if phase_mark is not None and w.requires_grad:
            w.register_hook(lambda g: mark("bwd_conv"))
            if fused and h.requires_grad:
                h.register_hook(lambda g: mark("bwd_radial"))
        mark("radial")
        if before_conv is not None:
            before_conv()
        mark("gather_wait")
        mid = conv_uvu(self.tp, node_features, edge_vec, edge_src, rowptr, w, scale=self.num_neighbors ** -0.5,
                       edge_attr_is_vector=True)
        if phase_mark is not None and mid.requires_grad:
            mid.register_hook(lambda g: mark("bwd_linear"))
        mark("conv")
        out = self.lin(mid)
        mark("linear")
        return out
