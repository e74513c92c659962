"""Edge -> node message passing on the GPU: CSR construction and the fused convolution step.

The reference performs (``e3nn/nn/models/v2106/points_convolution.py:105-106``)

    edge_features = tp(node_features[edge_src], edge_attr, weight)
    node_features = scatter(edge_features, edge_dst, dim_size=N).div(num_neighbors**0.5)

with ``scatter`` an unordered ``scatter_add_`` (``:13-17``).  Here the three steps (plus, optionally,
the spherical harmonics that produce ``edge_attr`` from the edge vectors) are one kernel over a
destination-sorted CSR: the ``[E, irreps_mid.dim]`` messages never exist in memory and every
destination row is summed in a fixed order.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .o3._tensor_product import TensorProduct


def csr_from_dst(edge_dst: torch.Tensor, num_nodes: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Stable destination sort of an edge list on the GPU.

    Returns ``perm`` (edge ids in destination order, equal to ``argsort(edge_dst, stable=True)``) and
    ``rowptr`` (``[0, cumsum(bincount(edge_dst, num_nodes))]``), both int64.
    Raises ``IndexError`` if a destination is outside ``[0, num_nodes)``.
    """
    _lib.require_cuda(edge_dst)
    if edge_dst.dtype != torch.int64:
        raise TypeError("edge_dst must be int64")
    edge_dst = edge_dst.contiguous()
    E, dev = edge_dst.numel(), edge_dst.device
    core = _lib.core()
    perm = torch.empty(E, dtype=torch.int64, device=dev)
    rowptr = torch.empty(num_nodes + 1, dtype=torch.int64, device=dev)
    nbytes = core.e3b_csr_scratch_bytes(E, num_nodes)
    scratch = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = core.e3b_csr_from_dst(_lib._ptr(edge_dst), E, num_nodes, _lib._ptr(perm), _lib._ptr(rowptr),
                                   _lib._ptr(scratch), scratch.numel(), _lib._ptr(status), _lib.stream_ptr())
    _lib.check(rc, "e3b_csr_from_dst")
    if int(status.item()) != 0:
        raise IndexError("edge_dst holds a value outside [0, num_nodes)")
    return perm, rowptr


class _ConvFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, node_x, x2, weight, edge_src, rowptr, perm, mod, in2_mode: int, scale: float):
        N = rowptr.numel() - 1
        E = edge_src.numel()
        out = torch.empty(N, mod.dout, dtype=torch.float32, device=node_x.device)
        status = _lib.status_word(node_x.device)
        with torch.cuda.device(node_x.device), _lib.nvtx_range("e3b_conv_fwd"):
            rc = mod.lib.e3b_conv_fwd(_lib._ptr(node_x), _lib._ptr(x2), in2_mode, _lib._ptr(edge_src), _lib._ptr(rowptr),
                                      _lib._ptr(perm), _lib._ptr(weight), _lib._ptr(out), N, node_x.shape[0], E,
                                      scale, _lib._ptr(status), _lib.stream_ptr())
        mod.check(rc, "e3b_conv_fwd")
        _lib.status_after_launch(node_x.device)
        ctx.save_for_backward(node_x, x2, weight, edge_src, rowptr, perm if perm is not None else torch.empty(0))
        ctx.meta = (mod, in2_mode, scale, perm is not None)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out):
        node_x, x2, weight, edge_src, rowptr, perm = ctx.saved_tensors
        mod, in2_mode, scale, has_perm = ctx.meta
        grad_out = grad_out.contiguous()
        N, E = rowptr.numel() - 1, edge_src.numel()
        gx = None
        if ctx.needs_input_grad[0]:
            gx = torch.empty_like(node_x)
            st = _lib.status_word(node_x.device)
            with torch.cuda.device(node_x.device), _lib.nvtx_range("e3b_conv_bwd_x"):
                rc = mod.lib.e3b_conv_bwd_x(_lib._ptr(x2), in2_mode, _lib._ptr(edge_src), _lib._ptr(rowptr),
                                            _lib._ptr(perm) if has_perm else None, _lib._ptr(weight), _lib._ptr(grad_out),
                                            _lib._ptr(gx), N, node_x.shape[0], E, scale, _lib._ptr(st), _lib.stream_ptr())
            mod.check(rc, "e3b_conv_bwd_x")
            _lib.status_after_launch(node_x.device)
            if not (ctx.needs_input_grad[1] or ctx.needs_input_grad[2]):
                return gx, None, None, None, None, None, None, None, None
        gw = torch.empty_like(weight)
        gx2 = torch.empty_like(x2)
        status = _lib.status_word(node_x.device)
        with torch.cuda.device(node_x.device), _lib.nvtx_range("e3b_conv_bwd"):
            rc = mod.lib.e3b_conv_bwd(_lib._ptr(node_x), _lib._ptr(x2), in2_mode, _lib._ptr(edge_src), _lib._ptr(rowptr),
                                      _lib._ptr(perm) if has_perm else None, _lib._ptr(weight), _lib._ptr(grad_out),
                                      _lib._ptr(gw), _lib._ptr(gx2), N, node_x.shape[0], E, scale, _lib._ptr(status),
                                      _lib.stream_ptr())
        mod.check(rc, "e3b_conv_bwd")
        _lib.status_after_launch(node_x.device)
        return gx, gx2, gw, None, None, None, None, None, None


def conv_uvu(
    tp: TensorProduct,
    node_features: torch.Tensor,
    edge_attr: torch.Tensor,
    edge_src: torch.Tensor,
    rowptr: torch.Tensor,
    weight: torch.Tensor,
    perm: Optional[torch.Tensor] = None,
    scale: float = 1.0,
    edge_attr_is_vector: bool = False,
    check_indices: bool = False,
) -> torch.Tensor:
    """``scatter(tp(node_features[edge_src], edge_attr, weight), edge_dst, N) * scale`` in one kernel.

    ``tp`` must consist of 'uvu' paths with per-edge weights (the layout built by the reference's
    ``Convolution``).  The destination of every edge is given by ``rowptr`` (``[N+1]``, from
    `csr_from_dst`): edge slot ``ee`` in ``[rowptr[n], rowptr[n+1])`` belongs to destination ``n`` and
    refers to edge ``perm[ee]`` (or ``ee`` itself when ``perm`` is ``None``, i.e. the edge arrays are
    already sorted by destination).  With ``edge_attr_is_vector=True`` ``edge_attr`` holds the edge
    vectors ``[E, 3]`` and the spherical harmonics (``normalize=True, normalization='component'``) are
    evaluated inside the kernel; ``tp.irreps_in2`` must then be ``Y^0..Y^L``.
    ``check_indices=True`` synchronises, reads the device's status word and raises ``IndexError`` if a source
    index was out of range.  Without it a reported condition (bad index, a bounded wait that gave up) is raised
    by the next e3nn_b200 call on the device after the kernel has finished, or by `e3nn_b200.check_status()`.
    """
    _lib.require_cuda(node_features, edge_attr, weight, edge_src, rowptr)
    if tp._uvw_ids or getattr(tp, "_uuu_ids", None) or tp.shared_weights:
        raise NotImplementedError("conv_uvu needs a TensorProduct made of 'uvu' paths with shared_weights=False")
    _lib.require_same_device(node_features, edge_attr, weight, edge_src, rowptr, perm)
    if edge_src.dtype != torch.int64 or rowptr.dtype != torch.int64 or (perm is not None and perm.dtype != torch.int64):
        raise TypeError("edge_src, rowptr and perm must be int64")
    _lib.poll_status(node_features.device)
    mod = tp._uvu_module()
    in2_mode = 1 if edge_attr_is_vector else 0
    E = edge_src.numel()
    torch._assert(node_features.shape[-1] == mod.d1, "Incorrect last dimension for node_features")
    torch._assert(edge_attr.shape == (E, 3 if edge_attr_is_vector else mod.d2), "Incorrect shape for edge_attr")
    torch._assert(weight.shape == (E, mod.wn), "Incorrect shape for weight")
    if edge_attr_is_vector and mod.sh_lmax < 0:
        raise ValueError(f"irreps_in2={tp.irreps_in2} is not a spherical-harmonics layout 0..L")
    for t in (node_features, edge_attr, weight):
        if t.dtype != torch.float32:
            raise TypeError(f"conv_uvu is fp32 only, got {t.dtype}")
    out = _ConvFunction.apply(
        node_features.contiguous(), edge_attr.contiguous(), weight.contiguous(), edge_src.contiguous(),
        rowptr.contiguous(), None if perm is None else perm.contiguous(), mod, in2_mode, float(scale),
    )
    if check_indices:  # synchronises: reads the status word the kernel wrote
        _lib.check_status(node_features.device, "conv_uvu")
    return out
