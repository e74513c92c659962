"""Sharding of a graph over the GPUs of one node: contiguous destination ranges + one all-gather.

Messages are independent per edge; the only couplings are the sum over a destination's incoming
edges and the read of arbitrary source rows.  Rank ``r`` therefore owns a contiguous range of
destination rows (chosen so that edge counts balance), every edge whose destination lies in it,
those edges' weights / vectors, and the output rows.  The input features of all nodes are
all-gathered once per layer into local memory; the fused kernel then reads local memory only, and
no output reduction across ranks is needed.  Nothing like this exists in the reference (its graphs
are single-device edge lists).
"""
from __future__ import annotations

import datetime
import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


# SMs a collective's kernel may occupy, and the same number the persistent kernel that overlaps it leaves free
# (``InteractionBlock.overlap_reserved_sms``).  Measured on 4 GPUs (262,144 atoms, radial layer under the feature
# all-gather): no limit 19.15 ms per step, 16 SMs 18.39 (the gather then ends 0.5 ms after the layer), 24 SMs 17.98,
# 32 SMs 17.94.
OVERLAP_SMS = int(os.environ.get("E3NN_B200_OVERLAP_SMS", "24"))      # 0: no limit on either side


def init_process_group(backend: str, device: Optional[torch.device] = None, timeout_s: float = 120.0, **kwargs) -> None:
    """``torch.distributed.init_process_group`` with the failure behaviour this package relies on: every collective
    carries a timeout (`timeout_s`), and with NCCL a collective that times out or fails asynchronously (a peer that
    died between steps) is turned into an exception in the waiting rank instead of a hang: the communicator's
    watchdog polls for asynchronous errors and aborts the communicator (``TORCH_NCCL_ASYNC_ERROR_HANDLING``, set
    here unless the caller chose a value).  NCCL's kernels are limited to ``OVERLAP_SMS`` CTAs (``NCCL_MAX_CTAS``,
    unless the caller chose a value): the collectives of a step run UNDER compute kernels that own whole SMs, and a
    collective spread over more SMs than those kernels leave free delays them by its whole duration.  Rendezvous
    settings come from the environment as usual."""
    if backend == "nccl":
        os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "1")
        if OVERLAP_SMS > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", str(OVERLAP_SMS))
        if device is not None:
            kwargs.setdefault("device_id", device)
    dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)


def partition_rows_by_edges(rowptr: torch.Tensor, world: int) -> List[int]:
    """Row boundaries ``b[0]=0 <= ... <= b[world]=N`` with ~E/world edges per part (equal row counts when those
    balance the edges to within 1 %).

    ``b[r]`` is the smallest row whose first edge slot is >= r*E/world, the same rule the fused
    kernel uses to split rows over its warp teams."""
    assert world >= 1
    rp = rowptr.detach().cpu()
    n = rp.numel() - 1
    e = int(rp[-1])
    if world > 1 and n % world == 0 and e > 0:
        # Equal row counts let the feature all-gather run as ONE all_gather_into_tensor instead of a group of
        # broadcasts of unequal slices; taken when the edge counts then stay within 1 % of the balanced split
        # (a system of uniform density).
        rows = n // world
        most = max(int(rp[(r + 1) * rows]) - int(rp[r * rows]) for r in range(world))
        if most * world <= 1.01 * e:
            return [r * rows for r in range(world + 1)]
    targets = torch.tensor([(e * r) // world for r in range(1, world)], dtype=rp.dtype)
    inner = torch.searchsorted(rp[:-1].contiguous(), targets, right=False).tolist() if world > 1 else []
    bounds = [0] + [min(int(v), n) for v in inner] + [n]
    for i in range(1, len(bounds)):
        bounds[i] = max(bounds[i], bounds[i - 1])
    return bounds


def local_shard(rowptr: torch.Tensor, bounds: List[int], rank: int) -> Tuple[int, int, int, int, torch.Tensor]:
    """(n0, n1, e0, e1, local_rowptr): rows [n0,n1), edge slots [e0,e1), CSR of the shard starting at 0."""
    n0, n1 = bounds[rank], bounds[rank + 1]
    e0, e1 = int(rowptr[n0]), int(rowptr[n1])
    return n0, n1, e0, e1, (rowptr[n0 : n1 + 1] - rowptr[n0]).contiguous()


def all_gather_rows(x_local: torch.Tensor, bounds: List[int], group: Optional[dist.ProcessGroup] = None,
                    out: Optional[torch.Tensor] = None, async_op: bool = False):
    """Concatenation over ranks of ``x_local`` (rank r holds rows [bounds[r], bounds[r+1])).

    Returns ``out``; with ``async_op`` returns ``(out, wait)`` where ``wait()`` makes the current stream wait for
    the collective (NCCL runs it on its own stream, so work enqueued before ``wait()`` overlaps the transfer).
    Uneven row counts: NCCL gathers them as one group of broadcasts (``all_gather`` on a list of slices);
    backends without that (gloo) get one broadcast per owner.
    """
    world = len(bounds) - 1
    n, d = bounds[-1], x_local.shape[1]
    if out is None:
        out = torch.empty(n, d, dtype=x_local.dtype, device=x_local.device)
    works = []
    if world == 1:
        out.copy_(x_local)
    else:
        sizes = [bounds[r + 1] - bounds[r] for r in range(world)]
        x_local = x_local.contiguous()
        if len(set(sizes)) == 1:
            works.append(dist.all_gather_into_tensor(out, x_local, group=group, async_op=True))
        elif dist.get_backend(group) == "nccl":
            works.append(dist.all_gather([out[bounds[r] : bounds[r + 1]] for r in range(world)], x_local, group=group,
                                         async_op=True))
        else:
            rank = dist.get_rank(group)
            out[bounds[rank] : bounds[rank + 1]].copy_(x_local)
            for r in range(world):
                if sizes[r] > 0:
                    src = dist.get_global_rank(group, r) if group is not None else r
                    works.append(dist.broadcast(out[bounds[r] : bounds[r + 1]], src=src, group=group, async_op=True))

    def wait() -> None:
        for w in works:
            w.wait()

    if async_op:
        return out, wait
    wait()
    return out
