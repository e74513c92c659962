"""Host side of the tensor-core ('tf32') mode of fully-connected tensor products."""
from __future__ import annotations

import torch

from .. import _lib
from ..codegen import uvw_post, uvw_tc


def tc_eligible(tp) -> bool:
    return uvw_post.plan_groups(tp._spec) is not None or uvw_tc.plan_groups(tp._spec) is not None


def uvw_tc_forward(tp, x2d: torch.Tensor, y2d: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool):
    """out[:, written columns] (+)= uvw(x, y; w) on the tcgen05 tensor cores (tf32 operands, fp32 accumulate)."""
    mod = _lib.uvw_tc_module(tp._spec)
    target = torch.empty_like(out) if accumulate else out
    _lib.poll_status(out.device)
    with torch.cuda.device(out.device), _lib.nvtx_range("e3b_uvw_tc_fwd"):
        rc = mod.lib.e3b_uvw_tc_fwd(_lib._ptr(x2d), _lib._ptr(y2d), _lib._ptr(w), _lib._ptr(target), x2d.shape[0], 0,
                                    _lib._ptr(_lib.status_word(out.device)), _lib.stream_ptr())
    mod.check(rc, "e3b_uvw_tc_fwd")
    _lib.status_after_launch(out.device)
    if accumulate:
        offs = tp.irreps_out.offsets()
        for i_out in tp._uvw_written:
            mul, ir = tp.irreps_out[i_out]
            sl = slice(offs[i_out], offs[i_out] + mul * ir.dim)
            out[:, sl] += target[:, sl]
    return out
