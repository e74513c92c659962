"""Drop-in ``TensorProduct`` / ``FullyConnectedTensorProduct`` for the 'uvu' and 'uvw' modes.

Constructor arguments, attributes (``irreps_in1/2/out``, ``instructions``, ``weight_numel``,
``internal_weights``, ``shared_weights``, ``weight``, ``output_mask``), weight layout, weight views,
broadcasting rules and error types follow ``e3nn/o3/_tensor_product/_tensor_product.py:23-609``
and ``_sub.py:10-68``.  The arithmetic runs in CUDA kernels only:

* 'uvu' paths: a per-layout generated module (``e3nn_b200/codegen/uvu.py``);
* 'uvw' paths: ``e3b_dense_fwd`` (fp32) or the tcgen05 tensor-core kernels (``math_mode='tf32'`` / ``'tf32x3'``);
* the other six modes (``_codegen.py:188-311``: 'uuu', 'uvuv', 'uvv', 'uuw', 'uvu<v', 'u<vw'): the channel pairs the mode
  couples become rows of a multiplicity-one 'uvu' product of the two irreps, evaluated by that product's generated
  module; the mode's weights follow (per pair, a sum over u, or a channel-mixing contraction on the Linear kernels).
  The slices and index selections around the kernels are torch operations.
"""
from __future__ import annotations

from math import prod
from typing import Iterator, List, Optional, Union

import numpy as np
import warnings

import torch

from .. import _lib
from ._dense_plan import uvw_plan
from ._irreps import Irreps
from ._spec import SUPPORTED_MODES, Instruction, TPSpec, normalize_tp_instructions


class _UvuFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x1, x2, w, mod, w_shared: bool, other_weights: bool = False):
        Z = x1.shape[0]
        out = torch.empty(Z, mod.dout, dtype=torch.float32, device=x1.device)
        with torch.cuda.device(x1.device):
            rc = mod.lib.e3b_uvu_fwd(_lib._ptr(x1), _lib._ptr(x2), _lib._ptr(w), _lib._ptr(out), Z, int(w_shared),
                                     _lib.stream_ptr())
        mod.check(rc, "e3b_uvu_fwd")
        ctx.save_for_backward(x1, x2, w)
        ctx.mod, ctx.w_shared, ctx.other_weights = mod, w_shared, other_weights
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out):
        x1, x2, w = ctx.saved_tensors
        mod = ctx.mod
        grad_out = grad_out.contiguous()
        # per-row weights: the kernel stores only the entries of its own paths; the entries of paths other engines
        # handle must read zero (shared weights are zeroed by the entry point itself)
        g1, g2 = torch.empty_like(x1), torch.empty_like(x2)
        gw = torch.zeros_like(w) if (ctx.other_weights and not ctx.w_shared) else torch.empty_like(w)
        with torch.cuda.device(x1.device):
            rc = mod.lib.e3b_uvu_bwd(_lib._ptr(x1), _lib._ptr(x2), _lib._ptr(w), _lib._ptr(grad_out), _lib._ptr(g1),
                                     _lib._ptr(g2), _lib._ptr(gw), x1.shape[0], int(ctx.w_shared), _lib.stream_ptr())
        mod.check(rc, "e3b_uvu_bwd")
        return g1, g2, gw, None, None, None


class _UvwFunction(torch.autograd.Function):
    """Weight-shared or per-row 'uvw' paths: forward on the engine the module's ``math_mode`` selects; gradients
    w.r.t. the two operands as two derived 'uvw' products of the cotangent (``TensorProduct._vjp_module``), w.r.t.
    shared weights by ``e3b_dense_bwd_w``, w.r.t. per-row weights by ``TensorProduct._uvw_row_weight_grad``."""

    @staticmethod
    def forward(ctx, x1, x2, w, out, tp, accumulate: bool):
        tp._uvw_run(x1, x2, w, out, accumulate)
        ctx.mark_dirty(out)
        ctx.save_for_backward(x1, x2, w)
        ctx.tp, ctx.accumulate = tp, accumulate
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out):
        x1, x2, w = ctx.saved_tensors
        tp = ctx.tp
        need1, need2, needw = ctx.needs_input_grad[:3]
        g = grad_out.contiguous()
        g1 = g2 = gw = None
        with torch.no_grad():
            if need1:
                g1 = tp._vjp_module(0)(g, x2, tp._vjp_weights(0, w))
            if need2:
                g2 = tp._vjp_module(1)(x1, g, tp._vjp_weights(1, w))
            if needw and not tp.shared_weights:
                gw = tp._uvw_row_weight_grad(x1, x2, g, w)
            elif needw:
                gw = torch.zeros_like(w)
                with torch.cuda.device(g.device):
                    rc = _lib.core().e3b_dense_bwd_w(tp._plan_host.ctypes.data, _lib._ptr(tp._plan_on(g.device)), _lib._ptr(x1),
                                                     _lib._ptr(x2), _lib._ptr(g), _lib._ptr(gw), x1.shape[0], _lib.stream_ptr())
                _lib.check(rc, "e3b_dense_bwd_w")
        return g1, g2, gw, (grad_out if ctx.accumulate else None), None, None


class TensorProduct(torch.nn.Module):
    """Tensor product with parametrised paths ('uvu' and 'uvw' connection modes)."""

    def __init__(
        self,
        irreps_in1,
        irreps_in2,
        irreps_out,
        instructions: List[tuple],
        in1_var=None,
        in2_var=None,
        out_var=None,
        irrep_normalization: str = None,
        path_normalization: str = None,
        internal_weights: Optional[bool] = None,
        shared_weights: Optional[bool] = None,
        compile_left_right: bool = True,
        compile_right: bool = False,
        normalization=None,
        _specialized_code: Optional[bool] = None,
        _optimize_einsums: Optional[bool] = None,
        math_mode: str = "fp32",
    ) -> None:
        super().__init__()
        if normalization is not None:
            irrep_normalization = normalization
        if irrep_normalization is None:
            irrep_normalization = "component"
        if path_normalization is None:
            path_normalization = "element"
        if compile_right:
            raise NotImplementedError("TensorProduct.right() is not part of the accelerated path")
        # 'fp32': CUDA-core kernels (<= 1e-5 x RMS); 'tf32x3' / 'tf32': tensor cores for the 'uvw' paths with
        # hi/lo-split (about 3e-5 x RMS) or plain (<= 2e-2 x RMS) tf32 operands.  'uvu' paths are always fp32.
        assert math_mode in ("fp32", "tf32x3", "tf32")
        self.math_mode = math_mode

        self.irreps_in1 = Irreps(irreps_in1)
        self.irreps_in2 = Irreps(irreps_in2)
        self.irreps_out = Irreps(irreps_out)
        self.instructions = normalize_tp_instructions(
            self.irreps_in1, self.irreps_in2, self.irreps_out, instructions, in1_var, in2_var, out_var,
            irrep_normalization, path_normalization,
        )
        for ins in self.instructions:
            if ins.connection_mode not in SUPPORTED_MODES:
                raise NotImplementedError(
                    f"connection mode '{ins.connection_mode}' is not implemented by e3nn_b200 "
                )
            if ins.connection_mode == "uvu":
                assert self.irreps_in1[ins.i_in1].mul == self.irreps_out[ins.i_out].mul
            if ins.connection_mode == "uvw":
                assert ins.has_weight
            if ins.connection_mode == "uuu":
                assert self.irreps_in1[ins.i_in1].mul == self.irreps_in2[ins.i_in2].mul == self.irreps_out[ins.i_out].mul
            if ins.connection_mode == "uvuv":
                assert self.irreps_in1[ins.i_in1].mul * self.irreps_in2[ins.i_in2].mul == self.irreps_out[ins.i_out].mul
            if ins.connection_mode == "uvv":
                assert self.irreps_in2[ins.i_in2].mul == self.irreps_out[ins.i_out].mul
            if ins.connection_mode in ("uuw", "uvu<v", "u<vw"):
                assert self.irreps_in1[ins.i_in1].mul == self.irreps_in2[ins.i_in2].mul
            if ins.connection_mode == "uuw" and not ins.has_weight:
                assert self.irreps_out[ins.i_out].mul == 1
            if ins.connection_mode == "uvu<v":
                m = self.irreps_in1[ins.i_in1].mul
                assert m * (m - 1) // 2 == self.irreps_out[ins.i_out].mul
            if ins.connection_mode == "u<vw":
                assert ins.has_weight

        self._in1_dim, self._in2_dim = self.irreps_in1.dim, self.irreps_in2.dim

        if shared_weights is False and internal_weights is None:
            internal_weights = False
        if shared_weights is None:
            shared_weights = True
        if internal_weights is None:
            internal_weights = shared_weights and any(i.has_weight for i in self.instructions)
        assert shared_weights or not internal_weights
        self.internal_weights = internal_weights
        self.shared_weights = shared_weights

        self.weight_numel = sum(prod(ins.path_shape) for ins in self.instructions if ins.has_weight)
        if internal_weights and self.weight_numel > 0:
            assert self.shared_weights, "Having internal weights impose shared weights"
            self.weight = torch.nn.Parameter(torch.randn(self.weight_numel))
        else:
            self.register_buffer("weight", torch.Tensor())

        if self.irreps_out.dim > 0:
            output_mask = torch.cat(
                [
                    torch.ones(mul * ir.dim)
                    if any(
                        (ins.i_out == i_out) and (ins.path_weight != 0) and (0 not in ins.path_shape)
                        for ins in self.instructions
                    )
                    else torch.zeros(mul * ir.dim)
                    for i_out, (mul, ir) in enumerate(self.irreps_out)
                ]
            )
        else:
            output_mask = torch.ones(0)
        self.register_buffer("output_mask", output_mask)

        self._spec = TPSpec(self.irreps_in1, self.irreps_in2, self.irreps_out, tuple(self.instructions), shared_weights)
        self._uvw_ids = [n for n, ins in self._spec.live_instructions() if ins.connection_mode == "uvw"]
        self._has_uvu = any(ins.connection_mode == "uvu" for _, ins in self._spec.live_instructions())
        self._uuu_ids = [n for n, ins in self._spec.live_instructions() if ins.connection_mode not in ("uvu", "uvw")]
        self._uuu_mods = {}
        self._plan_host = None
        self._plan_dev = {}
        if self._uvw_ids:
            self._plan_host, self._uvw_written = uvw_plan(self._spec)

    def __repr__(self) -> str:
        npath = sum(prod(i.path_shape) for i in self.instructions)
        return (
            f"{self.__class__.__name__}"
            f"({self.irreps_in1.simplify()} x {self.irreps_in2.simplify()} "
            f"-> {self.irreps_out.simplify()} | {npath} paths | {self.weight_numel} weights)"
        )

    # ---- weights (e3nn/o3/_tensor_product/_tensor_product.py:441-468) ------------------------
    def _prep_weights_python(self, weight):
        if isinstance(weight, list):
            weight_shapes = [ins.path_shape for ins in self.instructions if ins.has_weight]
            if not self.shared_weights:
                weight = [w.reshape(-1, prod(shape)) for w, shape in zip(weight, weight_shapes)]
            else:
                weight = [w.reshape(prod(shape)) for w, shape in zip(weight, weight_shapes)]
            return torch.cat(weight, dim=-1)
        return weight

    def _get_weights(self, weight) -> torch.Tensor:
        weight = self._prep_weights_python(weight)
        if weight is None:
            if self.weight_numel > 0 and not self.internal_weights:
                raise RuntimeError("Weights must be provided when the TensorProduct does not have `internal_weights`")
            return self.weight
        if self.shared_weights:
            torch._assert(weight.shape == (self.weight_numel,), "Invalid weight shape")
        else:
            torch._assert(weight.shape[-1] == self.weight_numel, "Invalid weight shape")
            torch._assert(weight.ndim > 1, "When shared weights is false, weights must have batch dimension")
        return weight

    def weight_view_for_instruction(self, instruction: int, weight: Optional[torch.Tensor] = None) -> torch.Tensor:
        if not self.instructions[instruction].has_weight:
            raise ValueError(f"Instruction {instruction} has no weights.")
        offset = sum(prod(ins.path_shape) for ins in self.instructions[:instruction] if ins.has_weight)
        ins = self.instructions[instruction]
        weight = self._get_weights(weight)
        batchshape = weight.shape[:-1]
        return weight.narrow(-1, offset, prod(ins.path_shape)).view(batchshape + ins.path_shape)

    def weight_views(self, weight: Optional[torch.Tensor] = None, yield_instruction: bool = False):
        weight = self._get_weights(weight)
        batchshape = weight.shape[:-1]
        offset = 0
        for ins_i, ins in enumerate(self.instructions):
            if ins.has_weight:
                flatsize = prod(ins.path_shape)
                this_weight = weight.narrow(-1, offset, flatsize).view(batchshape + ins.path_shape)
                offset += flatsize
                if yield_instruction:
                    yield ins_i, ins, this_weight
                else:
                    yield this_weight

    # ---- forward --------------------------------------------------------------------------
    def _uvu_module(self):
        return _lib.uvu_layout_module(self._uvu_only_spec())

    def _uvu_only_spec(self) -> TPSpec:
        if not hasattr(self, "_uvu_only"):
            # 'uvw' instructions are replaced by dead place-holders (zero path weight is not enough: the
            # generator skips them by mode), keeping the flat weight offsets of the 'uvu' paths.
            self._uvu_only = _UvuView(self._spec)
        return self._uvu_only

    def _plan_on(self, device) -> torch.Tensor:
        key = str(device)
        if key not in self._plan_dev:
            self._plan_dev[key] = torch.from_numpy(self._plan_host).to(device)
        return self._plan_dev[key]

    def forward(self, x, y, weight: Optional[torch.Tensor] = None):
        torch._assert(x.shape[-1] == self._in1_dim, "Incorrect last dimension for x")
        torch._assert(y.shape[-1] == self._in2_dim, "Incorrect last dimension for y")
        w = self._get_weights(weight)
        _lib.require_same_device(x, y, w if w.numel() > 0 else None)
        _lib.poll_status(x.device)
        for t in (x, y, w):
            if t.numel() > 0 and t.dtype != torch.float32:
                raise TypeError(f"e3nn_b200 tensor products are fp32 only, got {t.dtype}")

        # broadcast the leading dims (e3nn/o3/_tensor_product/_codegen.py:43-71)
        lead_shapes = [x.shape[:-1], y.shape[:-1]]
        if not self.shared_weights:
            lead_shapes.append(w.shape[:-1])
        lead = torch.broadcast_shapes(*lead_shapes)
        Z = int(np.prod(lead)) if len(lead) > 0 else 1
        out_dim = self.irreps_out.dim
        if Z == 0 or out_dim == 0:
            return x.new_zeros(*lead, out_dim)
        x2d = x.expand(*lead, self._in1_dim).reshape(Z, self._in1_dim).contiguous()
        y2d = y.expand(*lead, self._in2_dim).reshape(Z, self._in2_dim).contiguous()
        if self.shared_weights:
            w2d = w.contiguous()
        else:
            w2d = w.expand(*lead, self.weight_numel).reshape(Z, self.weight_numel).contiguous()
        if w2d.numel() == 0:
            w2d = x2d.new_zeros(1)

        if self._has_uvu:
            out = _UvuFunction.apply(x2d, y2d, w2d, self._uvu_module(), self.shared_weights, bool(self._uvw_ids or self._uuu_ids))
        elif self._uvw_ids and not self._uuu_ids:
            out = torch.empty(Z, out_dim, dtype=torch.float32, device=x.device)
            self._zero_unwritten(out)
        else:
            out = x2d.new_zeros(Z, out_dim)
        if self._uvw_ids:
            out = self._uvw_forward(x2d, y2d, w2d, out, accumulate=self._has_uvu)
        if self._uuu_ids:
            out = self._uuu_forward(x2d, y2d, w2d, out)
        return out.reshape(*lead, out_dim)

    def _uuu_sub(self, n: int) -> "TensorProduct":
        """The multiplicity-one 'uvu' product that evaluates 'uuu' instruction ``n`` on (row, channel) pairs."""
        ins = self.instructions[n]
        ir1, ir2, ir3 = self.irreps_in1[ins.i_in1].ir, self.irreps_in2[ins.i_in2].ir, self.irreps_out[ins.i_out].ir
        key = (str(ir1), str(ir2), str(ir3), float(ins.path_weight))
        if key not in self._uuu_mods:
            # 'none' normalisations: the final coefficient is sqrt(path_weight argument)
            self._uuu_mods[key] = TensorProduct(f"1x{ir1}", f"1x{ir2}", f"1x{ir3}", [(0, 0, 0, "uvu", False, ins.path_weight ** 2)],
                                                irrep_normalization="none", path_normalization="none")
        return self._uuu_mods[key]

    def _uuu_forward(self, x2d, y2d, w, out):
        """Paths whose channels pair up one to one before any weight is applied ('uuu', 'uvuv', 'uvv', 'uuw', 'uvu<v',
        'u<vw'): t[z, q, :] = pw * x1[z, u(q), :] (x) x2[z, v(q), :] with the (z, q) pairs as rows of a multiplicity-one
        product, then the mode's weights: per pair ('uuu', 'uvuv', 'uvu<v'), summed over u ('uvv'), or a channel-mixing
        contraction over q on the Linear kernels ('uuw', 'u<vw')."""
        Z = x2d.shape[0]
        o1, o2, oo = self.irreps_in1.offsets(), self.irreps_in2.offsets(), self.irreps_out.offsets()
        woffs = self._spec.weight_offsets()
        for n in self._uuu_ids:
            ins = self.instructions[n]
            (m1, ir1), (m2, ir2), (mo, ir3) = self.irreps_in1[ins.i_in1], self.irreps_in2[ins.i_in2], self.irreps_out[ins.i_out]
            mode = ins.connection_mode
            xa = x2d[:, o1[ins.i_in1] : o1[ins.i_in1] + m1 * ir1.dim].reshape(Z, m1, ir1.dim)
            xb = y2d[:, o2[ins.i_in2] : o2[ins.i_in2] + m2 * ir2.dim].reshape(Z, m2, ir2.dim)
            if mode in ("uuu", "uuw"):
                a, b, P = xa, xb, m1
            elif mode in ("uvuv", "uvv"):       # all pairs, q = u * m2 + v
                P = m1 * m2
                a = xa.unsqueeze(2).expand(Z, m1, m2, ir1.dim)
                b = xb.unsqueeze(1).expand(Z, m1, m2, ir2.dim)
            else:                                # 'uvu<v', 'u<vw': the pairs u < v in row-major order
                iu, iv = torch.triu_indices(m1, m1, 1, device=x2d.device)
                a, b, P = xa[:, iu], xb[:, iv], iu.numel()
            t = self._uuu_sub(n)(a.reshape(Z * P, ir1.dim), b.reshape(Z * P, ir2.dim)).view(Z, P, ir3.dim)
            wn = prod(ins.path_shape) if ins.has_weight else 0
            wp = None
            if ins.has_weight:
                wp = w[woffs[n] : woffs[n] + wn] if self.shared_weights else w[:, woffs[n] : woffs[n] + wn]
            if mode in ("uuu", "uvuv", "uvu<v"):
                r = t * (wp.view(1, P, 1) if self.shared_weights else wp.unsqueeze(-1)) if ins.has_weight else t
            elif mode == "uvv":
                t4 = t.view(Z, m1, m2, ir3.dim)
                if ins.has_weight:
                    t4 = t4 * (wp.view(1, m1, m2, 1) if self.shared_weights else wp.view(Z, m1, m2, 1))
                r = t4.sum(1)
            elif not ins.has_weight:             # 'uuw' without weights: the sum over u (one output channel)
                r = t.sum(1, keepdim=True)
            elif self.shared_weights:            # out[z, w, :] = sum_q W[q, w] t[z, q, :] on the Linear kernels
                key = ("mix", P, mo, str(ir3))
                if key not in self._uuu_mods:
                    from ._linear import Linear

                    self._uuu_mods[key] = Linear(f"{P}x{ir3}", f"{mo}x{ir3}", internal_weights=False, shared_weights=True)
                r = self._uuu_mods[key](t.reshape(Z, P * ir3.dim), wp * P ** 0.5)     # (undoes its fan-in factor)
            else:
                r = torch.einsum("zqw,zqk->zwk", wp.view(Z, P, mo), t)
            sl = slice(oo[ins.i_out], oo[ins.i_out] + mo * ir3.dim)
            out[:, sl] += r.reshape(Z, mo * ir3.dim)
        return out

    def _zero_unwritten(self, out: torch.Tensor) -> None:
        offs = self.irreps_out.offsets()
        for i_out, (mul, ir) in enumerate(self.irreps_out):
            if i_out not in self._uvw_written and mul * ir.dim > 0:
                with torch.cuda.device(out.device):
                    rc = _lib.core().e3b_fill_columns(_lib._ptr(out), out.shape[0], out.shape[1], offs[i_out],
                                                      mul * ir.dim, None, 0, _lib.stream_ptr())
                _lib.check(rc, "e3b_fill_columns")

    def _uvw_forward(self, x2d, y2d, w, out, accumulate: bool):
        if torch.is_grad_enabled() and (x2d.requires_grad or y2d.requires_grad or w.requires_grad or out.requires_grad):
            return _UvwFunction.apply(x2d, y2d, w, out, self, accumulate)
        return self._uvw_run(x2d, y2d, w, out, accumulate)

    def _uvw_run(self, x2d, y2d, w, out, accumulate: bool):
        """The 'uvw' paths on the engine of ``math_mode`` (no autograd bookkeeping)."""
        if self.math_mode == "tf32":
            from ._uvw_tc import tc_eligible, uvw_tc_forward

            if not hasattr(self, "_tc_ok"):
                self._tc_ok = tc_eligible(self)     # planning the groups costs a fraction of a millisecond: once
            if self._tc_ok:
                return uvw_tc_forward(self, x2d, y2d, w, out, accumulate)
            if not getattr(self, "_warned_tc", False):
                warnings.warn(f"{self}: layout not eligible for the tensor-core kernel, using the fp32 kernel")
                self._warned_tc = True
        if self.math_mode == "tf32x3" and self.shared_weights and not accumulate:
            # tensor cores with hi/lo-split tf32 operands when the layout fits the kernel
            if not hasattr(self, "_tcg_spec"):
                from ..codegen import tc_gemm

                self._tcg_spec = tc_gemm.uvw_gemm_spec(self._spec)
            if self._tcg_spec is not None:
                mod = _lib.tc_gemm_module(self._tcg_spec)
                mod.run(x2d, y2d, w, out, 2)
                return out
        w_row_stride = w.shape[1] if w.dim() == 2 else 0
        with torch.cuda.device(x2d.device):
            rc = _lib.core().e3b_dense_fwd(self._plan_host.ctypes.data, _lib._ptr(self._plan_on(x2d.device)), _lib._ptr(x2d),
                                           _lib._ptr(y2d), _lib._ptr(w), w_row_stride, _lib._ptr(out), x2d.shape[0],
                                           int(accumulate), _lib.stream_ptr())
        _lib.check(rc, "e3b_dense_fwd")
        return out

    # ---- gradients of the 'uvw' paths w.r.t. the operands -----------------------------------------------
    # The product is trilinear, so its transpose in one operand is again a 'uvw' product: of the cotangent and
    # the other operand, with each path's weights permuted and the same coefficient (the real 3j symbols of a
    # permuted triple are equal up to a sign, which goes into the weights).
    def _vjp_module(self, which: int) -> "TensorProduct":
        if not hasattr(self, "_vjp"):
            self._vjp = {}
        if which not in self._vjp:   # (the derived module shares weights exactly when this one does)
            from ._wigner import wigner_3j_numpy

            instr, signs = [], []
            for n in self._uvw_ids:
                ins = self.instructions[n]
                l1, l2, l3 = (self.irreps_in1[ins.i_in1].ir.l, self.irreps_in2[ins.i_in2].ir.l, self.irreps_out[ins.i_out].ir.l)
                c = wigner_3j_numpy(l1, l2, l3)
                if which == 0:    # d/dx1: (cotangent, x2) -> x1 slots
                    instr.append((ins.i_out, ins.i_in2, ins.i_in1, "uvw", True, ins.path_weight ** 2))
                    signs.append(float(np.sum(wigner_3j_numpy(l3, l2, l1) * c.transpose(2, 1, 0))))
                else:             # d/dx2: (x1, cotangent) -> x2 slots
                    instr.append((ins.i_in1, ins.i_out, ins.i_in2, "uvw", True, ins.path_weight ** 2))
                    signs.append(float(np.sum(wigner_3j_numpy(l1, l3, l2) * c.transpose(0, 2, 1))))
            ins_ = (self.irreps_out, self.irreps_in2, self.irreps_in1) if which == 0 else (self.irreps_in1, self.irreps_out, self.irreps_in2)
            mod = TensorProduct(*ins_, instr, irrep_normalization="none", path_normalization="none", internal_weights=False,
                                shared_weights=self.shared_weights, math_mode=self.math_mode)
            mod._vjp_signs = [1.0 if s > 0 else -1.0 for s in signs]
            mod._warned_tc = True     # a derived layout that misses the tensor-core kernel falls back to fp32 silently
            self._vjp[which] = mod
        return self._vjp[which]

    def _uvw_row_weight_grad(self, x1, x2, g, w) -> torch.Tensor:
        """Cotangent of per-row 'uvw' weights: grad[z, u, v, w] = sum_k t[z, (u, v), k] g[z, w, k], where t is the
        coupled pair product of the path (coefficient included), formed on the (z, u, v) rows of a multiplicity-one
        'uvu' module; the sum over k is one batched product."""
        Z = x1.shape[0]
        o1, o2, oo = self.irreps_in1.offsets(), self.irreps_in2.offsets(), self.irreps_out.offsets()
        offs = self._spec.weight_offsets()
        gw = torch.zeros_like(w)
        for n in self._uvw_ids:
            ins = self.instructions[n]
            (m1, ir1), (m2, ir2), (mo, ir3) = self.irreps_in1[ins.i_in1], self.irreps_in2[ins.i_in2], self.irreps_out[ins.i_out]
            a = x1[:, o1[ins.i_in1] : o1[ins.i_in1] + m1 * ir1.dim].reshape(Z, m1, 1, ir1.dim).expand(Z, m1, m2, ir1.dim)
            b = x2[:, o2[ins.i_in2] : o2[ins.i_in2] + m2 * ir2.dim].reshape(Z, 1, m2, ir2.dim).expand(Z, m1, m2, ir2.dim)
            t = self._uuu_sub(n)(a.reshape(Z * m1 * m2, ir1.dim), b.reshape(Z * m1 * m2, ir2.dim)).view(Z, m1 * m2, ir3.dim)
            gk = g[:, oo[ins.i_out] : oo[ins.i_out] + mo * ir3.dim].reshape(Z, mo, ir3.dim)
            gw[:, offs[n] : offs[n] + m1 * m2 * mo] = torch.bmm(t, gk.transpose(1, 2)).reshape(Z, -1)
        return gw

    def _vjp_weights(self, which: int, w: torch.Tensor) -> torch.Tensor:
        """Flat weights of `_vjp_module(which)`: per 'uvw' path [u, v, w] -> [w, v, u] (which = 0) or [u, w, v]."""
        signs = self._vjp_module(which)._vjp_signs
        offs = self._spec.weight_offsets()
        parts = []
        for n, sgn in zip(self._uvw_ids, signs):
            ins = self.instructions[n]
            block = w[..., offs[n] : offs[n] + prod(ins.path_shape)]
            view = block.reshape(block.shape[:-1] + tuple(ins.path_shape))
            view = view.transpose(-1, -3) if which == 0 else view.transpose(-1, -2)
            parts.append((view * sgn).reshape(block.shape[:-1] + (-1,)))
        return torch.cat(parts, dim=-1) if parts else w.new_zeros(0)


class _UvuView(TPSpec):
    """A `TPSpec` whose generator-visible paths are the 'uvu' ones of another spec."""

    def __init__(self, spec: TPSpec):
        object.__setattr__(self, "irreps_in1", spec.irreps_in1)
        object.__setattr__(self, "irreps_in2", spec.irreps_in2)
        object.__setattr__(self, "irreps_out", spec.irreps_out)
        object.__setattr__(self, "instructions", spec.instructions)
        object.__setattr__(self, "shared_weights", spec.shared_weights)

    def live_instructions(self):
        return [(n, ins) for n, ins in TPSpec.live_instructions(self) if ins.connection_mode == "uvu"]


class FullyConnectedTensorProduct(TensorProduct):
    """All allowed 'uvw' paths between the three layouts (``_sub.py:10-68``)."""

    def __init__(self, irreps_in1, irreps_in2, irreps_out, irrep_normalization: str = None,
                 path_normalization: str = None, **kwargs) -> None:
        irreps_in1, irreps_in2, irreps_out = Irreps(irreps_in1), Irreps(irreps_in2), Irreps(irreps_out)
        instr = [
            (i_1, i_2, i_out, "uvw", True, 1.0)
            for i_1, (_, ir_1) in enumerate(irreps_in1)
            for i_2, (_, ir_2) in enumerate(irreps_in2)
            for i_out, (_, ir_out) in enumerate(irreps_out)
            if ir_out in ir_1 * ir_2
        ]
        super().__init__(irreps_in1, irreps_in2, irreps_out, instr, irrep_normalization=irrep_normalization,
                         path_normalization=path_normalization, **kwargs)


class ElementwiseTensorProduct(TensorProduct):
    """Channel-by-channel product ``z_u = x_u (x) y_u`` without weights (``_sub.py:69-133``).

    The two layouts are cut into blocks of equal multiplicity; every block pair contributes one 'uuu' path per
    irrep of its product (optionally filtered by ``filter_ir_out``)."""

    def __init__(self, irreps_in1, irreps_in2, filter_ir_out=None, irrep_normalization: str = None, **kwargs) -> None:
        from ._irreps import Irrep

        a, b = Irreps(irreps_in1).simplify(), Irreps(irreps_in2).simplify()
        if filter_ir_out is not None:
            try:
                filter_ir_out = [Irrep(ir) for ir in filter_ir_out]
            except ValueError:
                raise ValueError(f"filter_ir_out (={filter_ir_out}) must be an iterable of e3nn.o3.Irrep")
        assert a.num_irreps == b.num_irreps
        # walk both layouts with one cursor each, emitting the common part of the two current blocks
        blocks1, blocks2 = [], []
        ia = ib = 0
        left_a = a[0].mul if len(a) else 0
        left_b = b[0].mul if len(b) else 0
        while ia < len(a) and ib < len(b):
            m = min(left_a, left_b)
            if m > 0:
                blocks1.append((m, a[ia].ir))
                blocks2.append((m, b[ib].ir))
            left_a -= m
            left_b -= m
            if left_a == 0:
                ia += 1
                left_a = a[ia].mul if ia < len(a) else 0
            if left_b == 0:
                ib += 1
                left_b = b[ib].mul if ib < len(b) else 0
        out, instr = [], []
        for n, ((mul, ir1), (_, ir2)) in enumerate(zip(blocks1, blocks2)):
            for ir in ir1 * ir2:
                if filter_ir_out is not None and ir not in filter_ir_out:
                    continue
                instr.append((n, n, len(out), "uuu", False))
                out.append((mul, ir))
        super().__init__(Irreps(blocks1), Irreps(blocks2), Irreps(out), instr, irrep_normalization=irrep_normalization, **kwargs)


class FullTensorProduct(TensorProduct):
    """Every pair of channels, ``z_uv = x_u (x) y_v``, without weights (``_sub.py:136-205``): one 'uvuv' path per
    pair of input irreps and irrep of their product, the output layout sorted by (l, p)."""

    def __init__(self, irreps_in1, irreps_in2, filter_ir_out=None, irrep_normalization: str = None, **kwargs) -> None:
        from ._irreps import Irrep

        a, b = Irreps(irreps_in1).simplify(), Irreps(irreps_in2).simplify()
        if filter_ir_out is not None:
            try:
                filter_ir_out = [Irrep(ir) for ir in filter_ir_out]
            except ValueError:
                raise ValueError(f"filter_ir_out (={filter_ir_out}) must be an iterable of e3nn.o3.Irrep")
        pairs = [(n1, n2, m1 * m2, ir) for n1, (m1, ir1) in enumerate(a) for n2, (m2, ir2) in enumerate(b) for ir in ir1 * ir2
                 if filter_ir_out is None or ir in filter_ir_out]
        out, position, _ = Irreps([(m, ir) for _, _, m, ir in pairs]).sort()
        instr = [(n1, n2, position[n], "uvuv", False) for n, (n1, n2, _, _) in enumerate(pairs)]
        super().__init__(a, b, out, instr, irrep_normalization=irrep_normalization, **kwargs)


def _square_alpha(ir_in, ir_out, normalization: str, diagonal: bool) -> float:
    """Variance factor of one path of a tensor square (``_sub.py:238-275``).  ``diagonal``: the u == v part, whose
    symmetric product has a different second moment than a product of independent channels."""
    if normalization == "none":
        return 1.0
    if not diagonal:
        return float(ir_out.dim) if normalization == "component" else float(ir_in[0].dim * ir_in[1].dim)
    d = ir_in[0].dim
    if normalization == "component":
        return ir_out.dim / (d + 2) if ir_out.l == 0 else ir_out.dim / 2
    return float(ir_out.dim * d) if ir_out.l == 0 else d * (d + 2) / 2


class TensorSquare(TensorProduct):
    """``x (x) x`` reduced into irreps (``_sub.py:208-420``).  A pair of different input blocks contributes once; within a
    block the pairs u < v and, for even l, the diagonal u == v.  Without ``irreps_out`` nothing is weighted and the
    output lists every product ('uvuv', 'uvu<v', 'uuu' paths, sorted by (l, p)); with ``irreps_out`` the same three
    kinds of pairs are mixed into the given channels by weights ('uvw', 'u<vw', 'uuw')."""

    def __init__(self, irreps_in, irreps_out=None, filter_ir_out=None, irrep_normalization: str = None, **kwargs) -> None:
        from ._irreps import Irrep

        if irrep_normalization is None:
            irrep_normalization = "component"
        assert irrep_normalization in ["component", "norm", "none"]
        irreps_in = Irreps(irreps_in).simplify()
        if filter_ir_out is not None:
            try:
                filter_ir_out = [Irrep(ir) for ir in filter_ir_out]
            except ValueError as exc:
                raise ValueError(f"Error constructing filter_ir_out irrep: {exc}") from exc
        if irreps_out is not None and filter_ir_out is not None:
            raise ValueError("Both `irreps_out` and `filter_ir_out` are not None, this is ambiguous.")
        connected = irreps_out is not None
        if connected:
            irreps_out = Irreps(irreps_out).simplify()
        instr = []
        if connected:
            # the reference walks the output slots inside each block pair: (pairs, diag) alternate per slot
            for n1, (m1, ir1) in enumerate(irreps_in):
                for n2 in range(n1, len(irreps_in)):
                    ir2 = irreps_in[n2].ir
                    for n_out, (_, ir_o) in enumerate(irreps_out):
                        if ir_o not in ir1 * ir2:
                            continue
                        if n1 < n2:
                            instr.append((n1, n2, n_out, "uvw", True, _square_alpha((ir1, ir2), ir_o, irrep_normalization, False)))
                            continue
                        if m1 > 1:
                            instr.append((n1, n1, n_out, "u<vw", True, _square_alpha((ir1, ir1), ir_o, irrep_normalization, False)))
                        if ir_o.l % 2 == 0:
                            instr.append((n1, n1, n_out, "uuw", True, _square_alpha((ir1, ir1), ir_o, irrep_normalization, True)))
        else:
            produced = []     # (mul, ir) of every product, in the order of the instructions

            def emit(n1, n2, ir, mode, mul, diagonal=False):
                alpha = _square_alpha((irreps_in[n1].ir, irreps_in[n2].ir), ir, irrep_normalization, diagonal)
                instr.append((n1, n2, len(produced), mode, False, alpha))
                produced.append((mul, ir))

            for n1, (m1, ir1) in enumerate(irreps_in):
                for n2 in range(n1, len(irreps_in)):
                    m2, ir2 = irreps_in[n2]
                    for ir in ir1 * ir2:
                        if filter_ir_out is not None and ir not in filter_ir_out:
                            continue
                        if n1 < n2:
                            emit(n1, n2, ir, "uvuv", m1 * m2)
                            continue
                        if m1 > 1:
                            emit(n1, n1, ir, "uvu<v", m1 * (m1 - 1) // 2)
                        if ir.l % 2 == 0:
                            emit(n1, n1, ir, "uuu", m1, diagonal=True)
            irreps_out, position, _ = Irreps(produced).sort()
            instr = [(a, b, position[c], mode, hw, alpha) for a, b, c, mode, hw, alpha in instr]
        self.irreps_in = irreps_in
        super().__init__(irreps_in, irreps_in, irreps_out, instr, irrep_normalization="none", **kwargs)

    def __repr__(self) -> str:
        npath = sum(prod(i.path_shape) for i in self.instructions)
        return f"{self.__class__.__name__}({self.irreps_in} -> {self.irreps_out.simplify()} | {npath} paths | {self.weight_numel} weights)"

    def forward(self, x, weight: Optional[torch.Tensor] = None):
        return super().forward(x, x, weight)
