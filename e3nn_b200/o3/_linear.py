"""Drop-in ``Linear``: per-irrep channel mixing (``e3nn/o3/_linear.py:28-345``).

Same constructor, attributes (``weight``, ``bias``, ``weight_numel``, ``bias_numel``,
``output_mask``, ``instructions``), weight layout and error types as the reference.  The
contraction runs in ``e3b_dense_fwd`` (fp32) or the tensor-core module; the gradient w.r.t. the features
reuses the same kernels with a transposed plan, the gradient w.r.t. the weights is ``e3b_dense_bwd_w`` (fp32),
the gradient w.r.t. the biases a column sum.  ``f_in`` / ``f_out`` and per-row weights are not implemented.
"""
from __future__ import annotations

from math import prod
from typing import List, NamedTuple, Optional, Tuple, Union

import torch

import hashlib

from .. import _lib
from ..codegen import tc_gemm
from ._dense_plan import linear_plan
from ._irreps import Irreps
from ._spec import LinearInstruction, normalize_linear_instructions


class LinearSlices(NamedTuple):
    slice: slice
    shape: Tuple[int, int]


class _LinearFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, lin):
        Z = x.shape[0]
        dev = x.device
        out = torch.empty(Z, lin.irreps_out.dim, dtype=torch.float32, device=dev)
        core = _lib.core()
        with torch.cuda.device(dev):
            s = _lib.stream_ptr()
            if lin._tc_fwd is None or lin._precision == 0:   # (the tensor-core module zero-fills by itself)
                for off, n in lin._unwritten:
                    _lib.check(core.e3b_fill_columns(_lib._ptr(out), Z, out.shape[1], off, n, None, 0, s), "e3b_fill_columns")
            if lin.weight_numel > 0 and lin._tc_fwd is not None and lin._precision > 0:
                    # tensor cores: hi/lo-split ('tf32x3') or plain ('tf32') tf32 operands
                _lib.tc_gemm_module(lin._tc_fwd).run(x, None, w, out, lin._precision)
            elif lin.weight_numel > 0:
                plan_dev = lin._plan_on(dev, False)
                rc = core.e3b_dense_fwd(lin._plan_host.ctypes.data, _lib._ptr(plan_dev), _lib._ptr(x), None,
                                        _lib._ptr(w), 0, _lib._ptr(out), Z, 0, s)
                _lib.check(rc, "e3b_dense_fwd")
            boff = 0
            for off, n, written in lin._bias_ranges:
                rc = core.e3b_fill_columns(_lib._ptr(out), Z, out.shape[1], off, n,
                                           bias.data_ptr() + 4 * boff, int(written), s)
                _lib.check(rc, "e3b_fill_columns")
                boff += n
        ctx.save_for_backward(x, w)
        ctx.lin = lin
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out):
        x, w = ctx.saved_tensors
        lin = ctx.lin
        grad_out = grad_out.contiguous()
        Z, dev = grad_out.shape[0], grad_out.device
        gx = gw = gb = None
        if ctx.needs_input_grad[1]:
            # dW[u, w] = pw * sum_{z, i} x[z, u, i] g[z, w, i]: the forward plan read the other way round (fp32)
            gw = torch.zeros_like(w)
            if lin.weight_numel > 0:
                with torch.cuda.device(dev):
                    rc = _lib.core().e3b_dense_bwd_w(lin._plan_host.ctypes.data, _lib._ptr(lin._plan_on(dev, False)),
                                                     _lib._ptr(x), None, _lib._ptr(grad_out), _lib._ptr(gw), Z,
                                                     _lib.stream_ptr())
                _lib.check(rc, "e3b_dense_bwd_w")
        if ctx.needs_input_grad[2]:
            parts = [grad_out[:, off : off + n].sum(0) for off, n, _ in lin._bias_ranges]
            gb = torch.cat(parts) if parts else torch.zeros(1, dtype=torch.float32, device=dev)
        if not ctx.needs_input_grad[0]:
            return None, gw, gb, None
        if lin.weight_numel > 0 and lin._tc_bwd is not None and lin._precision > 0:
            gx = torch.empty(Z, lin.irreps_in.dim, dtype=torch.float32, device=dev)
            _lib.tc_gemm_module(lin._tc_bwd).run(grad_out, None, w, gx, lin._precision)
            return gx, gw, gb, None
        gx = torch.zeros(Z, lin.irreps_in.dim, dtype=torch.float32, device=dev)
        if lin.weight_numel > 0:
            with torch.cuda.device(dev):
                rc = _lib.core().e3b_dense_fwd(lin._plan_t_host.ctypes.data, _lib._ptr(lin._plan_on(dev, True)),
                                               _lib._ptr(grad_out), None, _lib._ptr(w), 0, _lib._ptr(gx), Z, 1,
                                               _lib.stream_ptr())
            _lib.check(rc, "e3b_dense_fwd (transposed)")
        return gx, gw, gb, None


class Linear(torch.nn.Module):
    def __init__(
        self,
        irreps_in,
        irreps_out,
        *,
        f_in: Optional[int] = None,
        f_out: Optional[int] = None,
        internal_weights: Optional[bool] = None,
        shared_weights: Optional[bool] = None,
        instructions: Optional[List[Tuple[int, int]]] = None,
        biases: Union[bool, List[bool]] = False,
        path_normalization: str = "element",
        _optimize_einsums: Optional[bool] = None,
        math_mode: str = "fp32",
    ) -> None:
        super().__init__()
        # 'fp32': CUDA-core kernel (<= 1e-5 x RMS).  'tf32x3': tensor cores with hi/lo-split tf32 operands
        # (about 3e-5 x RMS).  'tf32': tensor cores, plain tf32 operands (<= 2e-2 x RMS).
        assert math_mode in ("fp32", "tf32x3", "tf32")
        self.math_mode = math_mode
        self._precision = {"fp32": 0, "tf32x3": 2, "tf32": 1}[math_mode]
        if f_in is not None or f_out is not None:
            raise NotImplementedError("Linear(f_in=..., f_out=...) is not implemented by e3nn_b200")
        irreps_in, irreps_out = Irreps(irreps_in), Irreps(irreps_out)
        self.instructions = normalize_linear_instructions(irreps_in, irreps_out, instructions, biases, None,
                                                          path_normalization)
        if shared_weights is False and internal_weights is None:
            internal_weights = False
        if shared_weights is None:
            shared_weights = True
        if internal_weights is None:
            internal_weights = True
        assert shared_weights or not internal_weights
        if not shared_weights:
            raise NotImplementedError("Linear with per-row weights is not implemented by e3nn_b200")
        self.internal_weights, self.shared_weights = internal_weights, shared_weights
        self.irreps_in, self.irreps_out = irreps_in, irreps_out

        live = [ins for ins in self.instructions if 0 not in ins.path_shape]
        self.weight_numel = sum(prod(ins.path_shape) for ins in live if ins.i_in != -1)
        self.bias_numel = sum(prod(ins.path_shape) for ins in live if ins.i_in == -1)
        # the flat weight vector skips empty instructions, exactly as the reference's code generator does
        packed = [ins if 0 not in ins.path_shape else ins._replace(path_shape=(0, 0)) for ins in self.instructions]
        self._plan_host, written = linear_plan(irreps_in, irreps_out, packed, transpose=False)
        self._plan_t_host, _ = linear_plan(irreps_in, irreps_out, packed, transpose=True)
        self._plan_dev = {}
        # tensor-core modules (None when the multiplicities do not fit the 32-wide K chunks / 16-wide N)
        tag = hashlib.sha1(repr((str(irreps_in), str(irreps_out), [(i.i_in, i.i_out, i.path_shape, repr(i.path_weight))
                                                                      for i in packed])).encode()).hexdigest()[:14]
        self._tc_fwd = tc_gemm.linear_gemm_spec(irreps_in, irreps_out, packed, False, "lin" + tag + "f")
        self._tc_bwd = tc_gemm.linear_gemm_spec(irreps_in, irreps_out, packed, True, "lin" + tag + "t")
        offs = irreps_out.offsets()
        bias_out = [ins.i_out for ins in self.instructions if ins.i_in == -1 and 0 not in ins.path_shape]
        self._unwritten = [
            (offs[i], mul * ir.dim) for i, (mul, ir) in enumerate(irreps_out)
            if i not in written and i not in bias_out and mul * ir.dim > 0
        ]
        self._bias_ranges = [(offs[i], irreps_out[i].dim, i in written) for i in bias_out]

        if internal_weights and self.weight_numel > 0:
            self.weight = torch.nn.Parameter(torch.randn(self.weight_numel))
        else:
            self.register_buffer("weight", torch.Tensor())
        if internal_weights and self.bias_numel > 0:
            self.bias = torch.nn.Parameter(torch.zeros(self.bias_numel))
        else:
            self.register_buffer("bias", torch.Tensor())

        if irreps_out.dim > 0:
            output_mask = torch.cat(
                [
                    torch.ones(mul_ir.dim)
                    if any((ins.i_out == i_out) and (0 not in ins.path_shape) for ins in self.instructions)
                    else torch.zeros(mul_ir.dim)
                    for i_out, mul_ir in enumerate(irreps_out)
                ]
            )
        else:
            output_mask = torch.ones(0)
        self.register_buffer("output_mask", output_mask)

        self.weight_index_slices = []
        for i, ins in enumerate(self.instructions):
            offset = sum(prod(p.path_shape) for p in self.instructions[:i])
            self.weight_index_slices.append(LinearSlices(slice(offset, offset + prod(ins.path_shape), None), ins.path_shape))

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}({self.irreps_in} -> {self.irreps_out} | {self.weight_numel} weights)"

    def _plan_on(self, device, transposed: bool) -> torch.Tensor:
        key = (str(device), transposed)
        if key not in self._plan_dev:
            host = self._plan_t_host if transposed else self._plan_host
            self._plan_dev[key] = torch.from_numpy(host).to(device)
        return self._plan_dev[key]

    def forward(self, features, weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None):
        if weight is None:
            if self.weight_numel > 0 and not self.internal_weights:
                raise RuntimeError("Weights must be provided when internal_weights = False")
            weight = self.weight
        if bias is None:
            if self.bias_numel > 0 and not self.internal_weights:
                raise RuntimeError("Biases must be provided when internal_weights = False")
            bias = self.bias
        _lib.require_cuda(features)
        if features.dtype != torch.float32:
            raise TypeError(f"e3nn_b200 Linear is fp32 only, got {features.dtype}")
        torch._assert(features.shape[-1] == self.irreps_in.dim, "Incorrect last dimension for features")
        lead = features.shape[:-1]
        x = features.reshape(-1, self.irreps_in.dim).contiguous()
        if x.shape[0] == 0 or self.irreps_out.dim == 0:
            return features.new_zeros(*lead, self.irreps_out.dim)
        if self.weight_numel > 0:
            _lib.require_operand(weight, x, "weight", self.weight_numel)
        if self.bias_numel > 0:
            _lib.require_operand(bias, x, "bias", self.bias_numel)
        _lib.poll_status(x.device)
        w = weight.reshape(-1).contiguous() if self.weight_numel > 0 else x.new_zeros(1)
        b = bias.reshape(-1).contiguous() if self.bias_numel > 0 else x.new_zeros(1)
        out = _LinearFunction.apply(x, w, b, self)
        return out.reshape(*lead, self.irreps_out.dim)

    def weight_view_for_instruction(self, instruction: int, weight: Optional[torch.Tensor] = None) -> torch.Tensor:
        if weight is None:
            assert self.internal_weights, "Weights must be provided when internal_weights = False"
            weight = self.weight
        batchshape = weight.shape[:-1]
        offset = sum(prod(ins.path_shape) for ins in self.instructions[:instruction])
        ins = self.instructions[instruction]
        return weight.narrow(-1, offset, prod(ins.path_shape)).view(batchshape + ins.path_shape)

    def weight_views(self, weight: Optional[torch.Tensor] = None, yield_instruction: bool = False):
        if weight is None:
            assert self.internal_weights, "Weights must be provided when internal_weights = False"
            weight = self.weight
        batchshape = weight.shape[:-1]
        offset = 0
        for ins_i, ins in enumerate(self.instructions):
            flatsize = prod(ins.path_shape)
            this_weight = weight.narrow(-1, offset, flatsize).view(batchshape + ins.path_shape)
            offset += flatsize
            if yield_instruction:
                yield ins_i, ins, this_weight
            else:
                yield this_weight
