"""ctypes bindings of the C-ABI libraries (``include/e3nn_b200.h``, ``include/e3nn_b200_layout.h``).

There is no CPU or PyTorch fallback: if the CUDA library is missing, loading fails with an
error that says how to build it, and every op raises for tensors that are not on a CUDA device.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_void_p
from typing import Dict, Optional

import torch

from . import _build

_core = None
_core_lock = threading.Lock()
_layout_cache: Dict[str, "LayoutModule"] = {}


class E3BError(RuntimeError):
    pass


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def stream_ptr() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise NotImplementedError(
                "e3nn_b200 runs on CUDA (sm_100a) only: got a tensor on device "
                f"'{t.device}'. There is no CPU implementation in this package."
            )


def core() -> ctypes.CDLL:
    """The fixed-function library; built on first use when nvcc is present."""
    global _core
    if _core is not None:
        return _core
    with _core_lock:
        if _core is not None:
            return _core
        path = _build.CORE_LIB
        if not os.path.exists(path):
            if _build.nvcc_path() is None:
                raise E3BError(
                    f"{path} is missing and nvcc is not available to build it. "
                    "Build it with `python -c 'import __graft_entry__ as g; g.build()'` on a machine with CUDA 12.9."
                )
            _build.build_core()
        lib = ctypes.CDLL(path)
        lib.e3b_abi_version.restype = c_int
        lib.e3b_last_error.restype = c_char_p
        lib.e3b_sh_fwd.argtypes = [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]
        lib.e3b_sh_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]
        lib.e3b_csr_scratch_bytes.argtypes = [c_int64, c_int64]
        lib.e3b_csr_scratch_bytes.restype = c_int64
        lib.e3b_csr_from_dst.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]
        lib.e3b_dense_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p]
        lib.e3b_dense_bwd_w.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]
        lib.e3b_fill_columns.argtypes = [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
        spec = [c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_float, c_float, c_int]
        lib.e3b_radial_embed_fwd.argtypes = [c_void_p] * 5 + [c_int64, c_int64] + spec + [c_void_p, c_void_p, c_void_p, c_void_p]
        lib.e3b_radial_embed_bwd.argtypes = [c_void_p] * 7 + [c_int64, c_int64] + spec + [c_void_p, c_void_p, c_void_p]
        lib.e3b_neighbor_scratch_bytes.argtypes = [c_int64, c_double, c_double]
        lib.e3b_neighbor_scratch_bytes.restype = c_int64
        lib.e3b_neighbor_count.argtypes = [c_void_p, c_int64, c_double, c_double, c_void_p, c_int64, c_void_p, c_void_p]
        lib.e3b_neighbor_fill.argtypes = [c_void_p, c_int64, c_double, c_double, c_void_p, c_int64, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_void_p]
        lib.e3b_gate_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]
        lib.e3b_gate_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]
        for name in ("e3b_sh_fwd", "e3b_sh_bwd", "e3b_csr_from_dst", "e3b_dense_fwd", "e3b_dense_bwd_w", "e3b_fill_columns",
                     "e3b_radial_embed_fwd", "e3b_radial_embed_bwd", "e3b_neighbor_count", "e3b_neighbor_fill",
                     "e3b_gate_fwd", "e3b_gate_bwd"):
            getattr(lib, name).restype = c_int
        _core = lib
    return _core


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = core().e3b_last_error().decode()
        raise E3BError(f"{what} failed with status {rc}: {msg}")


class LayoutModule:
    """A generated per-layout shared object (``include/e3nn_b200_layout.h``)."""

    def __init__(self, path: str):
        self.path = path
        lib = ctypes.CDLL(path)
        self.lib = lib
        lib.e3b_layout_info.argtypes = [POINTER(c_int32)]
        lib.e3b_layout_key.restype = c_char_p
        lib.e3b_layout_last_error.restype = c_char_p
        lib.e3b_uvu_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]
        lib.e3b_uvu_bwd.argtypes = [c_void_p] * 7 + [c_int64, c_int, c_void_p]
        lib.e3b_conv_fwd.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_int64, c_int64, c_int64, c_float, c_void_p, c_void_p]
        lib.e3b_conv_bwd.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_int64, c_int64, c_int64, c_float, c_void_p, c_void_p]
        lib.e3b_conv_select.argtypes = [c_int]
        lib.e3b_conv_bwd_x.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_int64, c_int64, c_int64, c_float, c_void_p, c_void_p]
        for name in ("e3b_uvu_fwd", "e3b_uvu_bwd", "e3b_conv_fwd", "e3b_conv_bwd", "e3b_layout_info", "e3b_conv_select",
                     "e3b_conv_bwd_x"):
            getattr(lib, name).restype = c_int
        dims = (c_int32 * 8)()
        lib.e3b_layout_info(dims)
        self.d1, self.d2, self.dout, self.wn, self.sh_lmax, self.group = (int(dims[i]) for i in range(6))
        self.key = lib.e3b_layout_key().decode()

    def check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise E3BError(f"{what} failed with status {rc}: {self.lib.e3b_layout_last_error().decode()}")


def uvu_layout_module(spec) -> LayoutModule:
    """Generated module of a 'uvu' layout: loaded from ``_layouts/`` or generated + compiled now."""
    key = spec.key()
    mod = _layout_cache.get(key)
    if mod is not None:
        return mod
    from .codegen import uvu

    so = os.path.join(_build.LAYOUT_DIR, f"uvu_{key}.so")
    if not os.path.exists(so) or _build.nvcc_path() is not None:
        so = _build.build_layout_module("uvu", key, uvu.emit_module(spec))
    mod = LayoutModule(so)
    if mod.key != key:
        raise E3BError(f"layout module {so} was built for another layout ({mod.key} != {key})")
    _layout_cache[key] = mod
    return mod


class TcModule:
    """A generated tensor-core module for one fully-connected ('uvw') layout."""

    def __init__(self, path: str):
        self.path = path
        lib = ctypes.CDLL(path)
        self.lib = lib
        lib.e3b_layout_info.argtypes = [POINTER(c_int32)]
        lib.e3b_layout_key.restype = c_char_p
        lib.e3b_layout_last_error.restype = c_char_p
        lib.e3b_uvw_tc_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p]
        lib.e3b_uvw_tc_fwd.restype = c_int
        dims = (c_int32 * 8)()
        lib.e3b_layout_info(dims)
        self.d1, self.d2, self.dout, self.wn = (int(dims[i]) for i in range(4))
        self.key = lib.e3b_layout_key().decode()

    def check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise E3BError(f"{what} failed with status {rc}: {self.lib.e3b_layout_last_error().decode()}")


_tc_cache: Dict[str, "TcModule"] = {}


def uvw_tc_module(spec) -> TcModule:
    key = spec.key()
    mod = _tc_cache.get(key)
    if mod is not None:
        return mod
    from .codegen import uvw_tc

    so = os.path.join(_build.LAYOUT_DIR, f"uvwtc_{key}.so")
    if not os.path.exists(so) or _build.nvcc_path() is not None:
        so = _build.build_layout_module("uvwtc", key, uvw_tc.emit_module(spec))
    mod = TcModule(so)
    if mod.key != key:
        raise E3BError(f"layout module {so} was built for another layout ({mod.key} != {key})")
    _tc_cache[key] = mod
    return mod


class TcGemmModule:
    """A generated fp32-accurate tensor-core module (``codegen/tc_gemm.py``) for one contraction layout."""

    def __init__(self, path: str):
        self.path = path
        lib = ctypes.CDLL(path)
        self.lib = lib
        lib.e3b_layout_key.restype = c_char_p
        lib.e3b_layout_last_error.restype = c_char_p
        lib.e3b_tc_gemm_scratch_bytes.restype = ctypes.c_longlong
        lib.e3b_tc_gemm_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p,
                                        c_void_p, c_void_p]
        lib.e3b_tc_gemm_fwd.restype = c_int
        self.key = lib.e3b_layout_key().decode()
        self.scratch_bytes = int(lib.e3b_tc_gemm_scratch_bytes())
        self._scratch: Dict[str, torch.Tensor] = {}
        self.last_status = None

    def check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise E3BError(f"{what} failed with status {rc}: {self.lib.e3b_layout_last_error().decode()}")

    def run(self, x1: torch.Tensor, x2: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor, precision: int = 2):
        dev = out.device
        # prepared weights live in a per-stream-ordered scratch tensor owned by the caller side (here)
        scratch = torch.empty(max(self.scratch_bytes, 16), dtype=torch.uint8, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            rc = self.lib.e3b_tc_gemm_fwd(_ptr(x1), _ptr(x2), _ptr(weight), _ptr(out), x1.shape[0], precision,
                                          _ptr(scratch), None, _ptr(status), stream_ptr())
        self.check(rc, "e3b_tc_gemm_fwd")
        self.last_status = status
        return out


_tcg_cache: Dict[str, "TcGemmModule"] = {}


def tc_gemm_module(gemm_spec) -> TcGemmModule:
    key = gemm_spec.key
    mod = _tcg_cache.get(key)
    if mod is not None:
        return mod
    from .codegen import tc_gemm

    so = os.path.join(_build.LAYOUT_DIR, f"tcg_{key}.so")
    if not os.path.exists(so) or _build.nvcc_path() is not None:
        so = _build.build_layout_module("tcg", key, tc_gemm.emit_module(gemm_spec))
    mod = TcGemmModule(so)
    if mod.key != key:
        raise E3BError(f"layout module {so} was built for another layout ({mod.key} != {key})")
    _tcg_cache[key] = mod
    return mod
