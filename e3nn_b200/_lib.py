"""ctypes bindings of the C-ABI libraries (``include/e3nn_b200.h``, ``include/e3nn_b200_layout.h``).

There is no CPU or PyTorch fallback: if the CUDA library is missing, loading fails with an
error that says how to build it, and every op raises for tensors that are not on a CUDA device.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
import threading
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_void_p
from typing import Dict, List, Optional

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


NVTX_ENABLED = os.environ.get("E3NN_B200_NVTX", "0") not in ("", "0")


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range around a kernel launch (visible in Nsight timelines) when E3NN_B200_NVTX=1; free otherwise."""
    if not NVTX_ENABLED:
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise NotImplementedError(
                "e3nn_b200 runs on CUDA (sm_100a) only: got a tensor on device "
                f"'{t.device}'. There is no CPU implementation in this package."
            )


# ------------------------------------------------------------------------------------------- kernel status
# Kernels report conditions they cannot raise themselves through a status word in device memory: 1 = a destination
# index out of range (CSR builder), 2 = a source / edge index out of range (the access was skipped), 3 = a bounded
# wait on an mbarrier gave up (the kernel returned early, its output is incomplete).  One word per device lives for
# the life of the process.  After every launch that can raise it, a 4-byte copy into pinned host memory is enqueued
# behind the kernel; the next call of any op on that device looks at the copy if it has landed (no
# synchronisation) and raises; `check_status` synchronises and raises.  A code stays until it is raised once.
class _DeviceStatus:
    def __init__(self, device: torch.device):
        self.device = device
        self.word = torch.zeros(1, dtype=torch.int32, device=device)
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event: Optional[torch.cuda.Event] = None

    def clear(self) -> None:
        self.word.zero_()
        self.host.zero_()
        self.event = None


_status: Dict[int, _DeviceStatus] = {}


def _device_status(device: torch.device) -> _DeviceStatus:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _status.get(idx)
    if st is None:
        st = _status[idx] = _DeviceStatus(torch.device("cuda", idx))
    return st


def status_word(device: torch.device) -> torch.Tensor:
    """The device's persistent int32 status word (pass its pointer to the kernels)."""
    return _device_status(device).word


def _raise_status(code: int, what: str) -> None:
    if code == 2:
        raise IndexError(f"{what}: an edge or source index was outside its range (the kernel skipped the access)")
    if code == 1:
        raise IndexError(f"{what}: a destination index was outside [0, num_nodes)")
    if code == 3:
        raise E3BError(f"{what}: a bounded wait inside a kernel gave up (status 3); the output of that launch is incomplete")
    raise E3BError(f"{what}: kernel status {code}")


def status_after_launch(device: torch.device) -> None:
    """Enqueue the read-back of the status word behind the launches made so far on the current stream."""
    if torch.cuda.is_current_stream_capturing():
        return
    st = _device_status(device)
    with torch.cuda.device(st.device):
        st.host.copy_(st.word, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
    st.event = ev


def poll_status(device: torch.device, what: str = "an earlier e3nn_b200 kernel") -> None:
    """Raise if an earlier launch on `device` has reported a condition and its read-back has landed.  Never waits."""
    st = _status.get(device.index if device.index is not None else torch.cuda.current_device())
    if st is None or st.event is None or torch.cuda.is_current_stream_capturing() or not st.event.query():
        return
    code = int(st.host[0])
    st.event = None
    if code != 0:
        st.clear()
        _raise_status(code, what)


def last_status_code(device: Optional[torch.device] = None) -> int:
    """Synchronise `device` (default: the current one) and return its status word without raising or clearing."""
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    st = _device_status(dev)
    return int(st.word.item())


def check_status(device: Optional[torch.device] = None, what: str = "e3nn_b200 kernels") -> None:
    """Synchronise `device` and raise if any launch since the last check reported a condition."""
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    code = last_status_code(dev)
    if code != 0:
        _device_status(dev).clear()
        _raise_status(code, what)


def require_same_device(*tensors: Optional[torch.Tensor]) -> None:
    """Every tensor whose pointer goes to a kernel must be on one CUDA device (a host pointer or another GPU's
    memory would be dereferenced by the kernel)."""
    first = None
    for t in tensors:
        if t is None:
            continue
        require_cuda(t)
        if first is None:
            first = t.device
        elif t.device != first:
            raise RuntimeError(f"expected all tensors on {first}, got one on {t.device}")


def require_operand(t: torch.Tensor, like: torch.Tensor, name: str, numel: Optional[int] = None,
                    dtype: torch.dtype = torch.float32) -> None:
    """A tensor whose pointer a kernel dereferences: on the device of `like`, of `dtype`, with `numel` elements.
    Raises the reference's error types (`RuntimeError` for device / dtype, `torch._assert` for the size) instead
    of letting the kernel read a host pointer or run past the end of a buffer."""
    if not t.is_cuda or t.device != like.device:
        raise RuntimeError(f"Expected all tensors to be on the same device, but {name} is on {t.device} "
                           f"and the features are on {like.device}")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")
    if numel is not None:
        torch._assert(t.numel() == numel, f"Invalid {name} shape: expected {numel} elements, got {t.numel()}")


def core() -> ctypes.CDLL:
    """The fixed-function library; (re)built on first use when nvcc is present and a source is newer."""
    global _core
    if _core is not None:
        return _core
    with _core_lock:
        if _core is not None:
            return _core
        path = _build.CORE_LIB
        if _build.nvcc_path() is not None:
            _build.build_core()        # compares modification times: a no-op when the library is up to date
        elif not os.path.exists(path):
            raise E3BError(
                f"{path} is missing and nvcc is not available to build it. "
                "Build it with `python -c 'import __graft_entry__ as g; g.build()'` on a machine with CUDA 12.9."
            )
        lib = ctypes.CDLL(path)
        lib.e3b_abi_version.restype = c_int
        lib.e3b_last_error.restype = c_char_p
        lib.e3b_sh_fwd.argtypes = [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]
        lib.e3b_sh_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]
        lib.e3b_csr_scratch_bytes.argtypes = [c_int64, c_int64]
        lib.e3b_csr_scratch_bytes.restype = c_int64
        lib.e3b_csr_from_dst.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]
        lib.e3b_dense_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p]
        lib.e3b_dense_fwd_gate.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                           c_int, c_int64, c_void_p]
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
        lib.e3b_neighbor_count_rows.argtypes = [c_void_p, c_int64, c_double, c_double, c_void_p, c_int64, c_int64, c_int64,
                                                c_void_p, c_void_p]
        lib.e3b_neighbor_fill_rows.argtypes = [c_void_p, c_int64, c_double, c_double, c_void_p, c_int64, c_int64, c_int64,
                                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        lib.e3b_gate_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]
        lib.e3b_gate_fwd_channels.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]
        lib.e3b_gate_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]
        lib.e3b_selftest_bounded_wait.argtypes = [c_void_p, ctypes.c_uint, c_void_p]
        lib.e3b_selftest_bounded_wait.restype = c_int
        for name in ("e3b_sh_fwd", "e3b_sh_bwd", "e3b_csr_from_dst", "e3b_dense_fwd", "e3b_dense_fwd_gate", "e3b_dense_bwd_w", "e3b_fill_columns",
                     "e3b_radial_embed_fwd", "e3b_radial_embed_bwd", "e3b_neighbor_count", "e3b_neighbor_fill",
                     "e3b_neighbor_count_rows", "e3b_neighbor_fill_rows",
                     "e3b_gate_fwd", "e3b_gate_fwd_channels", "e3b_gate_bwd"):
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
    from .codegen import uvw_post, uvw_tc

    # the kernel that applies the Clebsch-Gordan coupling after the matrix product, when the layout fits it
    kind, gen = ("uvwpost", uvw_post) if uvw_post.plan_groups(spec) is not None else ("uvwtc", uvw_tc)
    so = os.path.join(_build.LAYOUT_DIR, f"{kind}_{key}.so")
    if not os.path.exists(so) or _build.nvcc_path() is not None:
        so = _build.build_layout_module(kind, key, gen.emit_module(spec))
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
        lib.e3b_tc_gemm_fwd_gate.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64,
                                             c_int, c_void_p, c_void_p, c_void_p]
        lib.e3b_tc_gemm_fwd_gate.restype = c_int
        self.key = lib.e3b_layout_key().decode()
        self.scratch_bytes = int(lib.e3b_tc_gemm_scratch_bytes())
        self.group_work: List[int] = []         # relative cost of a row tile per group (set by tc_gemm_module)
        self._scratch: Dict[str, torch.Tensor] = {}

    def check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise E3BError(f"{what} failed with status {rc}: {self.lib.e3b_layout_last_error().decode()}")

    def run(self, x1: torch.Tensor, x2: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor, precision: int = 2):
        dev = out.device
        # prepared weights live in a per-stream-ordered scratch tensor owned by the caller side (here)
        scratch = torch.empty(max(self.scratch_bytes, 16), dtype=torch.uint8, device=dev)
        poll_status(dev)
        split = None
        if _tc_gemm_max_ctas is not None and self.group_work:
            n = cta_split(self.group_work, int(_tc_gemm_max_ctas))
            split = (ctypes.c_int * len(n))(*n)
        with torch.cuda.device(dev), nvtx_range("e3b_tc_gemm_fwd " + self.key):
            rc = self.lib.e3b_tc_gemm_fwd(_ptr(x1), _ptr(x2), _ptr(weight), _ptr(out), x1.shape[0], precision,
                                          _ptr(scratch), split, _ptr(status_word(dev)), stream_ptr())
        self.check(rc, "e3b_tc_gemm_fwd")
        status_after_launch(dev)
        return out

    def run_gate(self, x1: torch.Tensor, weight: torch.Tensor, gate_tbl: torch.Tensor, gate_cst: torch.Tensor,
                 gates: torch.Tensor, out: torch.Tensor, precision: int = 2):
        """The contraction (a Linear) with Gate as its epilogue: `out` receives the Gate's output rows."""
        dev = out.device
        scratch = torch.empty(max(self.scratch_bytes, 16), dtype=torch.uint8, device=dev)
        poll_status(dev)
        with torch.cuda.device(dev), nvtx_range("e3b_tc_gemm_fwd_gate " + self.key):
            rc = self.lib.e3b_tc_gemm_fwd_gate(_ptr(x1), _ptr(weight), _ptr(gate_tbl), _ptr(gate_cst), _ptr(gates),
                                               gates.shape[1], _ptr(out), out.shape[1], x1.shape[0], precision,
                                               _ptr(scratch), _ptr(status_word(dev)), stream_ptr())
        self.check(rc, "e3b_tc_gemm_fwd_gate")
        status_after_launch(dev)
        return out


_tcg_cache: Dict[str, "TcGemmModule"] = {}
_tc_gemm_max_ctas: Optional[int] = None


def cta_split(work: List[int], max_ctas: int) -> List[int]:
    """CTAs per group in proportion to the groups' work: at least one each, ``max(max_ctas, len(work))`` in total."""
    total, limit = sum(work), max(max_ctas, len(work))
    n = [max(1, limit * wk // total) for wk in work]
    g = len(n) - 1
    while sum(n) < limit:
        n[g] += 1
        g = (g - 1) % len(n)
    while sum(n) > limit and max(n) > 1:
        n[n.index(max(n))] -= 1
    return n


@contextlib.contextmanager
def tc_gemm_cta_limit(max_ctas: Optional[int]):
    """Inside the block the persistent tensor-core contractions launch at most ``max_ctas`` CTAs (one per SM), leaving
    the other SMs to a kernel that runs at the same time.  These kernels split their row tiles statically over their
    CTAs and take a whole SM each; when a collective's kernel already holds some SMs, the CTAs that cannot start
    until it ends hold the whole launch back by its duration, which costs more than giving up those SMs."""
    global _tc_gemm_max_ctas
    old = _tc_gemm_max_ctas
    _tc_gemm_max_ctas = max_ctas
    try:
        yield
    finally:
        _tc_gemm_max_ctas = old


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
    mod.group_work = [g.work() for g in gemm_spec.groups]
    _tcg_cache[key] = mod
    return mod
