"""Building the CUDA libraries in-tree with nvcc (sm_100a only).

Two kinds of shared objects are produced:

* ``e3nn_b200/lib/libe3nn_b200.so`` -- the fixed-function C-ABI library declared in
  ``include/e3nn_b200.h`` (spherical harmonics, CSR builder, dense 'uvw'/Linear kernels, ...);
* ``e3nn_b200/_layouts/<kind>_<key>.so`` -- one generated module per irreps layout, exporting
  the entry points of ``include/e3nn_b200_layout.h``.  A module is generated and compiled the
  first time a layout is used (nvcc must be on the machine) and reused afterwards.
"""
from __future__ import annotations

import contextlib
import fcntl
import os
import shutil
import subprocess
import threading
from typing import List, Optional

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LAYOUT_DIR = os.path.join(PKG, "_layouts")
CORE_LIB = os.path.join(LIB_DIR, "libe3nn_b200.so")
CORE_SOURCES = ["abi.cu", "sh.cu", "csr.cu", "dense.cu", "radial.cu", "neighbor.cu", "gate.cu", "selftest.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]
_lock = threading.Lock()


_target_locks = {}


@contextlib.contextmanager
def _build_lock(name: str):
    """One builder per target at a time, across threads (a lock per target) and across processes (an advisory lock
    on a file beside the target): ranks started together that all miss the same module take turns, and the later
    ones find the first one's result.  Different targets build in parallel."""
    with _lock:
        tl = _target_locks.setdefault(name, threading.Lock())
    with tl:
        os.makedirs(LAYOUT_DIR, exist_ok=True)
        with open(os.path.join(LAYOUT_DIR, f".lock_{name}"), "w") as f:
            fcntl.flock(f, fcntl.LOCK_EX)
            try:
                yield
            finally:
                fcntl.flock(f, fcntl.LOCK_UN)


def _write_atomic(path: str, text: str) -> None:
    tmp = f"{path}.tmp{os.getpid()}"
    with open(tmp, "w") as f:
        f.write(text)
    os.replace(tmp, path)


def nvcc_path() -> Optional[str]:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def _flags() -> List[str]:
    return list(NVCC_FLAGS)


def _run(cmd: List[str], what: str) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed while building {what}:\n{' '.join(cmd)}\n{proc.stdout}")


def generate_sh_header() -> str:
    from .codegen import sh

    path = os.path.join(CSRC, "sh_gen.cuh")
    text = sh.emit_header()
    with _build_lock("sh_gen"):
        if not os.path.exists(path) or open(path).read() != text:
            _write_atomic(path, text)
    return path


def _newer(target: str, deps: List[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps if os.path.exists(d))


def build_core(force: bool = False, verbose: bool = False) -> str:
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libe3nn_b200.so")
    header = generate_sh_header()
    with _build_lock("core"):
        os.makedirs(LIB_DIR, exist_ok=True)
        srcs = [os.path.join(CSRC, s) for s in CORE_SOURCES if os.path.exists(os.path.join(CSRC, s))]
        deps = srcs + [header, os.path.join(CSRC, "common.cuh"), os.path.join(PKG, "..", "include", "e3nn_b200.h")]
        deps += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
        if not force and _newer(CORE_LIB, deps):
            return CORE_LIB
        tmp = CORE_LIB + f".tmp{os.getpid()}"
        cmd = [nvcc] + _flags() + ["-shared", "-t", "0", "-o", tmp] + srcs
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        _run(cmd, "libe3nn_b200.so")
        os.replace(tmp, CORE_LIB)
    return CORE_LIB


def build_layout_module(kind: str, key: str, source: str, force: bool = False, extra_flags: Optional[List[str]] = None) -> str:
    """Write ``source`` to ``_layouts/<kind>_<key>.cu`` and compile it (reusing an up-to-date .so)."""
    os.makedirs(LAYOUT_DIR, exist_ok=True)
    cu = os.path.join(LAYOUT_DIR, f"{kind}_{key}.cu")
    so = os.path.join(LAYOUT_DIR, f"{kind}_{key}.so")
    generate_sh_header()
    with _build_lock(f"{kind}_{key}"):
        same = os.path.exists(cu) and open(cu).read() == source
        headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]     # every header a module may include
        if same and os.path.exists(so) and not force and _newer(so, [cu] + headers):
            return so
        nvcc = nvcc_path()
        if nvcc is None:
            raise RuntimeError(
                f"layout module {kind}_{key} is not built and nvcc is not available to build it; "
                "run __graft_entry__.build() (or e3nn_b200.prebuild) on a machine with the CUDA toolkit"
            )
        if not same:
            _write_atomic(cu, source)
        tmp = so + f".tmp{os.getpid()}"
        cmd = [nvcc] + _flags() + (extra_flags or []) + ["-I", CSRC, "-shared", "-o", tmp, cu]
        _run(cmd, os.path.basename(so))
        os.replace(tmp, so)
    return so
