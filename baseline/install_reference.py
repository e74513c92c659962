"""Install the unmodified e3nn reference next to this file, for the CPU arm of ``bench.py``.

    python baseline/install_reference.py [SOURCE_DIR]

``SOURCE_DIR`` (default: the ``E3NN_REFERENCE`` environment variable) is a checkout of e3nn 0.6.0 (the
directory that holds ``pyproject.toml`` and the ``e3nn`` package).  The package is installed offline
with pip into ``baseline/_ref`` (``--no-deps``: its one missing dependency, ``opt_einsum_fx``, cannot be
resolved without an index).  ``opt_einsum_fx`` only re-orders einsum contractions and removes dead FX
nodes, so an identity stand-in with its two entry points is written beside the package; the timed code
path is otherwise the stock one.  ``baseline/_ref`` is not tracked by git.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")

SHIM = '''"""Identity stand-in for opt_einsum_fx (contraction-order optimiser; no change of arithmetic)."""


def optimize_einsums_full(model, example_inputs, **kwargs):
    return model


def jitable(gm):
    return gm
'''


def installed() -> bool:
    return os.path.isfile(os.path.join(TARGET, "e3nn", "__init__.py")) and \
        os.path.isfile(os.path.join(TARGET, "opt_einsum_fx", "__init__.py"))


def install(source: str, force: bool = False) -> str:
    """pip-install ``source`` into ``baseline/_ref`` and write the stand-in; returns the outcome in one line."""
    if installed() and not force:
        return "already installed"
    if not os.path.isfile(os.path.join(source, "pyproject.toml")) and not os.path.isfile(os.path.join(source, "setup.py")):
        raise FileNotFoundError(f"{source} does not look like an e3nn checkout")
    os.makedirs(TARGET, exist_ok=True)
    base = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--upgrade",
            "--find-links", "/opt/wheelhouse", "--target", TARGET]
    proc = subprocess.run(base + [source], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    how = "pip --no-deps from the source tree"
    if proc.returncode != 0:
        # a read-only source tree: build from a scratch copy
        with tempfile.TemporaryDirectory() as tmp:
            copy = os.path.join(tmp, "e3nn_src")
            shutil.copytree(source, copy, ignore=shutil.ignore_patterns(".git"))
            proc = subprocess.run(base + [copy], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        how = "pip --no-deps from a scratch copy of the source tree"
        if proc.returncode != 0:
            raise RuntimeError("installing the reference failed:\n" + proc.stdout[-2000:])
    os.makedirs(os.path.join(TARGET, "opt_einsum_fx"), exist_ok=True)
    with open(os.path.join(TARGET, "opt_einsum_fx", "__init__.py"), "w") as f:
        f.write(SHIM)
    return how


if __name__ == "__main__":
    src = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("E3NN_REFERENCE", "")
    if not src:
        raise SystemExit("usage: python baseline/install_reference.py SOURCE_DIR  (or set E3NN_REFERENCE)")
    print(install(src, force="--force" in sys.argv))
