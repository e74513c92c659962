import json
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden_meta():
    with open(os.path.join(GOLDEN, "meta.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return {k: v for k, v in np.load(os.path.join(GOLDEN, name + ".npz")).items()}

    return load


def rel_err(a: torch.Tensor, ref: torch.Tensor) -> float:
    """max|a - ref| / rms(ref): the parity metric of the hot path."""
    ref = ref.double()
    rms = ref.pow(2).mean().sqrt().item()
    if rms == 0.0:
        rms = 1.0
    err = (a.double() - ref).abs().max().item() / rms
    log = os.environ.get("E3NN_B200_ERR_LOG")
    if log:      # margins of every parity assertion: file, line and value of each call
        import inspect

        fr = inspect.stack()[1]
        with open(log, "a") as f:
            f.write(f"{os.path.basename(fr.filename)}:{fr.lineno} {fr.function} {err:.3e}\n")
    return err


def fp32_bound(err32: float, tol: float = 1e-5) -> float:
    """Bound for an fp32 kernel on a case where plain fp32 arithmetic (the CPU oracle evaluated in fp32 on the same
    inputs, `err32` = its distance from the fp64 result) itself exceeds the 1e-5 x RMS budget: the kernel may be at
    most 1.5 x as far from the fp64 result as that evaluation, and never needs to be better than `tol`."""
    return max(tol, 1.5 * err32)
