"""Error reporting of the kernels: the per-device status word, bounded waits, and rejection of operands a kernel
must not dereference.  Nothing here faults or hangs the GPU: the one wait that runs out does so by design after a
few hundred polls and the kernel returns normally."""
import pytest
import torch

import e3nn_b200
from e3nn_b200 import _lib, layouts, o3
from e3nn_b200 import nn as bnn

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_reaches_python():
    dev = torch.device("cuda", 0)
    e3nn_b200.check_status()                      # start clean
    word = _lib.status_word(dev)
    rc = _lib.core().e3b_selftest_bounded_wait(_lib._ptr(word), 500, _lib.stream_ptr())
    assert rc == 0
    _lib.status_after_launch(dev)
    assert e3nn_b200.last_status_code() == 3      # the wait ran out, the kernel returned, the context is alive
    with pytest.raises(e3nn_b200.E3BError, match="bounded wait"):
        e3nn_b200.check_status()
    e3nn_b200.check_status()                      # raised once, then cleared
    # the device still computes
    x = torch.randn(1000, 3, device=dev)
    y = o3.spherical_harmonics([0, 1, 2], x, True, "component")
    assert torch.isfinite(y).all()


def test_status_is_raised_by_the_next_call_without_a_sync():
    dev = torch.device("cuda", 0)
    e3nn_b200.check_status()
    word = _lib.status_word(dev)
    assert _lib.core().e3b_selftest_bounded_wait(_lib._ptr(word), 200, _lib.stream_ptr()) == 0
    _lib.status_after_launch(dev)
    torch.cuda.synchronize()                      # the read-back has landed; poll_status itself never waits
    lin = o3.Linear("8x0e+8x1o", "8x0e+8x1o").to(dev)
    with pytest.raises(e3nn_b200.E3BError):
        lin(torch.randn(4, 32, device=dev))
    lin(torch.randn(4, 32, device=dev))           # cleared
    e3nn_b200.check_status()


def test_selftest_rejects_bad_limit():
    dev = torch.device("cuda", 0)
    word = _lib.status_word(dev)
    assert _lib.core().e3b_selftest_bounded_wait(_lib._ptr(word), 0, _lib.stream_ptr()) == -1
    assert _lib.core().e3b_selftest_bounded_wait(None, 10, _lib.stream_ptr()) == -1


def test_operands_on_the_wrong_device_or_of_the_wrong_size_are_rejected():
    dev = torch.device("cuda", 0)
    x = torch.randn(5, 32, device=dev)
    lin_cpu = o3.Linear("8x0e+8x1o", "8x0e+8x1o")            # parameters left on the host
    with pytest.raises(RuntimeError, match="same device"):
        lin_cpu(x)
    lin = o3.Linear("8x0e+8x1o", "8x0e+8x1o", internal_weights=False, shared_weights=True).to(dev)
    with pytest.raises(RuntimeError):
        lin(x, torch.randn(lin.weight_numel))                 # external weight on the host
    with pytest.raises(RuntimeError):
        lin(x, torch.randn(lin.weight_numel, device=dev, dtype=torch.float64))
    with pytest.raises((AssertionError, RuntimeError)):
        lin(x, torch.randn(lin.weight_numel - 1, device=dev))
    gate = bnn.Gate("4x0e", [torch.tanh], "2x0e", [torch.sigmoid], "2x1o")   # tables left on the host
    with pytest.raises(RuntimeError, match="same device"):
        gate(torch.randn(3, gate.irreps_in.dim, device=dev))
    fc = bnn.FullyConnectedNet([64, 64], math_mode="tf32x3")                  # weights left on the host
    with pytest.raises(RuntimeError):
        fc(torch.randn(128, 64, device=dev))
    tp = layouts.conv_tensor_product("8x0e+8x1o", "0e+1o", "0e+1o")
    N, E = 4, 8
    rowptr = torch.arange(0, E + 1, 2, device=dev)
    with pytest.raises((RuntimeError, NotImplementedError)):
        e3nn_b200.conv_uvu(tp, torch.randn(N, tp.irreps_in1.dim, device=dev), torch.randn(E, 3, device=dev),
                           torch.zeros(E, dtype=torch.int64, device=dev), rowptr, torch.randn(E, tp.weight_numel),
                           edge_attr_is_vector=True)
    e3nn_b200.check_status()


def test_second_differentiation_is_refused():
    dev = torch.device("cuda", 0)
    x = torch.randn(16, 3, device=dev, requires_grad=True)
    y = o3.spherical_harmonics([1, 2], x, True, "component")
    (g,) = torch.autograd.grad(y.pow(2).sum(), x, create_graph=True)
    with pytest.raises(RuntimeError, match="once_differentiable"):
        g.sum().backward()
