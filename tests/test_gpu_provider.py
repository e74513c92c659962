"""The reference-side binding of INTEGRATION.md: this package registered as the first code-generation provider of a
live e3nn (``e3nn/o3/_tensor_product/_tensor_product.py:17-21``), so that the reference's own ``TensorProduct`` /
``FullyConnectedTensorProduct`` modules run on these kernels.  Needs the unmodified reference installed in
``baseline/_ref`` (``baseline/install_reference.py``); skipped where it is absent."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

pytestmark = pytest.mark.gpu


def _reference():
    if not os.path.isfile(os.path.join(REF, "e3nn", "__init__.py")):
        pytest.skip("the reference is not installed in baseline/_ref")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import e3nn  # noqa: F401
    from e3nn import o3

    return o3


def test_provider_snippet_runs_the_reference_modules_on_these_kernels():
    o3 = _reference()
    from e3nn.o3._tensor_product import _tensor_product as _tp

    from e3nn_b200 import o3 as b200

    calls = []

    class _B200Main(torch.nn.Module):
        def __init__(self, irreps_in1, irreps_in2, irreps_out, instructions, shared_weights):
            super().__init__()
            ins = [(i.i_in1, i.i_in2, i.i_out, i.connection_mode, i.has_weight, i.path_weight ** 2) for i in instructions]
            self.tp = b200.TensorProduct(irreps_in1, irreps_in2, irreps_out, ins, irrep_normalization="none",
                                         path_normalization="none", internal_weights=False, shared_weights=shared_weights)

        def forward(self, x1, x2, w):
            calls.append(1)
            return self.tp(x1, x2, w)

    def b200_provider(irreps_in1, irreps_in2, irreps_out, instructions, shared_weights, specialized_code, optimize_einsums):
        # e3nn registers an fx.GraphModule (e3nn/util/codegen/_mixin.py): a three-node graph that calls the module
        root = torch.nn.Module()
        root.tp = _B200Main(str(irreps_in1), str(irreps_in2), str(irreps_out), instructions, shared_weights)
        graph = torch.fx.Graph()
        x1, x2, w = graph.placeholder("x1"), graph.placeholder("x2"), graph.placeholder("w")
        graph.output(graph.call_module("tp", (x1, x2, w)))
        return torch.fx.GraphModule(root, graph, class_name="tp_forward")

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    layout = ("8x0e+8x1o+4x2e", "0e+1o+2e", "8x0e+6x1o+4x2e")
    stock = o3.FullyConnectedTensorProduct(*layout)                       # the reference's own generated graph (CPU)
    ins = [(0, 0, 0, "uvu", True), (1, 1, 0, "uvu", True), (1, 0, 1, "uvu", True), (0, 1, 1, "uvu", True)]
    stock_u = o3.TensorProduct("4x0e+4x1o", "0e+1o", "4x0e+4x1o", ins, shared_weights=False, internal_weights=False)
    _tp._CODEGEN_PROVIDERS_LEFT_RIGHT.insert(0, b200_provider)
    try:
        patched = o3.FullyConnectedTensorProduct(*layout)                 # same class, main graph from the provider
        with torch.no_grad():
            patched.weight.copy_(stock.weight)      # (the generated sub-graphs hold different constant buffers)
        patched = patched.to(dev)
        x, y = torch.randn(300, stock.irreps_in1.dim), torch.randn(300, stock.irreps_in2.dim)
        out = patched(x.to(dev), y.to(dev))
        # 'uvu' with per-row weights through the same seam
        patched_u = o3.TensorProduct("4x0e+4x1o", "0e+1o", "4x0e+4x1o", ins, shared_weights=False, internal_weights=False).to(dev)
        xu, yu, wu = torch.randn(50, 16), torch.randn(50, 4), torch.randn(50, stock_u.weight_numel)
        out_u = patched_u(xu.to(dev), yu.to(dev), wu.to(dev))
    finally:
        _tp._CODEGEN_PROVIDERS_LEFT_RIGHT.remove(b200_provider)
    assert calls, "the provider's module was not called"
    ref = stock.double()(x.double(), y.double())
    rms = ref.pow(2).mean().sqrt().item()
    assert (out.cpu().double() - ref).abs().max().item() / rms < 1e-5
    ref_u = stock_u.double()(xu.double(), yu.double(), wu.double())
    assert (out_u.cpu().double() - ref_u).abs().max().item() / ref_u.pow(2).mean().sqrt().item() < 1e-5
