"""Host-side logic that needs no GPU: irreps bookkeeping, normalisation, CG, plans, ABI symbols."""
import ctypes
import json
import os
import re

import numpy as np
import pytest
import torch

from conftest import GOLDEN, ROOT
from e3nn_b200 import _build, layouts, o3
from e3nn_b200.o3._wigner import wigner_3j_numpy


def test_irreps_parsing_and_layout():
    ir = o3.Irreps("32x0e + 16x1o+2e")
    assert str(ir) == "32x0e+16x1o+1x2e" and ir.dim == 32 + 48 + 5 and ir.num_irreps == 49
    assert ir.slices() == [slice(0, 32), slice(32, 80), slice(80, 85)]
    assert ir.lmax == 2 and o3.Irrep("1o") in ir and o3.Irrep("1e") not in ir
    assert o3.Irreps("1e + 1e + 0e").simplify() == o3.Irreps("2x1e+1x0e")
    s = o3.Irreps("2o + 1e + 0e + 1e").sort()
    assert s.p == (3, 1, 0, 2) and s.inv == (2, 1, 3, 0) and str(s.irreps) == "1x0e+1x1e+1x1e+1x2o"
    assert [str(x) for x in o3.Irrep("1o") * o3.Irrep("2e")] == ["1o", "2o", "3o"]
    assert str(o3.Irreps.spherical_harmonics(3)) == "1x0e+1x1o+1x2e+1x3o"
    with pytest.raises(ValueError):
        o3.Irreps("3x1z")
    it = o3.Irrep.iterator()
    assert [str(next(it)) for _ in range(4)] == ["0e", "0o", "1o", "1e"]


def test_wigner_3j_matches_golden(golden):
    for key, ref in golden("wigner_3j").items():
        l1, l2, l3 = map(int, key.split("_"))
        assert np.abs(wigner_3j_numpy(l1, l2, l3) - ref).max() < 1e-12, key
    # identities the reference's specialised code relies on (_codegen.py:150-163, 252-253)
    for l in range(4):
        c = wigner_3j_numpy(0, l, l)[0]
        assert np.allclose(c, np.eye(2 * l + 1) / np.sqrt(2 * l + 1))
    eps = np.zeros((3, 3, 3))
    for a, b, c in [(0, 1, 2), (1, 2, 0), (2, 0, 1)]:
        eps[a, b, c], eps[a, c, b] = 1, -1
    assert np.allclose(np.abs(wigner_3j_numpy(1, 1, 1)), np.abs(eps) / np.sqrt(6))


def test_tp_normalisation_matches_reference(golden_meta):
    for name, m in golden_meta["cases"].items():
        if "irreps_in1" not in m:
            continue
        ins = [tuple(i[:5]) for i in m["instructions"]]
        if name == "tp_mixed_shared":
            ins[4] = ins[4] + (2.5,)
        if name == "tp_uuu_mixed_shared":
            ins[6] = ins[6] + (0.5,)
        if name == "tp_uvuv_mixed_unshared":
            ins[3] = ins[3] + (2.0,)
        if name in ("tp_rest_shared", "tp_rest_unshared"):
            ins[3] = ins[3] + (0.7,)
        tp = o3.TensorProduct(m["irreps_in1"], m["irreps_in2"], m["irreps_out"], ins, internal_weights=False,
                              shared_weights=m["shared_weights"], **m["norm_kwargs"])
        assert tp.weight_numel == m["weight_numel"], name
        assert np.allclose([i.path_weight for i in tp.instructions], [i[5] for i in m["instructions"]], rtol=1e-14)
        assert tp.output_mask.int().tolist() == m["output_mask"], name


def test_bench_layouts():
    tp = layouts.bench_conv_tp("cfg3_15")
    assert (len(tp.instructions), tp.weight_numel, tp.irreps_out.dim) == (15, 960, 3264)
    tp = layouts.bench_conv_tp("cfg3_11")
    assert (len(tp.instructions), tp.weight_numel, tp.irreps_out.dim) == (11, 704, 2240)
    tp = layouts.bench_conv_tp("cfg5_23")
    assert (len(tp.instructions), tp.weight_numel, tp.irreps_out.dim) == (23, 1472, 6336)
    tp = o3.FullyConnectedTensorProduct("128x0e+64x1o+32x2e", "0e+1o+2e+3o", "128x0e+64x1o+32x2e")
    assert (len(tp.instructions), tp.weight_numel) == (13, 59392)
    assert tp.weight.shape == (59392,) and tp.internal_weights and tp.shared_weights


def test_linear_metadata(golden_meta):
    for name in ("linear_cfg4", "linear_cfg5", "linear_small_bias"):
        m = golden_meta["cases"][name]
        lin = o3.Linear(m["irreps_in"], m["irreps_out"], biases=m["biases"])
        assert (lin.weight_numel, lin.bias_numel) == (m["weight_numel"], m["bias_numel"])
        assert [[i.i_in, i.i_out] for i in lin.instructions] == [i[:2] for i in m["instructions"]]
        assert np.allclose([i.path_weight for i in lin.instructions], [i[3] for i in m["instructions"]])
        assert lin.output_mask.int().tolist() == m["output_mask"]
    # doctest numbers of the reference (e3nn/o3/_linear.py:79-88)
    assert o3.Linear("4x0e+16x1o", "8x0e+8x1o").weight_numel == 160
    with pytest.raises(ValueError):
        o3.Linear("4x0e", "4x1o", instructions=[(0, 0)])
    with pytest.raises(IndexError):
        o3.Linear("4x0e", "4x0e", instructions=[(1, 0)])


def test_error_behaviour_without_gpu():
    tp = o3.FullyConnectedTensorProduct("2x0e+1x1o", "0e+1o", "2x0e+1x1o")
    with pytest.raises(NotImplementedError):
        tp(torch.randn(3, 5), torch.randn(3, 4))           # CPU tensors: no fallback
    with pytest.raises(AssertionError):
        tp(torch.randn(3, 4), torch.randn(3, 4))           # wrong last dimension
    with pytest.raises(KeyError):
        o3.TensorProduct("2x0e", "2x0e", "2x0e", [(0, 0, 0, "vuv", False)])      # not a connection mode (the reference: KeyError too)
    with pytest.raises(AssertionError):
        o3.TensorProduct("3x0e", "3x0e", "2x0e", [(0, 0, 0, "uvu<v", False)])    # 3 pairs u < v, not 2
    tp = o3.TensorProduct("2x0e", "0e", "2x0e", [(0, 0, 0, "uvu", True)], shared_weights=False)
    assert not tp.internal_weights
    with pytest.raises(RuntimeError):
        tp(torch.randn(3, 2), torch.randn(3, 1))           # external weights missing
    with pytest.raises(AssertionError):
        o3.TensorProduct("2x0e", "1o", "2x0e", [(0, 0, 0, "uvu", True)])   # parity / triangle
    with pytest.raises(ValueError):
        o3.SphericalHarmonics("1o+1e", True)                # parities inconsistent with one input
    with pytest.raises(NotImplementedError):
        o3.SphericalHarmonics(13, True)
    with pytest.raises(NotImplementedError):
        o3.spherical_harmonics(2, torch.randn(4, 3), True)


def test_state_dict_and_deepcopy():
    import copy

    tp = o3.FullyConnectedTensorProduct("4x0e+2x1o", "0e+1o", "4x0e+2x1o")
    sd = tp.state_dict()
    assert set(sd) == {"weight", "output_mask"}
    tp2 = copy.deepcopy(tp)
    assert torch.equal(tp2.weight, tp.weight)
    lin = o3.Linear("4x0e+2x1o", "3x0e+2x1o", biases=True)
    assert set(lin.state_dict()) == {"weight", "bias", "output_mask"}
    views = list(tp.weight_views())
    assert sum(v.numel() for v in views) == tp.weight_numel
    assert tp.weight_view_for_instruction(0).shape == tp.instructions[0].path_shape


def _declared_symbols(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(e3b_[a-z0-9_]+)\s*\(", text)))


def test_core_library_exports_every_declared_symbol():
    path = _build.build_core()
    lib = ctypes.CDLL(path)
    names = _declared_symbols("e3nn_b200.h")
    assert len(names) >= 8
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/e3nn_b200.h but not exported"
    lib.e3b_abi_version.restype = ctypes.c_int
    assert lib.e3b_abi_version() >= 1
    lib.e3b_csr_scratch_bytes.restype = ctypes.c_int64
    lib.e3b_csr_scratch_bytes.argtypes = [ctypes.c_int64, ctypes.c_int64]
    assert lib.e3b_csr_scratch_bytes(1000, 10) > 16000


def test_layout_module_exports_every_declared_symbol():
    tp = layouts.conv_tensor_product("8x0e+8x1o+8x2e", "0e+1o+2e", layouts.ALL_L2)
    mod = tp._uvu_module()
    for name in _declared_symbols("e3nn_b200_layout.h"):
        assert hasattr(mod.lib, name), f"{name} declared in include/e3nn_b200_layout.h but not exported"
    assert (mod.d1, mod.d2, mod.dout, mod.wn, mod.sh_lmax) == (72, 9, tp.irreps_out.dim, tp.weight_numel, 2)


def test_tensor_core_modules_export_every_declared_symbol():
    """include/e3nn_b200_tc.h: the tcg module exports e3b_tc_gemm_*, the uvwtc module e3b_uvw_tc_fwd (load only)."""
    from e3nn_b200 import _lib, o3
    from e3nn_b200.codegen import tc_gemm

    names = _declared_symbols("e3nn_b200_tc.h")
    assert {"e3b_tc_gemm_fwd", "e3b_tc_gemm_scratch_bytes", "e3b_uvw_tc_fwd"} <= set(names)
    gs = tc_gemm.matmul_gemm_spec(64, 128, False, 0.125, "hosttest64x128")
    mod = _lib.tc_gemm_module(gs)
    for name in ("e3b_tc_gemm_fwd", "e3b_tc_gemm_scratch_bytes", "e3b_layout_info", "e3b_layout_key", "e3b_layout_last_error"):
        assert hasattr(mod.lib, name), f"{name} not exported by the tc_gemm module"
    tp = o3.FullyConnectedTensorProduct("32x0e+32x1o", "0e+1o", "32x0e+32x1o", math_mode="tf32")
    tc = _lib.uvw_tc_module(tp._spec if hasattr(tp, "_spec") else tp.spec)
    for name in ("e3b_uvw_tc_fwd", "e3b_layout_info", "e3b_layout_key", "e3b_layout_last_error"):
        assert hasattr(tc.lib, name), f"{name} not exported by the uvw_tc module"


def test_cpu_tensors_are_rejected_by_the_new_entry_points():
    """No CPU fallback: the device-only front ends raise, the host neighbour list still works and is sorted."""
    import torch
    from e3nn_b200 import nn as bnn

    pos = torch.rand(50, 3) * 16.0
    with pytest.raises(NotImplementedError):
        bnn.neighbor_list_pbc(pos, 16.0, 5.0)
    with pytest.raises(NotImplementedError):
        bnn.edge_embed(pos, torch.zeros(3, dtype=torch.int64), torch.ones(3, dtype=torch.int64), None, torch.randn(8, 64),
                       5.0, 1.0, 1.0, "silu")
    src, dst, shift = bnn.radius_graph_pbc(pos, 16.0, 5.0)
    assert src.numel() == dst.numel() == shift.shape[0] and src.numel() % 2 == 0
    key = dst * 50 + src
    assert torch.all(key[1:] > key[:-1])                       # sorted by destination, then source, no duplicates
    vec = pos[src] - pos[dst] + shift
    assert float(vec.norm(dim=-1).max()) <= 5.0 + 1e-5


def test_gate_module_bookkeeping_matches_reference(golden_meta):
    """irreps_in / irreps_out of the drop-in Gate equal the reference's (stored with the golden vectors); the error
    conventions of e3nn/nn/_gate.py:91-101 and e3nn/nn/_activation.py:38-57 are kept."""
    import torch
    from e3nn_b200 import nn as bnn

    fn = {"silu": torch.nn.functional.silu, "tanh": torch.tanh, "sigmoid": torch.sigmoid, "abs": torch.abs,
          "relu": torch.relu, None: None}
    for name in ("gate_mixed", "gate_l3", "gate_abs_identity", "gate_no_scalars"):
        m = golden_meta["cases"][name]
        g = bnn.Gate(m["irreps_scalars"], [fn[a] for a in m["act_scalars"]], m["irreps_gates"],
                     [fn[a] for a in m["act_gates"]], m["irreps_gated"])
        assert str(g.irreps_in) == m["irreps_in"] and str(g.irreps_out) == m["irreps_out"]
    with pytest.raises(ValueError):
        bnn.Gate("4x0e", [torch.tanh], "3x0e", [torch.tanh], "4x1o")          # 3 gates for 4 gated irreps
    with pytest.raises(ValueError):
        bnn.Gate("4x1o", [None], "4x0e", [torch.tanh], "4x1o")               # non-scalar "scalars"
    with pytest.raises(ValueError):
        bnn.Gate("4x0o", [torch.nn.functional.silu], "", [], "")              # odd scalar, activation without parity
    with pytest.raises(NotImplementedError):
        bnn.Gate("4x0e", [torch.tanh], "4x0e", [torch.tanh], "4x1o")(torch.zeros(2, 20))   # CPU tensor


def test_elementwise_tensor_product_layout(golden_meta):
    """Block splitting and instruction list of `ElementwiseTensorProduct` against the reference's (golden meta)."""
    m = golden_meta["cases"]["tp_elementwise"]
    etp = o3.ElementwiseTensorProduct("4x0e+3x1o+2x2e+5x1e", "4x0e+3x1o+2x1o+5x2e")
    assert (str(etp.irreps_in1), str(etp.irreps_in2), str(etp.irreps_out)) == (m["irreps_in1"], m["irreps_in2"], m["irreps_out"])
    got = [(i.i_in1, i.i_in2, i.i_out, i.connection_mode, i.has_weight) for i in etp.instructions]
    assert got == [tuple(i[:5]) for i in m["instructions"]]
    assert np.allclose([i.path_weight for i in etp.instructions], [i[5] for i in m["instructions"]], rtol=1e-14)
    assert etp.weight_numel == 0
    dot = o3.ElementwiseTensorProduct("5x1o + 5x1e", "10x1e", ["0e", "0o"])   # the reference's doctest
    assert str(dot.irreps_out) == "5x0o+5x0e" and len(dot.instructions) == 2
    with pytest.raises(AssertionError):
        o3.ElementwiseTensorProduct("3x0e", "4x0e")


def test_full_tensor_product_layout(golden_meta):
    """Output layout (sorted by (l, p)) and instruction list of `FullTensorProduct` against the reference's."""
    m = golden_meta["cases"]["tp_full"]
    ftp = o3.FullTensorProduct("2x0e+3x1o+1x2e", "2x0e+2x1o+1x1e")
    assert (str(ftp.irreps_in1), str(ftp.irreps_in2), str(ftp.irreps_out)) == (m["irreps_in1"], m["irreps_in2"], m["irreps_out"])
    got = [(i.i_in1, i.i_in2, i.i_out, i.connection_mode, i.has_weight) for i in ftp.instructions]
    assert got == [tuple(i[:5]) for i in m["instructions"]]
    assert np.allclose([i.path_weight for i in ftp.instructions], [i[5] for i in m["instructions"]], rtol=1e-14)
    only = o3.FullTensorProduct("2x1o", "3x1o", ["0e"])
    assert str(only.irreps_out) == "6x0e"


@pytest.mark.parametrize("name", ["square_full", "square_connected"])
def test_tensor_square_layout(golden_meta, name):
    """Paths, coefficients and output layout of `TensorSquare` against the reference's (golden meta)."""
    m = golden_meta["cases"][name]
    sq = o3.TensorSquare(*m["args"])
    assert str(sq.irreps_out) == m["irreps_out"] and sq.weight_numel == m["weight_numel"]
    got = [(i.i_in1, i.i_in2, i.i_out, i.connection_mode, i.has_weight) for i in sq.instructions]
    assert got == [tuple(i[:5]) for i in m["instructions"]]
    assert np.allclose([i.path_weight for i in sq.instructions], [i[5] for i in m["instructions"]], rtol=1e-14)
    with pytest.raises(ValueError):
        o3.TensorSquare("2x1o", "3x0e", filter_ir_out=["0e"])


def test_cta_split_is_proportional_and_bounded():
    """CTA counts the persistent contraction kernels get when another kernel keeps some SMs (_lib.tc_gemm_cta_limit)."""
    from e3nn_b200 import _lib

    work = [3000, 1000, 1000, 500, 10]
    for limit in (148, 124, 5, 3):
        n = _lib.cta_split(work, limit)
        assert len(n) == len(work) and min(n) >= 1 and sum(n) == max(limit, len(work))
    n = _lib.cta_split(work, 124)
    assert n[0] > n[1] >= n[3] >= n[4] and abs(n[0] - 124 * 3000 / sum(work)) <= 3
    with _lib.tc_gemm_cta_limit(100):
        assert _lib._tc_gemm_max_ctas == 100
        with _lib.tc_gemm_cta_limit(None):
            assert _lib._tc_gemm_max_ctas is None
        assert _lib._tc_gemm_max_ctas == 100
    assert _lib._tc_gemm_max_ctas is None
