"""The CPU oracle against outputs of the reference itself (tests/golden/*.npz)."""
import numpy as np
import pytest
import torch

from conftest import rel_err
from oracle import e3nn_oracle as orc

TP_CASES = [
    "tp_cfg1_uvw", "tp_cfg4_uvw", "tp_small_uvw", "tp_cfg3_uvu_15", "tp_cfg3_uvu_11", "tp_cfg5_uvu_23",
    "tp_small_uvu", "tp_mixed_shared", "tp_mixed_unshared", "tp_elementwise", "tp_uuu_mixed_shared", "tp_uuu_unshared",
    "tp_full", "tp_uvuv_mixed_unshared", "tp_rest_shared", "tp_rest_unshared",
]


def test_wigner_3j(golden):
    g = golden("wigner_3j")
    assert len(g) > 50
    for key, ref in g.items():
        l1, l2, l3 = map(int, key.split("_"))
        assert np.abs(orc.wigner_3j(l1, l2, l3).numpy() - ref).max() < 1e-12, key


def test_spherical_harmonics(golden):
    g = golden("spherical_harmonics")
    vec = torch.from_numpy(g["vec"]).double()
    for norm in ("component", "integral", "norm"):
        for normalize in (1, 0):
            for lmax in (3, 6):
                out = orc.spherical_harmonics(list(range(lmax + 1)), vec, bool(normalize), norm)
                ref = torch.from_numpy(g[f"l{lmax}_{norm}_{normalize}_f64"])
                assert rel_err(out, ref) < 1e-12, (norm, normalize, lmax)
    out = orc.spherical_harmonics([2, 0, 3, 2], vec, True, "norm")
    assert rel_err(out, torch.from_numpy(g["ls_2_0_3_2_norm_1_f64"])) < 1e-12
    out = orc.spherical_harmonics(list(range(9)), vec, True, "component")
    assert rel_err(out, torch.from_numpy(g["l8_component_1_f64"])) < 1e-12
    # the single literal vector of the reference's tests: zero input -> (1, 0, 0, 0)
    z = orc.spherical_harmonics([0, 1], torch.zeros(1, 3, dtype=torch.float64), True, "component")
    assert torch.equal(z, torch.tensor([[1.0, 0, 0, 0]], dtype=torch.float64))


@pytest.mark.parametrize("name", TP_CASES)
def test_tensor_product(golden, golden_meta, name):
    g, m = golden(name), golden_meta["cases"][name]
    ins = [tuple(i[:5]) for i in m["instructions"]]
    x1, x2, w = (torch.from_numpy(g[k]).double() for k in ("x1", "x2", "w"))
    # normalisation: recomputed from scratch, then compared with the reference's coefficients
    raw = [tuple(i) for i in _raw_instructions(name, m)]
    pws = orc.tp_path_weights(m["irreps_in1"], m["irreps_in2"], m["irreps_out"], raw, **m["norm_kwargs"])
    assert np.allclose(pws, [i[5] for i in m["instructions"]], rtol=1e-14, atol=0)
    out = orc.tensor_product(m["irreps_in1"], m["irreps_in2"], m["irreps_out"], ins, x1, x2, w,
                             shared_weights=m["shared_weights"], path_weights=pws)
    assert rel_err(out, torch.from_numpy(g["out_f64"])) < 1e-12


def _raw_instructions(name, m):
    """Instruction tuples as a user would write them (before normalisation)."""
    if name == "tp_mixed_shared":
        return [(0, 0, 0, "uvu", True), (1, 1, 0, "uvw", True), (1, 0, 1, "uvu", True), (1, 1, 2, "uvu", False),
                (2, 1, 1, "uvw", True, 2.5), (2, 0, 3, "uvu", True), (1, 1, 3, "uvw", True)]
    if name == "tp_uuu_mixed_shared":
        return [(0, 0, 0, "uuu", True), (1, 3, 1, "uuu", True), (1, 1, 2, "uuu", False), (1, 1, 2, "uuu", True),
                (2, 0, 3, "uvu", True), (1, 2, 0, "uvw", True), (1, 1, 3, "uvw", True, 0.5)]
    if name in ("tp_rest_shared", "tp_rest_unshared"):
        return [(0, 0, 0, "uvv", True), (1, 0, 1, "uuw", True), (1, 0, 2, "uvu<v", True), (1, 0, 1, "u<vw", True, 0.7),
                (1, 0, 3, "uuw", False), (2, 2, 4, "uvv", False), (0, 1, 5, "uvu<v", False)]
    if name == "tp_uvuv_mixed_unshared":
        return [(1, 0, 0, "uvuv", True), (1, 0, 1, "uvuv", False), (1, 1, 2, "uvu", True), (0, 1, 3, "uvuv", True, 2.0),
                (1, 0, 3, "uvw", True)]
    return [tuple(i[:5]) for i in m["instructions"]]


def test_layout_builders(golden_meta):
    m = golden_meta["cases"]["tp_cfg3_uvu_15"]
    mid, ins = orc.conv_uvu_layout("64x0e+64x1o+64x2e", "0e+1o+2e", [(0, 1), (0, -1), (1, 1), (1, -1), (2, 1), (2, -1)])
    assert orc.parse_irreps(mid) == orc.parse_irreps(m["irreps_out"])
    assert [list(i) for i in ins] == [i[:5] for i in m["instructions"]]
    assert m["weight_numel"] == 960 and orc.irreps_dim(orc.parse_irreps(mid)) == 3264
    m = golden_meta["cases"]["tp_cfg5_uvu_23"]
    mid, ins = orc.conv_uvu_layout("64x0e+64x1o+64x2e+64x3o", "0e+1o+2e+3o", [(0, 1), (1, -1), (2, 1), (3, -1)])
    assert [list(i) for i in ins] == [i[:5] for i in m["instructions"]]
    assert m["weight_numel"] == 1472 and orc.irreps_dim(orc.parse_irreps(mid)) == 6336
    m = golden_meta["cases"]["tp_cfg4_uvw"]
    ins = orc.fctp_instructions(m["irreps_in1"], m["irreps_in2"], m["irreps_out"])
    assert [list(i[:5]) for i in ins] == [i[:5] for i in m["instructions"]]
    assert m["weight_numel"] == 59392


@pytest.mark.parametrize("name", ["linear_cfg4", "linear_cfg5", "linear_small_bias"])
def test_linear(golden, golden_meta, name):
    g, m = golden(name), golden_meta["cases"][name]
    x, w, b = (torch.from_numpy(g[k]).double() for k in ("x", "w", "b"))
    ins = orc.linear_instructions(m["irreps_in"], m["irreps_out"])
    ref_ins = [i for i in m["instructions"] if i[0] != -1]
    assert [[i, o] for i, o, _ in ins] == [i[:2] for i in ref_ins]
    assert np.allclose([pw for _, _, pw in ins], [i[3] for i in ref_ins], rtol=1e-14)
    biases = None
    if m["biases"]:
        biases = [l == 0 and p == 1 for _, l, p in orc.parse_irreps(m["irreps_out"])]
    out = orc.linear(m["irreps_in"], m["irreps_out"], x, w, b, biases)
    assert rel_err(out, torch.from_numpy(g["out_f64"])) < 1e-12


def test_radial(golden):
    g = golden("radial")
    r = torch.from_numpy(g["r"]).double()
    b = orc.bessel(r, 8, 5.0)
    assert rel_err(b, torch.from_numpy(g["bessel_f64"])) < 1e-13
    assert abs(orc.silu_second_moment_scale() - float(g["silu_cst"])) < 1e-12
    out = orc.radial_mlp(b, [torch.from_numpy(g["w0"]), torch.from_numpy(g["w1"])])
    assert rel_err(out, torch.from_numpy(g["out_f64"])) < 1e-12


def test_conv_small(golden, golden_meta):
    g, m = golden("conv_small"), golden_meta["cases"]["conv_small"]
    ins = [tuple(i) for i in m["instructions"]]
    node_x, vec, w, lw = (torch.from_numpy(g[k]).double() for k in ("node_x", "vec", "w", "lin_w"))
    src, dst = torch.from_numpy(g["src"]), torch.from_numpy(g["dst"])
    agg = orc.conv_uvu(m["irreps_node"], m["irreps_edge"], m["irreps_mid"], ins, node_x, vec, src, dst, w,
                       m["num_nodes"], [0, 1, 2], scale=m["scale"], chunk=7)
    assert rel_err(agg, torch.from_numpy(g["agg_f64"])) < 1e-12
    out = orc.linear(m["irreps_mid"], m["irreps_node"], agg, lw)
    assert rel_err(out, torch.from_numpy(g["out_f64"])) < 1e-12
    perm, rowptr = orc.csr_from_dst(dst, m["num_nodes"])
    assert torch.equal(dst[perm], torch.sort(dst).values) and rowptr[-1] == dst.numel()


@pytest.mark.parametrize("name", ["gate_mixed", "gate_l3", "gate_abs_identity", "gate_no_scalars"])
def test_gate(golden, golden_meta, name):
    """Gate.forward of the reference (e3nn/nn/_gate.py:127-144) on its sorted input layout."""
    g, m = golden(name), golden_meta["cases"][name]
    x = torch.from_numpy(g["x"]).double()
    out = orc.gate(m["irreps_scalars"], m["act_scalars"], m["irreps_gates"], m["act_gates"], m["irreps_gated"], x)
    assert rel_err(out, torch.from_numpy(g["out_f64"])) < 1e-12


@pytest.mark.parametrize("name", ["activation_mixed", "activation_abs", "activation_identity", "activation_relu_sigmoid"])
def test_activation(golden, golden_meta, name):
    """Activation.forward of the reference (e3nn/nn/_activation.py:80-111)."""
    g, m = golden(name), golden_meta["cases"][name]
    out = orc.activation(m["irreps_in"], m["acts"], torch.from_numpy(g["x"]).double())
    assert rel_err(out, torch.from_numpy(g["out_f64"])) < 1e-12


def test_radial_bases(golden, golden_meta):
    """soft_one_hot_linspace (all bases, both cutoff flags) and smooth_cutoff against the reference's values."""
    g, m = golden("radial_bases"), golden_meta["cases"]["radial_bases"]
    r = torch.from_numpy(g["r"])
    assert rel_err(orc.smooth_cutoff(r / 5.0), torch.from_numpy(g["smooth_cutoff"])) < 1e-13
    for basis in ("gaussian", "cosine", "smooth_finite", "fourier", "bessel"):
        for cutoff in (False, True):
            out = orc.soft_one_hot_linspace(r, m["start"], m["end"], m["number"], basis, cutoff)
            assert rel_err(out, torch.from_numpy(g[f"{basis}_{int(cutoff)}"])) < 1e-12, (basis, cutoff)


@pytest.mark.parametrize("name", ["square_full", "square_connected"])
def test_tensor_square(golden, golden_meta, name):
    """The oracle's 'uvuv' / 'uvu<v' / 'uuu' / 'uvw' / 'u<vw' / 'uuw' paths on the reference's TensorSquare outputs."""
    g, m = golden(name), golden_meta["cases"][name]
    ins = [tuple(i[:5]) for i in m["instructions"]]
    x, w = torch.from_numpy(g["x"]).double(), torch.from_numpy(g["w"]).double()
    irreps_in = m["args"][0]
    out = orc.tensor_product(irreps_in, irreps_in, m["irreps_out"], ins, x, x, w, shared_weights=True,
                             path_weights=[i[5] for i in m["instructions"]])
    assert rel_err(out, torch.from_numpy(g["out_f64"])) < 1e-12
