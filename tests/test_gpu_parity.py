"""Parity of the CUDA kernels (called through the C ABI) with the CPU oracle and the golden vectors.

Tolerance (fp32 kernels): max|out - ref64| <= 1e-5 x rms(ref64), the bound stated for this path.
Index work (CSR) must be bit-exact.
"""
import copy

import numpy as np
import pytest
import torch

import _cases
import e3nn_b200
from conftest import fp32_bound, rel_err
from e3nn_b200 import layouts, o3
from oracle import e3nn_oracle as orc

pytestmark = pytest.mark.gpu
TOL = 1e-5
DEV = "cuda"


def _ins(tp):
    return [(i.i_in1, i.i_in2, i.i_out, i.connection_mode, i.has_weight) for i in tp.instructions]


def _pws(tp):
    return [i.path_weight for i in tp.instructions]


def _oracle_tp(tp, x1, x2, w):
    return orc.tensor_product(str(tp.irreps_in1), str(tp.irreps_in2), str(tp.irreps_out), _ins(tp), x1, x2, w,
                              tp.shared_weights, path_weights=_pws(tp))


# ----------------------------------------------------------------------------- spherical harmonics
def test_sh_golden(golden):
    g = golden("spherical_harmonics")
    vec = torch.from_numpy(g["vec"]).to(DEV)
    for norm in ("component", "integral", "norm"):
        for normalize in (1, 0):
            for lmax in (3, 6):
                out = o3.spherical_harmonics(list(range(lmax + 1)), vec, bool(normalize), norm)
                ref = torch.from_numpy(g[f"l{lmax}_{norm}_{normalize}_f64"])
                assert rel_err(out.cpu(), ref) < TOL, (norm, normalize, lmax)
    out = o3.spherical_harmonics([2, 0, 3, 2], vec, True, "norm")
    assert rel_err(out.cpu(), torch.from_numpy(g["ls_2_0_3_2_norm_1_f64"])) < TOL
    out = o3.spherical_harmonics(list(range(9)), vec, True, "component")
    assert rel_err(out.cpu(), torch.from_numpy(g["l8_component_1_f64"])) < TOL
    z = o3.spherical_harmonics([0, 1], torch.zeros(1, 3, device=DEV), True, "component")
    assert torch.equal(z.cpu(), torch.tensor([[1.0, 0, 0, 0]]))


@pytest.mark.parametrize("lmax", [0, 1, 2, 3, 4, 7, 12])
def test_sh_oracle_and_backward(lmax):
    torch.manual_seed(lmax)
    n = 1000 + 37 * lmax  # ragged last tile
    vec = torch.randn(n, 3)
    vec[5] = 0.0
    ls = list(range(lmax + 1))
    for normalize in (True, False):
        base = vec if normalize else vec * 0.5
        v = base.clone().to(DEV).requires_grad_(True)
        out = o3.spherical_harmonics(ls, v, normalize, "component")
        v64 = base.double().requires_grad_(True)
        ref = orc.spherical_harmonics(ls, v64, normalize, "component")
        # the generated fp32 polynomials (powers of x, y, z up to degree l) lose about one digit by l = 12, where the
        # oracle's recurrence does not; the 1e-5 bound is the l <= 8 path's
        assert rel_err(out.detach().cpu(), ref.detach()) < (TOL if lmax <= 8 else 5e-5)
        g = torch.randn(n, (lmax + 1) ** 2)
        g[5] = 0.0  # the zero vector has an unbounded derivative when normalised
        out.backward(g.to(DEV))
        if lmax == 0:  # Y^0 is constant: zero gradient, and the oracle's output has no graph
            assert torch.all(v.grad == 0)
            continue
        ref.backward(g.double())
        assert rel_err(v.grad.cpu(), v64.grad) < 2e-5      # measured: 7.8e-6 at lmax 12


def test_sh_batch_shapes_and_module():
    sh = o3.SphericalHarmonics("0e+1o+2e+3o", True, "component")
    x = torch.randn(3, 1, 5, 3, device=DEV)
    assert sh(x).shape == (3, 1, 5, 16)
    assert o3.spherical_harmonics(2, torch.randn(0, 3, device=DEV), True).shape == (0, 5)
    with pytest.raises(TypeError):
        sh(x.double())


def test_sh_equivariance():
    torch.manual_seed(0)
    irreps = o3.Irreps.spherical_harmonics(4)
    R = o3.rand_matrix()
    x = torch.randn(64, 3)
    y1 = o3.spherical_harmonics(irreps, (x @ R.T).to(DEV), True, "component").cpu()
    y2 = o3.spherical_harmonics(irreps, x.to(DEV), True, "component").cpu() @ irreps.D_from_matrix(R).T
    assert (y1 - y2).abs().max() < 1e-4


# ----------------------------------------------------------------------------- tensor products
TP_CASES = [
    "tp_cfg1_uvw", "tp_cfg4_uvw", "tp_small_uvw", "tp_cfg3_uvu_15", "tp_cfg3_uvu_11", "tp_cfg5_uvu_23",
    "tp_small_uvu", "tp_mixed_shared", "tp_mixed_unshared", "tp_elementwise", "tp_uuu_mixed_shared", "tp_uuu_unshared",
    "tp_full", "tp_uvuv_mixed_unshared", "tp_rest_shared", "tp_rest_unshared",
]


def _tp_from_meta(name, m):
    ins = [tuple(i[:5]) for i in m["instructions"]]
    if name == "tp_mixed_shared":
        ins[4] = ins[4] + (2.5,)
    if name == "tp_uuu_mixed_shared":
        ins[6] = ins[6] + (0.5,)
    if name == "tp_uvuv_mixed_unshared":
        ins[3] = ins[3] + (2.0,)
    if name in ("tp_rest_shared", "tp_rest_unshared"):
        ins[3] = ins[3] + (0.7,)
    return o3.TensorProduct(m["irreps_in1"], m["irreps_in2"], m["irreps_out"], ins, internal_weights=False,
                            shared_weights=m["shared_weights"], **m["norm_kwargs"])


@pytest.mark.parametrize("name", TP_CASES)
def test_tp_golden(golden, golden_meta, name):
    g, m = golden(name), golden_meta["cases"][name]
    tp = _tp_from_meta(name, m)
    x1, x2, w = (torch.from_numpy(g[k]).to(DEV) for k in ("x1", "x2", "w"))
    out = tp(x1, x2, w)
    ref = torch.from_numpy(g["out_f64"])
    assert rel_err(out.cpu(), ref) < TOL
    # the reference's own fp32 result sits at a few 1e-6 from the same fp64 run
    assert rel_err(torch.from_numpy(g["out_f32"]), ref) < TOL


@pytest.mark.parametrize("name", ["tp_cfg3_uvu_15", "tp_small_uvu", "tp_mixed_shared", "tp_mixed_unshared", "tp_cfg5_uvu_23"])
def test_tp_uvu_backward(golden, golden_meta, name):
    g, m = golden(name), golden_meta["cases"][name]
    ins = [tuple(i[:5]) for i in m["instructions"] if i[3] == "uvu"]
    tp = o3.TensorProduct(m["irreps_in1"], m["irreps_in2"], m["irreps_out"], ins, internal_weights=False,
                          shared_weights=m["shared_weights"], **m["norm_kwargs"])
    torch.manual_seed(1)
    Z = 37
    x1, x2 = torch.randn(Z, tp.irreps_in1.dim), torch.randn(Z, tp.irreps_in2.dim)
    w = torch.randn(tp.weight_numel) if tp.shared_weights else torch.randn(Z, tp.weight_numel)
    a, b, c = (t.clone().to(DEV).requires_grad_(True) for t in (x1, x2, w))
    out = tp(a, b, c)
    a64, b64, c64 = (t.double().requires_grad_(True) for t in (x1, x2, w))
    ref = _oracle_tp(tp, a64, b64, c64)
    assert rel_err(out.detach().cpu(), ref.detach()) < TOL
    go = torch.randn_like(ref)
    ref.backward(go)
    out.backward(go.float().to(DEV))
    assert rel_err(a.grad.cpu(), a64.grad) < TOL
    assert rel_err(b.grad.cpu(), b64.grad) < TOL
    assert rel_err(c.grad.cpu(), c64.grad) < TOL   # shared weights: float atomics over rows, measured 1.2e-6


def test_tp_cfg1_full_batch():
    """benchmark case 1 (10,000-row fully connected product) as stated: 10,000 rows, internal weights ~ N(0,1), seed 0."""
    torch.manual_seed(0)
    tp = o3.FullyConnectedTensorProduct("32x0e+32x1o+32x2e", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e")
    x, y = torch.randn(10000, 288), torch.randn(10000, 9)
    out = tp.to(DEV)(x.to(DEV), y.to(DEV))
    ref = _oracle_tp(tp, x.double(), y.double(), tp.weight.detach().cpu().double())
    assert rel_err(out.detach().cpu(), ref) < TOL


def test_tp_broadcasting_and_weight_list():
    torch.manual_seed(0)
    tp = layouts.conv_tensor_product("8x0e+8x1o+8x2e", "0e+1o+2e", layouts.ALL_L2)
    x = torch.randn(1, 5, tp.irreps_in1.dim)
    y = torch.randn(4, 1, tp.irreps_in2.dim)
    w = torch.randn(4, 5, tp.weight_numel)
    out = tp(x.to(DEV), y.to(DEV), w.to(DEV))
    assert out.shape == (4, 5, tp.irreps_out.dim)
    ref = _oracle_tp(tp, x.expand(4, 5, -1).reshape(20, -1).double(), y.expand(4, 5, -1).reshape(20, -1).double(),
                     w.reshape(20, -1).double())
    assert rel_err(out.cpu().reshape(20, -1), ref) < TOL
    # weights given as a list of per-path tensors (flat batch, as the reference flattens them)
    xf, yf, wf = x.expand(4, 5, -1).reshape(20, -1), y.expand(4, 5, -1).reshape(20, -1), w.reshape(20, -1)
    views = [v.contiguous() for v in tp.weight_views(wf.to(DEV))]
    assert torch.equal(tp(xf.to(DEV), yf.to(DEV), views), out.reshape(20, -1))
    assert tp(x[:, :0].to(DEV), y[:, :0].to(DEV), w[:, :0].to(DEV)).shape == (4, 0, tp.irreps_out.dim)


def test_tp_bilinear_and_equivariant():
    torch.manual_seed(0)
    tp = o3.FullyConnectedTensorProduct("4x0e+3x1o+2x2e", "0e+1o+2e", "3x0e+2x1o+2x1e+1x2e+1x3o").to(DEV)
    x1, x2, y = (t.randn(16, -1).to(DEV) for t in (tp.irreps_in1, tp.irreps_in1, tp.irreps_in2))
    lhs = tp(x1 + 1.7 * x2, y)
    rhs = tp(x1, y) + 1.7 * tp(x2, y)
    assert (lhs - rhs).abs().max() < 1e-4
    R = o3.rand_matrix()
    D1, D2, Do = (ir.D_from_matrix(R).to(DEV) for ir in (tp.irreps_in1, tp.irreps_in2, tp.irreps_out))
    assert (tp(x1 @ D1.T, y @ D2.T) - tp(x1, y) @ Do.T).abs().max() < 1e-4


def test_tp_state_dict_roundtrip():
    tp = o3.FullyConnectedTensorProduct("4x0e+2x1o", "0e+1o", "4x0e+2x1o").to(DEV)
    tp2 = o3.FullyConnectedTensorProduct("4x0e+2x1o", "0e+1o", "4x0e+2x1o").to(DEV)
    tp2.load_state_dict(tp.state_dict())
    x, y = tp.irreps_in1.randn(8, -1).to(DEV), tp.irreps_in2.randn(8, -1).to(DEV)
    assert torch.equal(tp(x, y), tp2(x, y))
    assert torch.equal(copy.deepcopy(tp)(x, y), tp(x, y))


# ----------------------------------------------------------------------------- Linear
@pytest.mark.parametrize("name", ["linear_cfg4", "linear_cfg5", "linear_small_bias"])
def test_linear_golden(golden, golden_meta, name):
    g, m = golden(name), golden_meta["cases"][name]
    lin = o3.Linear(m["irreps_in"], m["irreps_out"], biases=m["biases"], internal_weights=False)
    x, w, b = (torch.from_numpy(g[k]).to(DEV) for k in ("x", "w", "b"))
    out = lin(x, w, b)
    assert rel_err(out.cpu(), torch.from_numpy(g["out_f64"])) < TOL


def test_linear_bias_placement_and_input_grad():
    # literal vector of the reference's test (tests/o3/linear_test.py:70-78)
    lin = o3.Linear("2x0e+1o+3x0e", "0e+1o+3x0e", biases=[True, False, True], internal_weights=True).to(DEV)
    with torch.no_grad():
        lin.weight.zero_()
        lin.bias.copy_(torch.tensor([1.0, 2.0, 3.0, 4.0]))
    out = lin(torch.randn(2, 8, device=DEV))
    assert torch.equal(out.cpu(), torch.tensor([[1.0, 0, 0, 0, 2, 3, 4]] * 2))
    torch.manual_seed(0)
    lin = o3.Linear("16x0e+8x1o+4x2e", "8x0e+8x1o+4x2e").to(DEV)
    x = torch.randn(33, lin.irreps_in.dim)
    xg = x.clone().to(DEV).requires_grad_(True)
    out = lin(xg)
    x64 = x.double().requires_grad_(True)
    ref = orc.linear(str(lin.irreps_in), str(lin.irreps_out), x64, lin.weight.detach().cpu().double())
    assert rel_err(out.detach().cpu(), ref.detach()) < TOL
    go = torch.randn_like(ref)
    ref.backward(go)
    lin.weight.requires_grad_(False)
    out = lin(xg)
    out.backward(go.float().to(DEV))
    assert rel_err(xg.grad.cpu(), x64.grad) < TOL


# ----------------------------------------------------------------------------- CSR (bit-exact)
@pytest.mark.parametrize("E,N", [(0, 5), (1, 1), (1000, 1), (5000, 37), (100_000, 70_000), (300_000, 255), (2049, 257)])
def test_csr_bit_exact(E, N):
    torch.manual_seed(E + N)
    dst = torch.randint(0, N, (E,))
    if E > 10:
        dst[dst == 3] = 4  # an empty row in the middle
    perm, rowptr = e3nn_b200.csr_from_dst(dst.to(DEV), N)
    ref_perm, ref_rowptr = orc.csr_from_dst(dst, N)
    assert torch.equal(perm.cpu(), ref_perm)
    assert torch.equal(rowptr.cpu(), ref_rowptr)


def test_csr_rejects_bad_index():
    dst = torch.tensor([0, 1, 7, 2])
    with pytest.raises(IndexError):
        e3nn_b200.csr_from_dst(dst.to(DEV), 4)
    with pytest.raises(NotImplementedError):
        e3nn_b200.csr_from_dst(dst, 8)


# ----------------------------------------------------------------------------- fused convolution
def test_conv_golden(golden, golden_meta):
    g, m = golden("conv_small"), golden_meta["cases"]["conv_small"]
    tp = o3.TensorProduct(m["irreps_node"], m["irreps_edge"], m["irreps_mid"], [tuple(i) for i in m["instructions"]],
                          internal_weights=False, shared_weights=False)
    node_x, vec, w, lw = (torch.from_numpy(g[k]).to(DEV) for k in ("node_x", "vec", "w", "lin_w"))
    src, dst = torch.from_numpy(g["src"]).to(DEV), torch.from_numpy(g["dst"]).to(DEV)
    perm, rowptr = e3nn_b200.csr_from_dst(dst, m["num_nodes"])
    agg = e3nn_b200.conv_uvu(tp, node_x, vec, src, rowptr, w, perm=perm, scale=m["scale"], edge_attr_is_vector=True)
    assert rel_err(agg.cpu(), torch.from_numpy(g["agg_f64"])) < TOL
    assert torch.all(agg[-2:] == 0)  # rows without incoming edges
    lin = o3.Linear(m["irreps_mid"], m["irreps_node"], internal_weights=False)
    assert rel_err(lin(agg, lw).cpu(), torch.from_numpy(g["out_f64"])) < TOL
    # same thing with precomputed spherical harmonics rows
    y = o3.spherical_harmonics([0, 1, 2], vec, True, "component")
    agg2 = e3nn_b200.conv_uvu(tp, node_x, y, src, rowptr, w, perm=perm, scale=m["scale"])
    assert rel_err(agg2.cpu(), torch.from_numpy(g["agg_f64"])) < TOL


@pytest.mark.parametrize("idx", range(6))
def test_conv_random_layouts_forward_backward(idx):
    tp = _cases.conv_tps()[idx]
    torch.manual_seed(idx)
    N, E = 50, 700
    node_x = torch.randn(N, tp.irreps_in1.dim)
    vec = torch.randn(E, 3)
    src, dst = torch.randint(0, N, (E,)), torch.randint(0, N - 3, (E,))
    w = torch.randn(E, tp.weight_numel)
    lmax = tp.irreps_in2.lmax
    perm, rowptr = e3nn_b200.csr_from_dst(dst.to(DEV), N)
    vg = vec.clone().to(DEV).requires_grad_(True)
    wg = w.clone().to(DEV).requires_grad_(True)
    xg = node_x.clone().to(DEV).requires_grad_(True)
    out = e3nn_b200.conv_uvu(tp, xg, vg, src.to(DEV), rowptr, wg, perm=perm, scale=0.3,
                             edge_attr_is_vector=True)
    v64, w64, x64 = vec.double().requires_grad_(True), w.double().requires_grad_(True), node_x.double().requires_grad_(True)
    ref = orc.conv_uvu(str(tp.irreps_in1), str(tp.irreps_in2), str(tp.irreps_out), _ins(tp), x64, v64, src,
                       dst, w64, N, list(range(lmax + 1)), scale=0.3)
    assert rel_err(out.detach().cpu(), ref.detach()) < TOL
    go = torch.randn_like(ref)
    ref.backward(go)
    out.backward(go.float().to(DEV))
    assert rel_err(wg.grad.cpu(), w64.grad) < TOL
    assert rel_err(vg.grad.cpu(), v64.grad) < TOL      # measured 4.0e-6
    # node features: the transpose of the gather, accumulated with float atomics (order not fixed)
    assert rel_err(xg.grad.cpu(), x64.grad) < TOL
    # only the node features require a gradient: the weight / vector kernel is skipped
    x2 = node_x.clone().to(DEV).requires_grad_(True)
    out2 = e3nn_b200.conv_uvu(tp, x2, vec.to(DEV), src.to(DEV), rowptr, w.to(DEV), perm=perm, scale=0.3, edge_attr_is_vector=True)
    out2.backward(go.float().to(DEV))
    assert rel_err(x2.grad.cpu(), x64.grad) < TOL


def test_conv_deterministic_and_sorted_equals_permuted():
    torch.manual_seed(0)
    tp = layouts.conv_tensor_product("8x0e+8x1o+8x2e", "0e+1o+2e", layouts.ALL_L2)
    N, E = 300, 9000
    node_x = torch.randn(N, tp.irreps_in1.dim, device=DEV)
    vec = torch.randn(E, 3, device=DEV)
    src, dst = torch.randint(0, N, (E,), device=DEV), torch.randint(0, N, (E,), device=DEV)
    w = torch.randn(E, tp.weight_numel, device=DEV)
    perm, rowptr = e3nn_b200.csr_from_dst(dst, N)
    a = e3nn_b200.conv_uvu(tp, node_x, vec, src, rowptr, w, perm=perm, edge_attr_is_vector=True)
    b = e3nn_b200.conv_uvu(tp, node_x, vec, src, rowptr, w, perm=perm, edge_attr_is_vector=True)
    assert torch.equal(a, b)  # fixed summation order: bitwise reproducible
    c = e3nn_b200.conv_uvu(tp, node_x, vec[perm], src[perm], rowptr, w[perm], perm=None, edge_attr_is_vector=True)
    assert torch.equal(a, c)


def test_conv_cfg3_layout_medium():
    """benchmark case 3 (l <= 2 fused convolution) layout (15 paths), reduced graph: 512 nodes, in-degree 32, random sources."""
    torch.manual_seed(0)
    tp = layouts.bench_conv_tp("cfg3_15")
    N, deg = 512, 32
    E = N * deg
    dst = torch.arange(E) // deg
    src = torch.randint(0, N, (E,))
    node_x = torch.randn(N, 576)
    vec = torch.nn.functional.normalize(torch.randn(E, 3), dim=-1)
    w = torch.randn(E, 960)
    rowptr = torch.arange(0, E + 1, deg)
    out = e3nn_b200.conv_uvu(tp, node_x.to(DEV), vec.to(DEV), src.to(DEV), rowptr.to(DEV), w.to(DEV),
                             scale=deg ** -0.5, edge_attr_is_vector=True)
    ref = orc.conv_uvu(str(tp.irreps_in1), str(tp.irreps_in2), str(tp.irreps_out), _ins(tp), node_x.double(),
                       vec.double(), src, dst, w.double(), N, [0, 1, 2], scale=deg ** -0.5, chunk=4096)
    assert rel_err(out.cpu(), ref) < TOL


# ----------------------------------------------------------------------------- tensor-core 'uvw' (tf32)
TOL_TF32 = 2e-2  # stated bound for the tf32 tensor-core path


@pytest.mark.parametrize("layout", [
    ("32x0e+32x1o+32x2e", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e"),          # benchmark case 1 (10,000-row fully connected product)
    ("128x0e+64x1o+32x2e", "0e+1o+2e+3o", "128x0e+64x1o+32x2e"),          # benchmark case 4 (1,048,576-row fully connected product)
] + _cases.UVW_TC_EXTRA_LAYOUTS)
@pytest.mark.parametrize("Z", [1, 300, 5000])
def test_uvw_tensor_core(layout, Z):
    torch.manual_seed(Z)
    tp = o3.FullyConnectedTensorProduct(*layout, math_mode="tf32").to(DEV)
    with torch.no_grad():
        for view in tp.weight_views():
            view.div_((view.shape[0] * view.shape[1]) ** 0.5)  # ~N(0,1)/sqrt(fan_in) as in config 4
    x, y = torch.randn(Z, tp.irreps_in1.dim), torch.randn(Z, tp.irreps_in2.dim)
    with torch.no_grad():
        out = tp(x.to(DEV), y.to(DEV))
        torch.cuda.synchronize()
    e3nn_b200.check_status()   # raises if a bounded wait inside the kernel gave up
    ref = _oracle_tp(tp, x.double(), y.double(), tp.weight.detach().cpu().double())
    err = rel_err(out.cpu(), ref)
    assert err < TOL_TF32, err
    assert err > 1e-6  # tf32 rounding must be visible: guards against silently running the fp32 kernel


# ----------------------------------------------------------------------------- bulk-copy pipelined convolution kernel
@pytest.mark.parametrize("layout", ["cfg3_15", "cfg3_11", "cfg5_23"])
def test_conv_pipelined_kernel(layout):
    """64-channel layouts take the bulk-copy (TMA) pipelined kernel when the edges are sorted by
    destination; it must agree with the oracle and with the direct-load kernel on a ragged graph
    (empty rows, rows of one edge, one long row)."""
    torch.manual_seed(3)
    tp = layouts.bench_conv_tp(layout)
    mod = tp._uvu_module()
    assert mod.lib.e3b_conv_select(0) == 1, "module was generated without the pipelined kernel"
    N = 700
    deg = torch.randint(0, 9, (N,))
    deg[5] = 0
    deg[6] = 1
    deg[77] = 96
    deg[N - 1] = 0
    dst = torch.repeat_interleave(torch.arange(N), deg)
    E = dst.numel()
    rowptr = torch.zeros(N + 1, dtype=torch.int64)
    rowptr[1:] = torch.cumsum(deg, 0)
    src = torch.randint(0, N, (E,))
    node_x = torch.randn(N, tp.irreps_in1.dim)
    vec = torch.randn(E, 3)
    vec[3] = 0.0
    w = torch.randn(E, tp.weight_numel)
    args = (tp, node_x.to(DEV), vec.to(DEV), src.to(DEV), rowptr.to(DEV), w.to(DEV))
    fast = e3nn_b200.conv_uvu(*args, scale=0.7, edge_attr_is_vector=True, check_indices=True)
    mod.lib.e3b_conv_select(1)
    try:
        slow = e3nn_b200.conv_uvu(*args, scale=0.7, edge_attr_is_vector=True)
    finally:
        mod.lib.e3b_conv_select(0)
    lmax = tp.irreps_in2.lmax
    ref = orc.conv_uvu(str(tp.irreps_in1), str(tp.irreps_in2), str(tp.irreps_out), _ins(tp), node_x.double(),
                       vec.double(), src, dst, w.double(), N, list(range(lmax + 1)), scale=0.7, chunk=2048)
    err_fast, err_slow = rel_err(fast.cpu(), ref), rel_err(slow.cpu(), ref)
    # one row sums 96 messages sequentially in fp32 while most rows sum ~4, and the metric divides by
    # the global RMS: the long row dominates the error of both kernels alike
    assert err_fast < 2e-5 and err_slow < 2e-5, (err_fast, err_slow)
    assert rel_err(fast.cpu(), slow.cpu()) < 2e-5   # two fp32 summation orders of the same 96-message row
    assert torch.all(fast[5] == 0) and torch.all(fast[N - 1] == 0)
    again = e3nn_b200.conv_uvu(*args, scale=0.7, edge_attr_is_vector=True)
    assert torch.equal(fast, again)  # fixed summation order
    # gradients w.r.t. the per-edge weights and the edge vectors: pipelined kernel vs oracle autograd
    vg = vec.clone().to(DEV).requires_grad_(True)
    wg = w.clone().to(DEV).requires_grad_(True)
    xg = node_x.clone().to(DEV).requires_grad_(True)
    out_g = e3nn_b200.conv_uvu(tp, xg, vg, src.to(DEV), rowptr.to(DEV), wg, scale=0.7, edge_attr_is_vector=True)
    go = torch.randn(N, tp.irreps_out.dim)
    out_g.backward(go.to(DEV))
    v64, w64, x64 = vec.double().requires_grad_(True), w.double().requires_grad_(True), node_x.double().requires_grad_(True)
    ref_g = orc.conv_uvu(str(tp.irreps_in1), str(tp.irreps_in2), str(tp.irreps_out), _ins(tp), x64, v64, src, dst,
                         w64, N, list(range(lmax + 1)), scale=0.7, chunk=2048)
    ref_g.backward(go.double())
    assert rel_err(wg.grad.cpu(), w64.grad) < TOL
    # node-feature gradient: pipelined kernel vs oracle, and vs the direct-load kernel (atomics: not bitwise)
    assert rel_err(xg.grad.cpu(), x64.grad) < TOL
    mod.lib.e3b_conv_select(1)
    try:
        xs = node_x.clone().to(DEV).requires_grad_(True)
        e3nn_b200.conv_uvu(tp, xs, vec.to(DEV), src.to(DEV), rowptr.to(DEV), w.to(DEV), scale=0.7,
                           edge_attr_is_vector=True).backward(go.to(DEV))
    finally:
        mod.lib.e3b_conv_select(0)
    assert rel_err(xg.grad.cpu(), xs.grad.cpu()) < TOL
    gv, gv_ref = vg.grad.cpu(), v64.grad.clone()
    gv[3] = 0.0      # the zero vector has an unbounded derivative under normalisation
    gv_ref[3] = 0.0
    assert rel_err(gv, gv_ref) < TOL       # measured 4.0e-6
    bad = src.clone()
    bad[10] = N + 5
    with pytest.raises(IndexError):
        e3nn_b200.conv_uvu(tp, node_x.to(DEV), vec.to(DEV), bad.to(DEV), rowptr.to(DEV), w.to(DEV),
                           edge_attr_is_vector=True, check_indices=True)


# ----------------------------------------------------------------------------- interaction block (forward + d/d positions)
@pytest.mark.parametrize("irreps,lmax", [("8x0e+8x1o+8x2e", 2), ("64x0e+64x1o+64x2e+64x3o", 3)])
def test_interaction_block_forward_and_position_gradient(irreps, lmax):
    """benchmark case 5 (interaction block) at reduced size: periodic box at density 0.05, 5 A cutoff, Bessel(8) -> 64 -> weights,
    SH lmax, 'uvu', scatter / sqrt(n), Linear; loss = sum(out * G); gradient w.r.t. the positions."""
    from e3nn_b200 import nn as bnn

    torch.manual_seed(11)
    n_atoms = 600
    box = (n_atoms / 0.05) ** (1 / 3)
    pos = torch.rand(n_atoms, 3) * box
    src, dst, shift = bnn.radius_graph_pbc(pos, box, 5.0)
    num_neighbors = src.numel() / n_atoms
    block = bnn.InteractionBlock(irreps, lmax, num_basis=8, hidden=64, r_max=5.0, num_neighbors=num_neighbors,
                                 linear_math_mode="fp32", radial_math_mode="fp32").to(DEV)
    node_x = torch.randn(n_atoms, block.irreps_node.dim)
    G = torch.randn(n_atoms, block.irreps_out.dim)
    perm, rowptr = e3nn_b200.csr_from_dst(dst.to(DEV), n_atoms)
    assert torch.equal(perm.cpu(), torch.arange(src.numel()))  # the neighbour list is already sorted by destination

    p = pos.clone().to(DEV).requires_grad_(True)
    for prm in block.parameters():
        prm.requires_grad_(False)
    out = block(p, node_x.to(DEV), src.to(DEV), dst.to(DEV), rowptr, shift.to(DEV))
    (out * G.to(DEV)).sum().backward()

    tp = block.tp
    p64 = pos.double().requires_grad_(True)
    ref = orc.interaction_block(
        str(tp.irreps_in1), str(tp.irreps_in2), str(tp.irreps_out), _ins(tp), str(block.irreps_out), p64,
        node_x.double(), src, dst, shift.double(),
        [block.fc.layer0.weight.detach().cpu().double(), block.fc.layer1.weight.detach().cpu().double()],
        block.lin.weight.detach().cpu().double(), 8, 5.0, num_neighbors, list(range(lmax + 1)), chunk=4096)
    (ref * G.double()).sum().backward()
    # context: the same chain evaluated by the oracle in fp32 on the CPU.  With ~26 x 23 x 64 products per
    # output behind a 64-term fp32 radial network, fp32 itself sits at about 1e-5 x RMS on this block;
    # the kernels must not be worse than that.
    p32 = pos.clone().requires_grad_(True)
    ref32 = orc.interaction_block(
        str(tp.irreps_in1), str(tp.irreps_in2), str(tp.irreps_out), _ins(tp), str(block.irreps_out), p32,
        node_x, src, dst, shift,
        [block.fc.layer0.weight.detach().cpu(), block.fc.layer1.weight.detach().cpu()],
        block.lin.weight.detach().cpu(), 8, 5.0, num_neighbors, list(range(lmax + 1)), chunk=4096)
    (ref32 * G).sum().backward()
    err32 = rel_err(ref32.detach(), ref.detach())
    err = rel_err(out.detach().cpu(), ref.detach())
    assert err < fp32_bound(err32), (err, err32)
    # gradient: long chain through sin/r, silu and the SH Jacobian; bounded by the same chain in fp32 on the CPU
    gerr32 = rel_err(p32.grad, p64.grad)
    assert rel_err(p.grad.cpu(), p64.grad) < fp32_bound(gerr32), (rel_err(p.grad.cpu(), p64.grad), gerr32)
    # default mode of the block: the Linear on the tensor cores with hi/lo-split tf32 operands
    fast = bnn.InteractionBlock(irreps, lmax, num_basis=8, hidden=64, r_max=5.0, num_neighbors=num_neighbors).to(DEV)
    fast.load_state_dict(block.state_dict())
    for prm in fast.parameters():
        prm.requires_grad_(False)
    p2 = pos.clone().to(DEV).requires_grad_(True)
    out2 = fast(p2, node_x.to(DEV), src.to(DEV), dst.to(DEV), rowptr, shift.to(DEV))
    (out2 * G.to(DEV)).sum().backward()
    # hi/lo-split tf32 operands (the benchmark's mode): measured 2.1e-5 / 2.2e-5
    assert rel_err(out2.detach().cpu(), ref.detach()) < 5e-5
    assert rel_err(p2.grad.cpu(), p64.grad) < 5e-5


# ----------------------------------------------------------------------------- self-connection with node attributes
@pytest.mark.parametrize("mode", ["fp32", "tf32x3"])
def test_self_connection_with_node_attributes(mode):
    """FullyConnectedTensorProduct(node, node_attr, node) with a multi-channel scalar second operand: the
    self-connection / lin1 / lin2 of e3nn/nn/models/v2106/points_convolution.py:56-58,89-92 ('uvw', in2 = 4x0e)."""
    torch.manual_seed(4)
    node, attr = "32x0e+32x1o+16x2e", "4x0e"
    tp = o3.FullyConnectedTensorProduct(node, attr, node, math_mode=mode).to(DEV)
    x = torch.randn(333, tp.irreps_in1.dim)
    a = torch.nn.functional.one_hot(torch.randint(0, 4, (333,)), 4).float()
    out = tp(x.to(DEV), a.to(DEV))
    ref = _oracle_tp(tp, x.double(), a.double(), tp.weight.detach().cpu().double())
    assert rel_err(out.detach().cpu(), ref) < (TOL if mode == "fp32" else TOL_TF32X3)


# ----------------------------------------------------------------------------- two interaction blocks with a Gate between them
@pytest.mark.parametrize("mode", ["fp32", "tf32x3"])
def test_two_layer_network_forward_and_gradients(mode):
    """block -> Gate -> block, the composition of gate_points_2101.py:275-334: output, gradient w.r.t. the positions
    (through both blocks) and w.r.t. the input features (through the convolution's node-feature gradient, the Gate
    and both Linears) against the same chain evaluated by the oracle in fp64."""
    from e3nn_b200 import nn as bnn

    torch.manual_seed(23)
    n_atoms = 400
    box = (n_atoms / 0.05) ** (1 / 3)
    pos = torch.rand(n_atoms, 3) * box
    src, dst, shift, rowptr = bnn.neighbor_list_pbc(pos.to(DEV), box, 5.0)
    nn_avg = src.numel() / n_atoms
    node, gate_in = "16x0e+16x1o+16x2e", "48x0e+16x1o+16x2e"
    kw = dict(num_basis=8, hidden=64, r_max=5.0, num_neighbors=nn_avg, linear_math_mode=mode, radial_math_mode=mode)
    b1 = bnn.InteractionBlock(node, 2, irreps_out=gate_in, **kw).to(DEV)
    gate = bnn.Gate("16x0e", [torch.nn.functional.silu], "32x0e", [torch.sigmoid], "16x1o+16x2e").to(DEV)
    b2 = bnn.InteractionBlock(node, 2, **kw).to(DEV)
    assert str(gate.irreps_in) == gate_in and str(gate.irreps_out) == node
    for m in (b1, b2):
        for prm in m.parameters():
            prm.requires_grad_(False)
    x = torch.randn(n_atoms, b1.irreps_node.dim)
    G = torch.randn(n_atoms, b2.irreps_out.dim)
    p = pos.clone().to(DEV).requires_grad_(True)
    xg = x.clone().to(DEV).requires_grad_(True)
    h = gate(b1(p, xg, src, dst, rowptr, shift))
    out = b2(p, h, src, dst, rowptr, shift)
    (out * G.to(DEV)).sum().backward()

    p64, x64 = pos.double().requires_grad_(True), x.double().requires_grad_(True)
    srcc, dstc, shiftc = src.cpu(), dst.cpu(), shift.cpu().double()

    def oracle_block(b, feats):
        tp = b.tp
        return orc.interaction_block(
            str(tp.irreps_in1), str(tp.irreps_in2), str(tp.irreps_out), _ins(tp), str(b.irreps_out), p64, feats, srcc, dstc,
            shiftc, [b.fc.layer0.weight.detach().cpu().double(), b.fc.layer1.weight.detach().cpu().double()],
            b.lin.weight.detach().cpu().double(), 8, 5.0, nn_avg, [0, 1, 2], chunk=4096)

    h64 = orc.gate("16x0e", ["silu"], "32x0e", ["sigmoid"], "16x1o+16x2e", oracle_block(b1, x64))
    ref = oracle_block(b2, h64)
    (ref * G.double()).sum().backward()
    tol = 2e-5 if mode == "fp32" else 2e-4      # two blocks deep: twice the single-block budget (fp32: measured 8.4e-6, 1.4e-5)
    assert rel_err(out.detach().cpu(), ref.detach()) < tol
    assert rel_err(xg.grad.cpu(), x64.grad) < tol
    assert rel_err(p.grad.cpu(), p64.grad) < 2 * tol


# ----------------------------------------------------------------------------- device neighbour list (cell list)
@pytest.mark.parametrize("n_atoms,inside", [(2000, True), (5000, False), (40, True)])
def test_neighbor_list_matches_kdtree(n_atoms, inside):
    """Device cell list against the host k-d tree builder: identical (dst, src)-sorted index lists (bit-exact),
    the same shifts, and rowptr = cumsum(bincount(dst)).  `inside=False` puts a third of the atoms outside the box."""
    from e3nn_b200 import nn as bnn
    from e3nn_b200.nn._interaction import _radius_graph_pbc_host

    torch.manual_seed(n_atoms)
    box = max((n_atoms / 0.05) ** (1 / 3), 15.5)
    pos = torch.rand(n_atoms, 3) * box
    if not inside:
        pos[::3] += box * torch.randint(-2, 3, (pos[::3].shape[0], 3)).float()
    src_h, dst_h, shift_h = _radius_graph_pbc_host(pos, box, 5.0)
    src, dst, shift, rowptr = bnn.neighbor_list_pbc(pos.to(DEV), box, 5.0)
    assert torch.equal(src.cpu(), src_h) and torch.equal(dst.cpu(), dst_h)
    assert (shift.cpu() - shift_h).abs().max().item() < 1e-4
    ref_rowptr = torch.zeros(n_atoms + 1, dtype=torch.int64)
    ref_rowptr[1:] = torch.cumsum(torch.bincount(dst_h, minlength=n_atoms), 0)
    assert torch.equal(rowptr.cpu(), ref_rowptr)
    # every edge vector is within the cutoff and the list is symmetric
    vec = pos.to(DEV)[src] - pos.to(DEV)[dst] + shift
    assert vec.norm(dim=-1).max().item() <= 5.0 + 1e-3
    fwd = set(zip(src.cpu().tolist(), dst.cpu().tolist()))
    assert all((d, s) in fwd for s, d in list(fwd)[:2000])
    # run-to-run identical (rows are sorted after the atomics-ordered scatter)
    src2, dst2, shift2, _ = bnn.neighbor_list_pbc(pos.to(DEV), box, 5.0)
    assert torch.equal(src, src2) and torch.equal(shift, shift2)
    # the dispatching front end picks the device builder for CUDA positions
    s3, d3, _ = bnn.radius_graph_pbc(pos.to(DEV), box, 5.0)
    assert torch.equal(s3, src) and torch.equal(d3, dst)


def test_neighbor_list_row_ranges_concatenate_to_the_full_list():
    """A rank's shard (destination rows [n0, n1)) is bit-identical to the matching slice of the full list; an empty
    range and the whole range are valid."""
    from e3nn_b200 import nn as bnn

    torch.manual_seed(5)
    n_atoms, box = 3000, (3000 / 0.05) ** (1 / 3)
    pos = (torch.rand(n_atoms, 3) * box).to(DEV)
    src, dst, shift, rowptr = bnn.neighbor_list_pbc(pos, box, 5.0)
    bounds = [0, 0, 700, 701, 2222, n_atoms]
    parts = [bnn.neighbor_list_pbc(pos, box, 5.0, rows=(a, b)) for a, b in zip(bounds, bounds[1:])]
    assert torch.equal(torch.cat([p[0] for p in parts]), src)
    assert torch.equal(torch.cat([p[1] for p in parts]), dst)
    assert torch.equal(torch.cat([p[2] for p in parts]), shift)
    for (a, b), (s_, d_, sh_, rp_) in zip(zip(bounds, bounds[1:]), parts):
        assert rp_.numel() == b - a + 1 and torch.equal(rp_, rowptr[a:b + 1] - rowptr[a])
        assert d_.numel() == 0 or (int(d_.min()) >= a and int(d_.max()) < b)
    with pytest.raises(IndexError):
        bnn.neighbor_list_pbc(pos, box, 5.0, rows=(10, n_atoms + 1))


def test_neighbor_list_edge_cases():
    from e3nn_b200 import nn as bnn

    empty = bnn.neighbor_list_pbc(torch.zeros(0, 3, device=DEV), 20.0, 5.0)
    assert empty[0].numel() == 0 and empty[3].tolist() == [0]
    lone = bnn.neighbor_list_pbc(torch.tensor([[1.0, 2.0, 3.0]], device=DEV), 20.0, 5.0)
    assert lone[0].numel() == 0 and lone[3].tolist() == [0, 0]
    with pytest.raises(NotImplementedError):
        bnn.neighbor_list_pbc(torch.rand(10, 3, device=DEV), 12.0, 5.0)      # box < 3 x cutoff
    # two atoms across the periodic boundary see each other through the image
    pair = torch.tensor([[0.5, 10.0, 10.0], [19.5, 10.0, 10.0]], device=DEV)
    src, dst, shift, rowptr = bnn.neighbor_list_pbc(pair, 20.0, 5.0)
    assert src.tolist() == [1, 0] and dst.tolist() == [0, 1] and rowptr.tolist() == [0, 1, 2]
    vec = pair[src] - pair[dst] + shift
    assert torch.allclose(vec, torch.tensor([[-1.0, 0.0, 0.0], [1.0, 0.0, 0.0]], device=DEV))


# ----------------------------------------------------------------------------- Gate
@pytest.mark.parametrize("name", ["gate_mixed", "gate_l3", "gate_abs_identity", "gate_no_scalars"])
def test_gate_golden_and_gradient(golden, golden_meta, name):
    """Gate kernel against the reference's output on the golden rows, and its gradient against autograd through
    the oracle (fp64) on larger seeded rows with leading batch dimensions."""
    from e3nn_b200 import nn as bnn

    fn = {"silu": torch.nn.functional.silu, "tanh": torch.tanh, "sigmoid": torch.sigmoid, "abs": torch.abs,
          "relu": torch.relu, None: None}
    g, m = golden(name), golden_meta["cases"][name]
    gate = bnn.Gate(m["irreps_scalars"], [fn[a] for a in m["act_scalars"]], m["irreps_gates"],
                    [fn[a] for a in m["act_gates"]], m["irreps_gated"]).to(DEV)
    out = gate(torch.from_numpy(g["x"]).to(DEV))
    assert rel_err(out.cpu(), torch.from_numpy(g["out_f64"])) < TOL
    torch.manual_seed(3)
    x = torch.randn(5, 301, gate.irreps_in.dim)
    go = torch.randn(5, 301, gate.irreps_out.dim)
    x64 = x.double().requires_grad_(True)
    ref = orc.gate(m["irreps_scalars"], m["act_scalars"], m["irreps_gates"], m["act_gates"], m["irreps_gated"], x64)
    ref.backward(go.double())
    xg = x.clone().to(DEV).requires_grad_(True)
    o = gate(xg)
    assert o.shape == ref.shape and rel_err(o.detach().cpu(), ref.detach()) < TOL
    o.backward(go.to(DEV))
    assert rel_err(xg.grad.cpu(), x64.grad) < TOL
    assert gate(torch.zeros(0, gate.irreps_in.dim, device=DEV)).shape == (0, gate.irreps_out.dim)


@pytest.mark.parametrize("name", ["activation_mixed", "activation_abs", "activation_identity", "activation_relu_sigmoid"])
def test_activation_golden_and_gradient(golden, golden_meta, name):
    """Activation module against the reference's output on the golden rows (its irreps_out too), and its gradient
    against autograd through the fp64 oracle."""
    from e3nn_b200 import nn as bnn

    fn = {"silu": torch.nn.functional.silu, "tanh": torch.tanh, "sigmoid": torch.sigmoid, "abs": torch.abs,
          "relu": torch.relu, None: None}
    g, m = golden(name), golden_meta["cases"][name]
    act = bnn.Activation(m["irreps_in"], [fn[a] for a in m["acts"]]).to(DEV)
    assert str(act.irreps_out) == m["irreps_out"]
    out = act(torch.from_numpy(g["x"]).to(DEV))
    assert rel_err(out.cpu(), torch.from_numpy(g["out_f64"])) < TOL
    torch.manual_seed(8)
    x = torch.randn(3, 257, act.irreps_in.dim)
    go = torch.randn(3, 257, act.irreps_out.dim)
    x64 = x.double().requires_grad_(True)
    ref = orc.activation(m["irreps_in"], m["acts"], x64)
    ref.backward(go.double())
    xg = x.clone().to(DEV).requires_grad_(True)
    o = act(xg)
    o.backward(go.to(DEV))
    assert rel_err(o.detach().cpu(), ref.detach()) < TOL and rel_err(xg.grad.cpu(), x64.grad) < TOL
    assert act(torch.zeros(0, act.irreps_in.dim, device=DEV)).shape == (0, act.irreps_out.dim)


def test_linear_gate_fused_tensor_cores():
    """The same pair with the Linear on the tensor cores (hi/lo-split tf32 operands): Gate as the epilogue of the
    tcgen05 kernel, against the fp64 oracle (1e-4, the bound of that Linear mode) and the two-module path."""
    from e3nn_b200 import nn as bnn

    gate = bnn.Gate("64x0e", [torch.nn.functional.silu], "192x0e", [torch.sigmoid], "64x1o+64x2e+64x3o").to(DEV)
    lin = o3.Linear("64x0e+64x1o+64x2e+64x3o", gate.irreps_in, math_mode="tf32x3").to(DEV)
    fused = bnn.LinearGate(lin, gate, fuse=True).to(DEV)
    assert lin._tc_fwd is not None
    torch.manual_seed(23)
    x = torch.randn(777, lin.irreps_in.dim)
    with torch.no_grad():
        assert fused.fusable(x.to(DEV))
        out = fused(x.to(DEV))
        two = gate(lin(x.to(DEV)))
    e3nn_b200.check_status()
    y = orc.linear(str(lin.irreps_in), str(gate.irreps_in), x.double(), lin.weight.detach().cpu().double())
    ref = orc.gate("64x0e", ["silu"], "192x0e", ["sigmoid"], "64x1o+64x2e+64x3o", y)
    assert out.shape == ref.shape and rel_err(out.cpu(), ref) < TOL_TF32X3
    assert rel_err(out.cpu(), two.cpu().double()) < 2e-6


@pytest.mark.parametrize("name", ["gate_mixed", "gate_l3", "gate_abs_identity"])
def test_linear_gate_fused(golden_meta, name):
    """Gate as the epilogue of the Linear that feeds it: equal to ``gate(linear(x))`` of the fp64 oracle within the fp32
    bound, and to the two modules run one after the other; with a gradient required the two-module path runs."""
    from e3nn_b200 import nn as bnn

    fn = {"silu": torch.nn.functional.silu, "tanh": torch.tanh, "sigmoid": torch.sigmoid, "abs": torch.abs,
          "relu": torch.relu, None: None}
    m = golden_meta["cases"][name]
    gate = bnn.Gate(m["irreps_scalars"], [fn[a] for a in m["act_scalars"]], m["irreps_gates"],
                    [fn[a] for a in m["act_gates"]], m["irreps_gated"]).to(DEV)
    irreps_x = "24x0e+8x0o+16x1o+8x1e+8x2e+4x2o+8x3o"
    lin = o3.Linear(irreps_x, gate.irreps_in).to(DEV)
    fused = bnn.LinearGate(lin, gate, fuse=True).to(DEV)
    torch.manual_seed(17)
    x = torch.randn(3, 211, lin.irreps_in.dim)
    with torch.no_grad():
        assert fused.fusable(x.to(DEV))
        out = fused(x.to(DEV))
        two = gate(lin(x.to(DEV)))
    e3nn_b200.check_status()
    y = orc.linear(irreps_x, str(gate.irreps_in), x.double().reshape(-1, x.shape[-1]), lin.weight.detach().cpu().double())
    ref = orc.gate(m["irreps_scalars"], m["act_scalars"], m["irreps_gates"], m["act_gates"], m["irreps_gated"], y)
    ref = ref.reshape(*x.shape[:-1], -1)
    assert out.shape == ref.shape and rel_err(out.cpu(), ref) < TOL
    assert rel_err(out.cpu(), two.cpu().double()) < 2e-6
    # training: gradients through the pair of modules
    xg = x.clone().to(DEV).requires_grad_(True)
    assert not fused.fusable(xg)
    o = fused(xg)
    o.sum().backward()
    assert xg.grad is not None and lin.weight.grad is not None


# ----------------------------------------------------------------------------- fused edge embedding
@pytest.mark.gpu
@pytest.mark.parametrize("act,hidden,nb,with_shift", [("silu", 64, 8, True), ("tanh", 32, 5, False), ("relu", 128, 16, True)])
def test_edge_embed_matches_fp64_chain(act, hidden, nb, with_shift):
    """edge_vec, Bessel basis and first radial layer in one kernel, and their pull-back to the positions,
    against the same chain written with torch operators in fp64 (e3nn/math/_bessel.py:6-37, e3nn/nn/_fc.py:38-48)."""
    from e3nn_b200 import nn as bnn

    torch.manual_seed(5)
    N, E, c = 300, 4001, 5.0          # E is not a multiple of the 32-edge batches
    pos = torch.rand(N, 3) * 6.0
    src = torch.randint(0, N, (E,))
    dst = torch.randint(0, N, (E,))
    src[7] = dst[7]                   # a zero-length edge (r = 0 branch of the basis)
    shift = torch.randn(E, 3) * 0.3 if with_shift else None
    if shift is not None:
        shift[7] = 0.0
    w0 = torch.randn(nb, hidden)
    w_scale, act_scale = nb ** -0.5, bnn.normalize2mom_constant(act)
    gh, gv = torch.randn(E, hidden), torch.randn(E, 3)

    f = {"silu": torch.nn.functional.silu, "tanh": torch.tanh, "relu": torch.relu}[act]
    p64 = pos.double().requires_grad_(True)
    vec64 = p64[src] - p64[dst] + (shift.double() if shift is not None else 0.0)
    r = vec64.pow(2).sum(-1).clamp_min(1e-300).sqrt() * (vec64.pow(2).sum(-1) > 0)
    h64 = act_scale * f(bnn.bessel(r, nb, c) @ (w0.double() * w_scale))
    ((h64 * gh.double()).sum() + (vec64 * gv.double()).sum()).backward()

    p = pos.clone().to(DEV).requires_grad_(True)
    vec, h = bnn.edge_embed(p, src.to(DEV), dst.to(DEV), shift.to(DEV) if shift is not None else None, w0.to(DEV), c,
                            w_scale, act_scale, act, check_indices=True)
    ((h * gh.to(DEV)).sum() + (vec * gv.to(DEV)).sum()).backward()
    assert rel_err(vec.detach().cpu(), vec64.detach()) < 1e-6
    assert rel_err(h.detach().cpu(), h64.detach()) < TOL
    assert rel_err(p.grad.cpu(), p64.grad) < TOL
    bad = src.clone()
    bad[11] = N
    with pytest.raises(IndexError):
        bnn.edge_embed(pos.to(DEV), bad.to(DEV), dst.to(DEV), None, w0.to(DEV), c, w_scale, act_scale, act, check_indices=True)
    # empty edge list
    v0, h0 = bnn.edge_embed(pos.to(DEV), src[:0].to(DEV), dst[:0].to(DEV), None, w0.to(DEV), c, w_scale, act_scale, act)
    assert v0.shape == (0, 3) and h0.shape == (0, hidden)


@pytest.mark.parametrize("basis,cutoff,envelope", [("gaussian", True, None), ("gaussian", False, "smooth_cutoff"),
                                                   ("cosine", True, None), ("smooth_finite", True, "smooth_cutoff"),
                                                   ("smooth_finite", False, None), ("fourier", True, None),
                                                   ("fourier", False, None), ("soft_bessel", True, "smooth_cutoff"),
                                                   ("soft_bessel", False, None)])
def test_edge_embed_basis_families(basis, cutoff, envelope):
    """The soft_one_hot_linspace families and the smooth_cutoff envelope in the fused edge embedding against the
    oracle's restatement of e3nn/math/_soft_one_hot_linspace.py:100-140 / gate_points_2101.py:136-141 in fp64,
    values and position gradient (radii span both sides of the cutoff)."""
    from e3nn_b200 import nn as bnn

    torch.manual_seed(17)
    N, E, nb, hidden, start, end = 200, 3000, 8, 64, 0.5, 5.0
    pos = torch.rand(N, 3) * 5.5
    src, dst = torch.randint(0, N, (E,)), torch.randint(0, N, (E,))
    dst = torch.where(dst == src, (dst + 1) % N, dst)          # no zero-length edges: soft bessel is 0/0 there
    w0 = torch.randn(nb, hidden)
    w_scale, act_scale, bscale = nb ** -0.5, bnn.normalize2mom_constant("silu"), nb ** 0.5
    gh, gv = torch.randn(E, hidden), torch.randn(E, 3)
    p64 = pos.double().requires_grad_(True)
    vec64 = p64[src] - p64[dst]
    r = vec64.norm(dim=-1)
    B = bscale * orc.soft_one_hot_linspace(r, start, end, nb, "bessel" if basis == "soft_bessel" else basis, cutoff)
    h64 = act_scale * torch.nn.functional.silu(B @ (w0.double() * w_scale))
    if envelope is not None:
        h64 = h64 * orc.smooth_cutoff(r / end)[:, None]
    ((h64 * gh.double()).sum() + (vec64 * gv.double()).sum()).backward()
    p = pos.clone().to(DEV).requires_grad_(True)
    vec, h = bnn.edge_embed(p, src.to(DEV), dst.to(DEV), None, w0.to(DEV), end, w_scale, act_scale, "silu", basis=basis,
                            cutoff=cutoff, start=start, basis_scale=bscale, envelope=envelope)
    ((h * gh.to(DEV)).sum() + (vec * gv.to(DEV)).sum()).backward()
    assert rel_err(h.detach().cpu(), h64.detach()) < TOL
    assert rel_err(p.grad.cpu(), p64.grad) < TOL      # measured 2.3e-6 over the nine basis / cutoff combinations


# ----------------------------------------------------------------------------- tensor-core contractions with split operands
TOL_TF32X3 = 1e-4   # hi/lo-split tf32 operands: measured 1e-5 .. 4e-5 x RMS on these layouts


@pytest.mark.parametrize("Z", [1, 77, 4097])
def test_uvw_tensor_core_split_operands(Z):
    torch.manual_seed(Z)
    tp = o3.FullyConnectedTensorProduct("128x0e+64x1o+32x2e", "0e+1o+2e+3o", "128x0e+64x1o+32x2e", math_mode="tf32x3").to(DEV)
    x, y = torch.randn(Z, 480), torch.randn(Z, 16)
    with torch.no_grad():
        out = tp(x.to(DEV), y.to(DEV))
    assert tp._tcg_spec is not None
    e3nn_b200.check_status()
    ref = _oracle_tp(tp, x.double(), y.double(), tp.weight.detach().cpu().double())
    assert rel_err(out.cpu(), ref) < TOL_TF32X3
    tp32 = o3.FullyConnectedTensorProduct("128x0e+64x1o+32x2e", "0e+1o+2e+3o", "128x0e+64x1o+32x2e").to(DEV)
    with torch.no_grad():
        tp32.weight.copy_(tp.weight)
        assert rel_err(tp32(x.to(DEV), y.to(DEV)).cpu(), ref) < TOL   # strict fp32 mode: CUDA-core kernel


@pytest.mark.parametrize("irreps,Z", [
    (("64x0e+32x1o+32x2e", "32x0e+64x1o+32x2e"), 1000),
    (("128x0e+64x1o+32x2e", "128x0e+64x1o+32x2e"), 1000),
    # input blocks 128 and 256 channels wide with 2l+1 = 3 and 5: the transposed contraction runs with swapped operands
    (("128x0e+128x1o+256x2e+128x3o", "64x0e+64x1o+32x2e+32x3o"), 1000),
    (("128x0e+128x1o+256x2e+128x3o", "64x0e+64x1o+32x2e+32x3o"), 43),
    (("128x0e+128x1o+256x2e+128x3o", "64x0e+64x1o+32x2e+32x3o"), 1),
])
def test_linear_math_modes_forward_and_transpose(irreps, Z):
    torch.manual_seed(5)
    x = torch.randn(Z, o3.Irreps(irreps[0]).dim)
    ref_lin = o3.Linear(*irreps).to(DEV)
    ref_lin.weight.requires_grad_(False)
    x64 = x.double().requires_grad_(True)
    ref = orc.linear(irreps[0], irreps[1], x64, ref_lin.weight.detach().cpu().double())
    go = torch.randn_like(ref)
    ref.backward(go)
    for mode, lo, hi in (("fp32", 0.0, TOL), ("tf32x3", 0.0, TOL_TF32X3), ("tf32", 1e-5, TOL_TF32)):
        lin = o3.Linear(*irreps, math_mode=mode).to(DEV)
        assert lin._tc_fwd is not None and lin._tc_bwd is not None
        with torch.no_grad():
            lin.weight.copy_(ref_lin.weight)
        lin.weight.requires_grad_(False)
        xg = x.clone().to(DEV).requires_grad_(True)
        out = lin(xg)
        out.backward(go.float().to(DEV))
        e_fwd, e_bwd = rel_err(out.detach().cpu(), ref.detach()), rel_err(xg.grad.cpu(), x64.grad)
        assert lo <= e_fwd < hi and e_bwd < hi, (mode, e_fwd, e_bwd)


# ----------------------------------------------------------------------------- gradients of the weight-shared paths
@pytest.mark.parametrize("layout,mode,tol", [
    (("8x0e+8x1o+4x2e", "1x0e+1x1o+1x2e", "8x0e+6x1o+4x2e+2x1e"), "fp32", TOL),
    (("5x0e+3x1o+2x2e+1x3o", "2x0e+3x1o+1x2e", "4x0e+2x0o+3x1o+2x1e+1x2e"), "fp32", TOL),   # multiplicities > 1 on both sides
    (("32x0e+32x1o+32x2e", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e"), "fp32", TOL),              # benchmark case 1 (10,000-row fully connected product)
    (("32x0e+32x1o+32x2e", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e"), "tf32x3", 1e-4),
    (("128x0e+64x1o+32x2e", "0e+1o+2e+3o", "128x0e+64x1o+32x2e"), "tf32", TOL_TF32),         # benchmark case 4 (1,048,576-row fully connected product)
])
def test_uvw_gradients(layout, mode, tol):
    """Cotangents of a fully connected product w.r.t. both operands and the shared weights against autograd
    through the fp64 oracle (the reference obtains them from autograd through its einsums)."""
    torch.manual_seed(11)
    tp = o3.FullyConnectedTensorProduct(*layout, math_mode=mode).to(DEV)
    with torch.no_grad():
        for view in tp.weight_views():
            view.div_((view.shape[0] * view.shape[1]) ** 0.5)
    Z = 777
    x, y = torch.randn(Z, tp.irreps_in1.dim), torch.randn(Z, tp.irreps_in2.dim)
    go = torch.randn(Z, tp.irreps_out.dim)
    xg, yg = x.to(DEV).requires_grad_(True), y.to(DEV).requires_grad_(True)
    out = tp(xg, yg)
    out.backward(go.to(DEV))
    x64, y64 = x.double().requires_grad_(True), y.double().requires_grad_(True)
    w64 = tp.weight.detach().cpu().double().requires_grad_(True)
    ref = _oracle_tp(tp, x64, y64, w64)
    ref.backward(go.double())
    assert rel_err(out.detach().cpu(), ref.detach()) < tol
    assert rel_err(xg.grad.cpu(), x64.grad) < tol
    assert rel_err(yg.grad.cpu(), y64.grad) < tol
    assert rel_err(tp.weight.grad.cpu(), w64.grad) < max(tol, TOL)
    # external weights, only the weights require a gradient
    tp2 = o3.FullyConnectedTensorProduct(*layout, internal_weights=False, math_mode=mode).to(DEV)
    wg = tp.weight.detach().clone().requires_grad_(True)
    tp2(x.to(DEV), y.to(DEV), wg).backward(go.to(DEV))
    assert rel_err(wg.grad.cpu(), w64.grad) < max(tol, TOL)


def test_uvw_weight_gradient_many_rows():
    """The weight gradient sums over the rows: 200,000 rows through several row tiles per block."""
    torch.manual_seed(12)
    tp = o3.FullyConnectedTensorProduct("16x0e+8x1o", "1x0e+1x1o", "8x0e+8x1o").to(DEV)
    Z = 200_000
    x, y, go = torch.randn(Z, tp.irreps_in1.dim), torch.randn(Z, tp.irreps_in2.dim), torch.randn(Z, tp.irreps_out.dim)
    tp(x.to(DEV), y.to(DEV)).backward(go.to(DEV))
    w64 = tp.weight.detach().cpu().double().requires_grad_(True)
    _oracle_tp(tp, x.double(), y.double(), w64).backward(go.double())
    assert rel_err(tp.weight.grad.cpu(), w64.grad) < TOL


def test_mixed_uvu_uvw_gradients():
    """A product with both kinds of paths: the two autograd nodes share the output rows."""
    torch.manual_seed(13)
    ir1, ir2, iro = o3.Irreps("4x0e+4x1o"), o3.Irreps("1x0e+1x1o"), o3.Irreps("4x0e+4x1o+3x1o")
    instr = [(0, 0, 0, "uvu", True), (1, 1, 0, "uvu", True), (1, 0, 1, "uvu", True), (0, 1, 2, "uvw", True),
             (1, 0, 2, "uvw", True), (1, 1, 0, "uvw", True)]
    tp = o3.TensorProduct(ir1, ir2, iro, instr).to(DEV)
    Z = 100
    x, y, go = torch.randn(Z, ir1.dim), torch.randn(Z, ir2.dim), torch.randn(Z, iro.dim)
    xg, yg = x.to(DEV).requires_grad_(True), y.to(DEV).requires_grad_(True)
    out = tp(xg, yg)
    out.backward(go.to(DEV))
    x64, y64 = x.double().requires_grad_(True), y.double().requires_grad_(True)
    w64 = tp.weight.detach().cpu().double().requires_grad_(True)
    ref = _oracle_tp(tp, x64, y64, w64)
    ref.backward(go.double())
    assert rel_err(out.detach().cpu(), ref.detach()) < TOL
    assert rel_err(xg.grad.cpu(), x64.grad) < TOL
    assert rel_err(yg.grad.cpu(), y64.grad) < TOL
    assert rel_err(tp.weight.grad.cpu(), w64.grad) < TOL


@pytest.mark.parametrize("mode,tol", [("fp32", TOL), ("tf32x3", 1e-4)])
def test_linear_weight_and_bias_gradients(mode, tol):
    torch.manual_seed(14)
    lin = o3.Linear("64x0e+64x1o+32x2e+3x3o", "64x0e+32x1o+32x2e+5x0e", biases=[True, False, False, True], math_mode=mode).to(DEV)
    with torch.no_grad():
        lin.bias.normal_()
    Z = 5000
    x = torch.randn(Z, lin.irreps_in.dim)
    go = torch.randn(Z, lin.irreps_out.dim)
    xg = x.to(DEV).requires_grad_(True)
    out = lin(xg)
    out.backward(go.to(DEV))
    x64 = x.double().requires_grad_(True)
    w64 = lin.weight.detach().cpu().double().requires_grad_(True)
    b64 = lin.bias.detach().cpu().double().requires_grad_(True)
    ref = orc.linear(str(lin.irreps_in), str(lin.irreps_out), x64, w64, b64, biases=[True, False, False, True])
    ref.backward(go.double())
    assert rel_err(out.detach().cpu(), ref.detach()) < tol
    assert rel_err(xg.grad.cpu(), x64.grad) < tol
    assert rel_err(lin.weight.grad.cpu(), w64.grad) < TOL
    assert rel_err(lin.bias.grad.cpu(), b64.grad) < TOL


@pytest.mark.parametrize("name", ["tp_elementwise", "tp_uuu_mixed_shared", "tp_uuu_unshared", "tp_full", "tp_rest_shared", "tp_rest_unshared",
                                  "tp_uvuv_mixed_unshared", "tp_mixed_unshared"])
def test_uuu_gradients(golden, golden_meta, name):
    """'uuu' and 'uvuv' paths (alone, and mixed with 'uvu' / 'uvw'): all cotangents against autograd through the fp64
    oracle."""
    g, m = golden(name), golden_meta["cases"][name]
    tp = _tp_from_meta(name, m)
    x1, x2, w = (torch.from_numpy(g[k]) for k in ("x1", "x2", "w"))
    torch.manual_seed(3)
    go = torch.randn(x1.shape[0], tp.irreps_out.dim)
    d = [t.to(DEV).requires_grad_(True) for t in (x1, x2, w)]
    out = tp(d[0], d[1], d[2] if w.numel() > 0 else None)
    out.backward(go.to(DEV))
    r = [t.double().requires_grad_(True) for t in (x1, x2, w)]
    ref = _oracle_tp(tp, *r)
    ref.backward(go.double())
    assert rel_err(out.detach().cpu(), ref.detach()) < TOL
    assert rel_err(d[0].grad.cpu(), r[0].grad) < TOL
    assert rel_err(d[1].grad.cpu(), r[1].grad) < TOL
    if w.numel() > 0:
        assert rel_err(d[2].grad.cpu(), r[2].grad) < TOL


def test_elementwise_tensor_product_module():
    """`ElementwiseTensorProduct` end to end (layout splitting + kernels) against the reference's output."""
    etp = o3.ElementwiseTensorProduct("4x0e+3x1o+2x2e+5x1e", "4x0e+3x1o+2x1o+5x2e")
    torch.manual_seed(4)
    x1, x2 = torch.randn(50, etp.irreps_in1.dim), torch.randn(50, etp.irreps_in2.dim)
    out = etp(x1.to(DEV), x2.to(DEV))
    ref = _oracle_tp(etp, x1.double(), x2.double(), torch.zeros(0, dtype=torch.float64))
    assert rel_err(out.cpu(), ref) < TOL
    assert etp.weight_numel == 0
    # filter: the scalar products only
    dot = o3.ElementwiseTensorProduct("5x1o+5x1e", "10x1e", ["0e", "0o"])
    assert str(dot.irreps_out) == "5x0o+5x0e"
    a, b = torch.randn(9, 30), torch.randn(9, 30)
    o = dot(a.to(DEV), b.to(DEV)).cpu()
    assert rel_err(o, _oracle_tp(dot, a.double(), b.double(), torch.zeros(0, dtype=torch.float64))) < TOL
    # component normalisation of a scalar output: w3j = delta / sqrt(3), coefficient 1 -> dot product / sqrt(3)
    assert rel_err(o, ((a.view(9, 10, 3) * b.view(9, 10, 3)).sum(-1) / 3 ** 0.5).double()) < TOL


@pytest.mark.parametrize("modes", [("fp32", "fp32"), ("tf32x3", "tf32x3")])
def test_interaction_block_training_gradients(modes):
    """One training step of the block: gradients w.r.t. every parameter (radial layers, Linear) and the node
    features against autograd through the fp64 oracle."""
    from e3nn_b200 import nn as bnn

    torch.manual_seed(21)
    n_atoms, irreps, lmax = 400, "16x0e+16x1o+16x2e", 2
    box = (n_atoms / 0.05) ** (1 / 3)
    pos = torch.rand(n_atoms, 3) * box
    src, dst, shift = bnn.radius_graph_pbc(pos, box, 5.0)
    nn_avg = src.numel() / n_atoms
    block = bnn.InteractionBlock(irreps, lmax, num_basis=8, hidden=64, r_max=5.0, num_neighbors=nn_avg,
                                 linear_math_mode=modes[0], radial_math_mode=modes[1]).to(DEV)
    node_x = torch.randn(n_atoms, block.irreps_node.dim)
    G = torch.randn(n_atoms, block.irreps_out.dim)
    _, rowptr = e3nn_b200.csr_from_dst(dst.to(DEV), n_atoms)
    xg = node_x.to(DEV).requires_grad_(True)
    out = block(pos.to(DEV), xg, src.to(DEV), dst.to(DEV), rowptr, shift.to(DEV))
    (out * G.to(DEV)).sum().backward()

    tp = block.tp
    w0, w1, wl = (t.detach().cpu().double().requires_grad_(True)
                  for t in (block.fc.layer0.weight, block.fc.layer1.weight, block.lin.weight))
    x64 = node_x.double().requires_grad_(True)
    ref = orc.interaction_block(
        str(tp.irreps_in1), str(tp.irreps_in2), str(tp.irreps_out), _ins(tp), str(block.irreps_out), pos.double(),
        x64, src, dst, shift.double(), [w0, w1], wl, 8, 5.0, nn_avg, list(range(lmax + 1)), chunk=4096)
    (ref * G.double()).sum().backward()
    tol = 5e-5 if modes[0] == "fp32" else 2e-4
    assert rel_err(out.detach().cpu(), ref.detach()) < tol
    assert rel_err(xg.grad.cpu(), x64.grad) < tol
    assert rel_err(block.lin.weight.grad.cpu(), wl.grad) < tol
    assert rel_err(block.fc.layer1.weight.grad.cpu(), w1.grad) < tol
    assert rel_err(block.fc.layer0.weight.grad.cpu(), w0.grad) < tol


def test_uvuv_weighted_gradients():
    """Weighted 'uvuv' paths next to 'uvu' and 'uvw' ones, shared weights: all cotangents vs the fp64 oracle."""
    torch.manual_seed(31)
    tp = o3.TensorProduct("2x0e+3x1o", "2x1o+4x0e", "6x0e+6x1e+3x1o+8x0e",
                          [(1, 0, 0, "uvuv", True), (1, 0, 1, "uvuv", False), (1, 1, 2, "uvu", True), (0, 1, 3, "uvuv", True, 2.0),
                           (1, 0, 3, "uvw", True)]).to(DEV)
    Z = 40
    x, y, go = torch.randn(Z, tp.irreps_in1.dim), torch.randn(Z, tp.irreps_in2.dim), torch.randn(Z, tp.irreps_out.dim)
    xg, yg = x.to(DEV).requires_grad_(True), y.to(DEV).requires_grad_(True)
    out = tp(xg, yg)
    out.backward(go.to(DEV))
    x64, y64 = x.double().requires_grad_(True), y.double().requires_grad_(True)
    w64 = tp.weight.detach().cpu().double().requires_grad_(True)
    ref = _oracle_tp(tp, x64, y64, w64)
    ref.backward(go.double())
    assert rel_err(out.detach().cpu(), ref.detach()) < TOL
    assert rel_err(xg.grad.cpu(), x64.grad) < TOL
    assert rel_err(yg.grad.cpu(), y64.grad) < TOL
    assert rel_err(tp.weight.grad.cpu(), w64.grad) < TOL


@pytest.mark.parametrize("name", ["square_full", "square_connected"])
def test_tensor_square(golden, golden_meta, name):
    """`TensorSquare` (unweighted and weighted forms) against the reference's outputs; gradients vs the fp64 oracle."""
    g, m = golden(name), golden_meta["cases"][name]
    sq = o3.TensorSquare(*m["args"], internal_weights=False) if len(m["args"]) > 1 else o3.TensorSquare(*m["args"])
    x, w = torch.from_numpy(g["x"]), torch.from_numpy(g["w"])
    xg, wg = x.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True)
    out = sq(xg, wg if w.numel() > 0 else None)
    assert rel_err(out.detach().cpu(), torch.from_numpy(g["out_f64"])) < TOL
    torch.manual_seed(5)
    go = torch.randn(x.shape[0], sq.irreps_out.dim)
    out.backward(go.to(DEV))
    x64, w64 = x.double().requires_grad_(True), w.double().requires_grad_(True)
    ref = _oracle_tp(sq, x64, x64, w64)
    ref.backward(go.double())
    assert rel_err(xg.grad.cpu(), x64.grad) < TOL
    if w.numel() > 0:
        assert rel_err(wg.grad.cpu(), w64.grad) < TOL


def test_norm_module():
    """`o3.Norm` (e3nn/o3/_norm.py): per-channel Euclidean norms, the reference's doctest shape, squared form."""
    torch.manual_seed(8)
    norm = o3.Norm("17x1o")
    assert norm(torch.randn(17 * 3, device=DEV)).shape == (17,)
    irreps = o3.Irreps("5x0e+4x1o+3x2e+2x3o")
    x = torch.randn(200, irreps.dim)
    want, off = [], 0
    for mul, ir in irreps:
        want.append(x[:, off : off + mul * ir.dim].double().view(200, mul, ir.dim).norm(dim=-1))
        off += mul * ir.dim
    want = torch.cat(want, dim=1)
    got = o3.Norm(irreps)(x.to(DEV)).cpu()
    assert str(o3.Norm(irreps).irreps_out) == "14x0e"
    assert rel_err(got, want) < TOL
    assert rel_err(o3.Norm(irreps, squared=True)(x.to(DEV)).cpu(), want ** 2) < TOL
    xg = x.to(DEV).requires_grad_(True)
    o3.Norm(irreps)(xg).sum().backward()
    x64 = x.double().requires_grad_(True)
    off, total = 0, 0.0
    for mul, ir in irreps:
        total = total + x64[:, off : off + mul * ir.dim].view(200, mul, ir.dim).norm(dim=-1).sum()
        off += mul * ir.dim
    total.backward()
    assert rel_err(xg.grad.cpu(), x64.grad) < TOL


# ----------------------------------------------------------------------------- product + Linear as one product
@pytest.mark.parametrize("layout,mode,tol", [
    (("32x0e+32x1o+32x2e", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e"), "fp32", TOL),
    (("8x0e+8x1o+4x2e", "1x0e+1x1o+1x2e", "8x0e+6x1o+4x2e+2x1e"), "fp32", TOL),
    (("128x0e+64x1o+32x2e", "0e+1o+2e+3o", "128x0e+64x1o+32x2e"), "tf32", TOL_TF32),      # benchmark case 4 (1,048,576-row fully connected product)
])
def test_tensor_product_linear_fused(layout, mode, tol):
    """``TensorProductLinear(tp, lin)(x, y)`` against ``lin(tp(x, y))`` evaluated by the fp64 oracle, forward and the
    gradients w.r.t. both operands and both modules' weights."""
    torch.manual_seed(21)
    tp = o3.FullyConnectedTensorProduct(*layout, math_mode=mode).to(DEV)
    with torch.no_grad():
        for view in tp.weight_views():
            view.div_((view.shape[0] * view.shape[1]) ** 0.5)
    lin = o3.Linear(tp.irreps_out, tp.irreps_out).to(DEV)
    fused = o3.TensorProductLinear(tp, lin)
    Z = 515
    x, y = torch.randn(Z, tp.irreps_in1.dim), torch.randn(Z, tp.irreps_in2.dim)
    go = torch.randn(Z, lin.irreps_out.dim)
    xg, yg = x.to(DEV).requires_grad_(True), y.to(DEV).requires_grad_(True)
    out = fused(xg, yg)
    out.backward(go.to(DEV))
    e3nn_b200.check_status()
    x64, y64 = x.double().requires_grad_(True), y.double().requires_grad_(True)
    w64 = tp.weight.detach().cpu().double().requires_grad_(True)
    l64 = lin.weight.detach().cpu().double().requires_grad_(True)
    ref = orc.linear(str(tp.irreps_out), str(lin.irreps_out), _oracle_tp(tp, x64, y64, w64), l64)
    ref.backward(go.double())
    assert rel_err(out.detach().cpu(), ref.detach()) < tol
    assert rel_err(xg.grad.cpu(), x64.grad) < tol
    assert rel_err(yg.grad.cpu(), y64.grad) < tol
    wtol = tol                # weight gradients: float atomics over all rows, measured 3.6e-6 in the fp32 case
    assert rel_err(tp.weight.grad.cpu(), w64.grad) < wtol
    assert rel_err(lin.weight.grad.cpu(), l64.grad) < wtol
    # the two modules side by side give the same result
    with torch.no_grad():
        two_step = lin(tp(x.to(DEV), y.to(DEV)))
    assert rel_err(out.detach().cpu(), two_step.cpu().double()) < max(tol, 2e-6)
