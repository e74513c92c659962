"""The CUDA path at the full sizes of the benchmark configurations.

The oracle cannot evaluate millions of edges in seconds, so these tests check properties that do not depend on
the size: rows sampled from the full-size output against the oracle evaluated on just the edges that feed them,
linearity in the features, run-to-run determinism, norms of the spherical harmonics, and translation invariance
(the position gradients of an interaction block sum to zero).
"""
import pytest
import torch

import e3nn_b200
from conftest import rel_err
from e3nn_b200 import layouts, o3
from oracle import e3nn_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-5


def _ins(tp):
    return [(i.i_in1, i.i_in2, i.i_out, i.connection_mode, i.has_weight) for i in tp.instructions]


def test_spherical_harmonics_config2_full_size():
    """4,194,304 vectors, l <= 3, 'component': sum_m Y_lm^2 = 2l+1 on every row; 2,000 sampled rows vs the oracle."""
    E = 4_194_304
    gen = torch.Generator(device=DEV).manual_seed(0)
    vec = torch.randn(E, 3, device=DEV, generator=gen)
    out = o3.spherical_harmonics("0e+1o+2e+3o", vec, True, "component")
    assert out.shape == (E, 16)
    off = 0
    for l in range(4):
        n2 = out[:, off : off + 2 * l + 1].double().pow(2).sum(1)
        assert (n2 - (2 * l + 1)).abs().max().item() < 1e-4 * (2 * l + 1)
        off += 2 * l + 1
    idx = torch.randint(0, E, (2000,), generator=torch.Generator().manual_seed(1))
    ref = orc.spherical_harmonics([0, 1, 2, 3], vec[idx.to(DEV)].cpu().double(), True, "component")
    assert rel_err(out[idx.to(DEV)].cpu(), ref) < TOL
    assert torch.equal(out, o3.spherical_harmonics("0e+1o+2e+3o", vec, True, "component"))


@pytest.mark.parametrize("layout,nodes,degree", [("cfg3_15", 65536, 32), ("cfg3_11", 65536, 32)])
def test_conv_config3_full_size(layout, nodes, degree):
    """2,097,152 edges, in-degree 32: sampled destination rows vs the oracle on their own edges, linearity in the
    node features, bitwise determinism."""
    tp = layouts.bench_conv_tp(layout)
    E = nodes * degree
    gen = torch.Generator(device=DEV).manual_seed(5)
    x1 = torch.randn(nodes, tp.irreps_in1.dim, device=DEV, generator=gen)
    x2 = torch.randn(nodes, tp.irreps_in1.dim, device=DEV, generator=gen)
    vec = torch.nn.functional.normalize(torch.randn(E, 3, device=DEV, generator=gen), dim=-1)
    src = torch.randint(0, nodes, (E,), device=DEV, generator=gen)
    rowptr = torch.arange(0, E + 1, degree, device=DEV, dtype=torch.int64)
    w = torch.randn(E, tp.weight_numel, device=DEV, generator=gen)
    scale = degree ** -0.5

    def conv(x):
        return e3nn_b200.conv_uvu(tp, x, vec, src, rowptr, w, scale=scale, edge_attr_is_vector=True)

    o1 = conv(x1)
    assert torch.equal(o1, conv(x1))                       # fixed summation order
    o2 = conv(x2)
    o12 = conv(0.5 * x1 - 2.0 * x2)
    assert rel_err(o12.cpu(), (0.5 * o1.double() - 2.0 * o2.double()).cpu()) < TOL
    # sampled destination rows, first and last included
    rows = torch.cat([torch.tensor([0, nodes - 1]), torch.randint(0, nodes, (46,), generator=torch.Generator().manual_seed(2))])
    e_idx = (rows[:, None] * degree + torch.arange(degree)[None, :]).reshape(-1)
    lmax = tp.irreps_in2.lmax
    ref = orc.conv_uvu(str(tp.irreps_in1), str(tp.irreps_in2), str(tp.irreps_out), _ins(tp), x1.cpu().double(),
                       vec[e_idx.to(DEV)].cpu().double(), src[e_idx.to(DEV)].cpu(),
                       torch.arange(rows.numel()).repeat_interleave(degree), w[e_idx.to(DEV)].cpu().double(),
                       rows.numel(), list(range(lmax + 1)), scale=scale, chunk=512)
    assert rel_err(o1[rows.to(DEV)].cpu(), ref) < TOL


@pytest.mark.parametrize("mode,tol", [("fp32", TOL), ("tf32x3", 3e-5), ("tf32", 2e-2)])     # measured 1.2e-6, 7.4e-6, 3.0e-3
def test_uvw_config4_full_size(mode, tol):
    """1,048,576 rows of the fully connected product of config 4: 256 sampled rows vs the oracle, determinism."""
    Z = 1_048_576
    tp = o3.FullyConnectedTensorProduct("128x0e+64x1o+32x2e", "0e+1o+2e+3o", "128x0e+64x1o+32x2e", math_mode=mode).to(DEV)
    torch.manual_seed(6)
    with torch.no_grad():
        tp.weight.copy_(torch.randn(tp.weight_numel))
        for view in tp.weight_views():
            view.div_((view.shape[0] * view.shape[1]) ** 0.5)
    gen = torch.Generator(device=DEV).manual_seed(7)
    x = torch.randn(Z, tp.irreps_in1.dim, device=DEV, generator=gen)
    y = torch.randn(Z, tp.irreps_in2.dim, device=DEV, generator=gen)
    with torch.no_grad():
        out = tp(x, y)
        assert torch.equal(out, tp(x, y))
    idx = torch.cat([torch.tensor([0, Z - 1]), torch.randint(0, Z, (254,), generator=torch.Generator().manual_seed(8))]).to(DEV)
    pws = [i.path_weight for i in tp.instructions]
    ref = orc.tensor_product(str(tp.irreps_in1), str(tp.irreps_in2), str(tp.irreps_out), _ins(tp), x[idx].cpu().double(),
                             y[idx].cpu().double(), tp.weight.detach().cpu().double(), True, path_weights=pws)
    assert rel_err(out[idx].cpu(), ref) < tol


def test_interaction_config5_full_size():
    """262,144 atoms, 5 A cutoff (6.86 M edges): sampled atoms' output rows vs the oracle on their own neighbourhoods,
    translation invariance of the position gradient (it sums to zero), neighbour-list symmetry."""
    from e3nn_b200 import nn as bnn

    torch.cuda.empty_cache()   # the step holds about 100 GB: hand back what earlier tests left in the allocator
    n_atoms = 262_144
    box = (n_atoms / 0.05) ** (1.0 / 3.0)
    torch.manual_seed(9)
    pos = torch.rand(n_atoms, 3) * box
    pos_d = pos.to(DEV)
    src, dst, shift, rowptr = bnn.neighbor_list_pbc(pos_d, box, 5.0)
    E = src.numel()
    assert 25.5 < E / n_atoms < 26.9
    assert int(rowptr[-1]) == E and torch.all(dst[1:] >= dst[:-1])
    # every pair appears in both directions: in-degree == out-degree for every atom
    assert torch.equal(torch.bincount(src, minlength=n_atoms), torch.bincount(dst, minlength=n_atoms))
    block = bnn.InteractionBlock("64x0e+64x1o+64x2e+64x3o", 3, num_basis=8, hidden=64, r_max=5.0, num_neighbors=E / n_atoms).to(DEV)
    for prm in block.parameters():
        prm.requires_grad_(False)
    gen = torch.Generator(device=DEV).manual_seed(10)
    node_x = torch.randn(n_atoms, 1024, device=DEV, generator=gen)
    G = torch.randn(n_atoms, block.irreps_out.dim, device=DEV, generator=gen)
    p = pos_d.clone().requires_grad_(True)
    out = block(p, node_x, src, dst, rowptr, shift)
    (out * G).sum().backward()
    g = p.grad.double()
    assert torch.isfinite(g).all()
    assert g.sum(0).abs().max().item() < 1e-4 * g.abs().sum(0).max().item()
    # the neighbourhoods of a few atoms, relabelled, through the oracle
    rows = torch.cat([torch.tensor([0, n_atoms - 1]), torch.randint(0, n_atoms, (10,), generator=torch.Generator().manual_seed(11))])
    rp = rowptr.cpu()
    e_idx = torch.cat([torch.arange(int(rp[r]), int(rp[r + 1])) for r in rows.tolist()])
    s_sub, d_sub, sh_sub = src[e_idx.to(DEV)].cpu(), dst[e_idx.to(DEV)].cpu(), shift[e_idx.to(DEV)].cpu()
    atoms, inverse = torch.unique(torch.cat([s_sub, d_sub]), return_inverse=True)
    s_loc, d_loc = inverse[: s_sub.numel()], inverse[s_sub.numel():]
    tp = block.tp
    ref = orc.interaction_block(
        str(tp.irreps_in1), str(tp.irreps_in2), str(tp.irreps_out), _ins(tp), str(block.irreps_out),
        pos[atoms].double(), node_x[atoms.to(DEV)].cpu().double(), s_loc, d_loc, sh_sub.double(),
        [block.fc.layer0.weight.detach().cpu().double(), block.fc.layer1.weight.detach().cpu().double()],
        block.lin.weight.detach().cpu().double(), 8, 5.0, E / n_atoms, [0, 1, 2, 3], chunk=512)
    local = torch.searchsorted(atoms, rows)
    assert rel_err(out.detach()[rows.to(DEV)].cpu(), ref[local]) < 3e-5     # hi/lo-split tf32 Linear and radial layer: measured 8.4e-6
