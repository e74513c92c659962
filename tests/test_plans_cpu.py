"""Host logic of the weight-shared paths, checked on the CPU: the dense plans (interpreted here in numpy exactly as
the kernels read them) and the construction of the transposed products that give the operand gradients."""
import numpy as np
import torch

from conftest import rel_err
from e3nn_b200 import o3
from e3nn_b200.o3._dense_plan import MAGIC, linear_plan
from oracle import e3nn_oracle as orc


def _i2f(v: int) -> float:
    return float(np.int32(v).view(np.float32))


def run_plan(plan: np.ndarray, x1: np.ndarray, x2, W: np.ndarray, accumulate_into=None) -> np.ndarray:
    """out[z, out_off + w * dim3 + k] (+)= sum_K A[z, k, K] * W[wbase(K) + w * wstride], A from the CG triples."""
    assert plan[0] == MAGIC
    d1, d2, dout, n_groups = (int(v) for v in plan[1:5])
    off_groups, off_kent, off_pathk, off_cg = (int(v) for v in plan[7:11])
    assert x1.shape[1] == d1 and (x2 is None or x2.shape[1] == d2)
    Z = x1.shape[0]
    out = np.zeros((Z, dout)) if accumulate_into is None else accumulate_into
    for g in range(n_groups):
        out_off, mul_out, dim3, K, kent_start, w_stride = (int(v) for v in plan[off_groups + 6 * g : off_groups + 6 * g + 6])
        block = np.zeros((Z, mul_out, dim3))
        for kk in range(K):
            path, x1off, x2off, wbase = (int(v) for v in plan[off_kent + 4 * (kent_start + kk) : off_kent + 4 * (kent_start + kk) + 4])
            wrow = W[wbase + np.arange(mul_out) * w_stride]
            for k in range(dim3):
                pk = int(plan[off_pathk + path]) + 2 * k
                cstart, ccount = int(plan[pk]), int(plan[pk + 1])
                a = np.zeros(Z)
                for c in range(cstart, cstart + ccount):
                    i, j, coef = int(plan[off_cg + 3 * c]), int(plan[off_cg + 3 * c + 1]), _i2f(plan[off_cg + 3 * c + 2])
                    a += coef * x1[:, x1off + i] * (x2[:, x2off + j] if x2off >= 0 else 1.0)
                block[:, :, k] += a[:, None] * wrow[None, :]
        out[:, out_off : out_off + mul_out * dim3] += block.reshape(Z, -1)
    return out


def _ins(tp):
    return [(i.i_in1, i.i_in2, i.i_out, i.connection_mode, i.has_weight) for i in tp.instructions]


def _oracle_tp(tp, x1, x2, w):
    return orc.tensor_product(str(tp.irreps_in1), str(tp.irreps_in2), str(tp.irreps_out), _ins(tp), x1, x2, w,
                              tp.shared_weights, path_weights=[i.path_weight for i in tp.instructions])


def test_uvw_plan_matches_oracle():
    torch.manual_seed(0)
    tp = o3.FullyConnectedTensorProduct("3x0e+2x1o+4x2e+1x1e", "2x0e+3x1o+1x2e", "5x0e+2x1o+3x2e+2x1e+1x3o")
    x1, x2 = torch.randn(9, tp.irreps_in1.dim, dtype=torch.float64), torch.randn(9, tp.irreps_in2.dim, dtype=torch.float64)
    w = tp.weight.detach().double()
    got = run_plan(tp._plan_host, x1.numpy(), x2.numpy(), w.numpy())
    # the plan stores its coefficients in fp32
    assert rel_err(torch.from_numpy(got), _oracle_tp(tp, x1, x2, w)) < 1e-6


def test_linear_plans_forward_and_transposed_with_mixed_multiplicities():
    torch.manual_seed(1)
    lin = o3.Linear("6x0e+4x1o+3x2e", "5x0e+2x0e+4x1o+3x2e+1x1o")   # two outputs of different width from one input
    x = torch.randn(7, lin.irreps_in.dim, dtype=torch.float64, requires_grad=True)
    w = lin.weight.detach().double()
    ref = orc.linear(str(lin.irreps_in), str(lin.irreps_out), x, w)
    got = run_plan(lin._plan_host, x.detach().numpy(), None, w.numpy())
    assert rel_err(torch.from_numpy(got), ref.detach()) < 1e-6
    go = torch.randn_like(ref)
    ref.backward(go)
    # the transposed plan may hold several groups per input irrep (one per output multiplicity): accumulated
    gx = run_plan(lin._plan_t_host, go.numpy(), None, w.numpy())
    assert rel_err(torch.from_numpy(gx), x.grad) < 1e-6
    strides = {int(lin._plan_t_host[int(lin._plan_t_host[7]) + 6 * g + 5]) for g in range(int(lin._plan_t_host[4]))}
    assert {5, 2} <= strides


def test_operand_gradients_are_transposed_products():
    """`TensorProduct._vjp_module` / `_vjp_weights` against autograd through the oracle (fp64, exact up to rounding)."""
    torch.manual_seed(2)
    tp = o3.FullyConnectedTensorProduct("5x0e+3x1o+2x2e+1x3o", "2x0e+3x1o+1x2e", "4x0e+2x0o+3x1o+2x1e+1x2e")
    Z = 6
    x = torch.randn(Z, tp.irreps_in1.dim, dtype=torch.float64, requires_grad=True)
    y = torch.randn(Z, tp.irreps_in2.dim, dtype=torch.float64, requires_grad=True)
    w = tp.weight.detach().double()
    go = torch.randn(Z, tp.irreps_out.dim, dtype=torch.float64)
    _oracle_tp(tp, x, y, w).backward(go)
    m0, m1 = tp._vjp_module(0), tp._vjp_module(1)
    assert set(m0._vjp_signs) <= {1.0, -1.0} and -1.0 in m0._vjp_signs     # odd permutations of (1, 1, 1)-like triples
    g1 = _oracle_tp(m0, go, y.detach(), tp._vjp_weights(0, w))
    g2 = _oracle_tp(m1, x.detach(), go, tp._vjp_weights(1, w))
    assert rel_err(g1, x.grad) < 1e-12
    assert rel_err(g2, y.grad) < 1e-12
    # and through the plans the kernels would read
    g1p = run_plan(m0._plan_host, go.numpy(), y.detach().numpy(), tp._vjp_weights(0, w).numpy())
    assert rel_err(torch.from_numpy(g1p), x.grad) < 1e-6


def test_linear_plan_rejects_nothing_it_accepts_in_forward():
    # empty instruction lists and zero-multiplicity irreps build (degenerate) plans
    plan, written = linear_plan(o3.Irreps("0x0e+2x1o"), o3.Irreps("3x1o"), o3.Linear("0x0e+2x1o", "3x1o").instructions)
    assert written == [0] and int(plan[4]) == 1


# ----------------------------------------------------------------------------- planner of the post-coupling 'uvw' kernel
UVW_POST_LAYOUTS = [
    ("128x0e+64x1o+32x2e", "0e+1o+2e+3o", "128x0e+64x1o+32x2e"),
    ("32x0e+32x1o+32x2e", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e"),
    ("64x0e+64x1o+64x2e", "0e+1o+2e", "48x0e+32x1o+16x2e"),
    ("96x0e+32x1e+32x2e+32x3o", "0e+1o+2e+3o", "64x0e+32x1o+32x2e+16x3o"),
    ("32x0e+32x1o", "0e+1o", "256x0e+16x1o"),
    ("64x0e+64x1o+64x2e+64x3o", "0e", "64x0e+64x1o+64x2e+64x3o"),
]


def test_uvw_post_plan_covers_every_path_and_fits_the_sm():
    from e3nn_b200 import o3
    from e3nn_b200.codegen import uvw_post

    for layout in UVW_POST_LAYOUTS:
        tp = o3.FullyConnectedTensorProduct(*layout, math_mode="tf32")
        groups = uvw_post.plan_groups(tp._spec)
        assert groups is not None, layout
        covered = {}
        for g in groups:
            assert g.smem_bytes() <= uvw_post.SMEM_LIMIT and g.nacc() <= uvw_post.MAX_ACC_REGS
            assert g.nstage() >= max(b.d1 for b in g.blocks) + 1          # a chunk's component tiles fit the ring together
            assert g.nslots * g.slot_cols <= uvw_post.TMEM_COLS
            for b in g.blocks:
                assert b.ncols <= uvw_post.MAX_N and b.ncols % 16 == 0
                col = 0
                for p in b.paths:                                          # the paths of a block lie side by side
                    m = g.members[p.member]
                    assert p.coloff == col
                    col += m.width
                    covered.setdefault(p.index, []).append((m.col0, m.width))
                assert col == b.ncols
            for j in g.jobs:
                assert 0 <= j.slot0 and j.slot0 + j.nslot <= g.nslots
                assert j.cols(g.blocks) <= j.nslot * g.slot_cols
            # every stage the producers emit is consumed by exactly one job, in the producers' order
            assert sum(len(j.comps) * j.nchunk for j in g.jobs) == g.tiles_per_row_tile()
        # every live path: all of its output channels, once
        for n, ins in tp._spec.live_instructions():
            mul_o = tp._spec.irreps_out[ins.i_out].mul
            slabs = sorted(covered[n])
            assert slabs[0][0] == 0 and sum(w for _, w in slabs) == mul_o
            assert all(a[0] + a[1] == b[0] for a, b in zip(slabs, slabs[1:]))


def test_uvw_post_slot_schedule_is_safe():
    """The issuing thread may overwrite a tensor-memory slot only after the epilogue has read the job that held it,
    and it learns that from mbarrier phases (one bit): replay the static schedule over several row tiles and check
    that (a) every job's slots are free of unread accumulators once its waits are done, and (b) the completions of
    every barrier are observed one by one, in order, before the next job that arrives on that barrier is issued."""
    from e3nn_b200 import o3
    from e3nn_b200.codegen import uvw_post

    for layout in UVW_POST_LAYOUTS:
        tp = o3.FullyConnectedTensorProduct(*layout, math_mode="tf32")
        for g in uvw_post.plan_groups(tp._spec):
            holder = [None] * g.nslots              # (tile, job) whose accumulators a slot holds, None once observed as read
            observed = [0] * g.nslots               # completions of empty[b] the issuing thread has seen
            produced = [0] * g.nslots               # jobs issued so far whose first slot is b (= arrivals the barrier will get)
            for tile in range(4):
                for ji, j in enumerate(g.jobs):
                    for bar, idx, prev in j.waits:
                        if prev and tile == 0:
                            continue                # nothing ran before the first tile
                        t = tile - 1 if prev else tile
                        n = t * g.uses[bar] + idx   # the completion this wait is for
                        assert n == observed[bar], (layout, tile, ji, bar)       # in order, none skipped: parity is enough
                        assert n < produced[bar]                                    # that job has been issued
                        observed[bar] += 1
                        for s in range(g.nslots):   # its slots are free now
                            if holder[s] is not None and holder[s][2] == (bar, n):
                                holder[s] = None
                    for s in range(j.slot0, j.slot0 + j.nslot):
                        assert holder[s] is None, (layout, tile, ji, s, holder[s])
                    n_mine = tile * g.uses[j.slot0] + j.use_idx
                    assert n_mine == produced[j.slot0]                             # the epilogue's phase arithmetic
                    assert observed[j.slot0] == produced[j.slot0]                  # no unobserved completion on my barrier
                    produced[j.slot0] += 1
                    for s in range(j.slot0, j.slot0 + j.nslot):
                        holder[s] = (tile, ji, (j.slot0, n_mine))


def test_transposed_linear_swaps_operands_only_where_it_pays():
    """Groups of a transposed Linear run with swapped MMA operands when 2l+1 is 3 or 5 and the group is a whole number
    of 128-channel MMA tiles; forward Linears, scalars and 2l+1 = 7 keep the row order."""
    from e3nn_b200 import o3

    lin = o3.Linear("128x0e+128x1o+256x2e+128x3o", "64x0e+64x1o+32x2e+32x3o", math_mode="tf32x3")
    assert [(g.n, g.dim, g.swap) for g in lin._tc_bwd.groups] == [(128, 1, False), (128, 3, True), (256, 5, True), (128, 7, False)]
    assert not any(g.swap for g in lin._tc_fwd.groups)
    small = o3.Linear("64x0e+64x1o", "64x0e+64x1o", math_mode="tf32x3")
    assert not any(g.swap for g in small._tc_bwd.groups)          # 64 channels: half an MMA tile
    for g in lin._tc_bwd.groups:
        assert not (g.swap and g.staged_epilogue())
