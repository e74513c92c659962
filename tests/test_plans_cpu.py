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
