"""Generate the golden vectors in this folder by running the reference e3nn itself.

Run where the e3nn 0.6.0 sources are available: the ``E3NN_REFERENCE`` environment variable
names the directory that contains the ``e3nn`` package.  The only missing dependency of the reference,
``opt_einsum_fx`` (a contraction-order optimiser that does not change the mathematics),
is replaced by an identity stand-in before ``import e3nn``.

    python tests/golden/make_golden.py              (everything)
    python tests/golden/make_golden.py --only-gate  (only the Gate cases, leaving the other files untouched)
    python tests/golden/make_golden.py --only-activation
    python tests/golden/make_golden.py --only-radial-bases
    python tests/golden/make_golden.py --only-uuu

Every case stores its fp32 inputs and the reference's fp64 output on those inputs
(inputs upcast to fp64), plus the reference's own fp32 output for context.  The files
are small on purpose: the layouts are those of the benchmark configurations, the batch is a handful of rows.
"""
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _import_reference():
    stub = types.ModuleType("opt_einsum_fx")
    stub.optimize_einsums_full = lambda model, example_inputs, **kw: model
    stub.jitable = lambda gm: gm
    sys.modules["opt_einsum_fx"] = stub
    ref = os.environ.get("E3NN_REFERENCE")
    if not ref:
        raise SystemExit("set E3NN_REFERENCE to the directory that contains the e3nn package")
    sys.path.insert(0, ref)
    import e3nn  # noqa: F401
    from e3nn import o3

    return e3nn, o3


def _np(t):
    return t.detach().cpu().numpy()


def _run_both(fn, *inputs32):
    """fn evaluated at fp64 (on upcast inputs) and fp32."""
    out64 = fn(torch.float64, *[t.double() if t.is_floating_point() else t for t in inputs32])
    out32 = fn(torch.float32, *inputs32)
    return _np(out64), _np(out32)


def conv_layout(o3, irreps_node, irreps_edge, keep):
    """Instruction list of the Convolution recipe (nn/models/v2106/points_convolution.py:60-76)."""
    irreps_node, irreps_edge, keep = o3.Irreps(irreps_node), o3.Irreps(irreps_edge), o3.Irreps(keep)
    mid, ins = [], []
    for i, (mul, ir_in) in enumerate(irreps_node):
        for j, (_, ir_edge) in enumerate(irreps_edge):
            for ir_out in ir_in * ir_edge:
                if ir_out in keep or ir_out == o3.Irrep(0, 1):
                    ins.append((i, j, len(mid), "uvu", True))
                    mid.append((mul, ir_out))
    mid, p, _ = o3.Irreps(mid).sort()
    ins = [(a, b, p[c], m, t) for a, b, c, m, t in ins]
    return mid, ins


GATE_CASES = {
    "gate_mixed": ("16x0e+8x0o", ["silu", "tanh"], "8x0e+4x0o", ["sigmoid", "tanh"], "8x1o+4x2e"),
    "gate_l3": ("32x0e", ["silu"], "24x0e", ["sigmoid"], "8x1o+8x2e+8x3o"),
    "gate_abs_identity": ("4x0o", ["abs"], "6x0e", [None], "2x1e+4x1o"),
    "gate_no_scalars": ("", [], "3x0e", ["relu"], "3x2e"),
}


def gate_cases(meta):
    """Gate.forward of the reference on seeded rows (e3nn/nn/_gate.py:127-144); activations are stored by name."""
    from e3nn.nn import Gate

    fn = {"silu": torch.nn.functional.silu, "tanh": torch.tanh, "sigmoid": torch.sigmoid, "abs": torch.abs,
          "relu": torch.relu, None: None}
    gen = torch.Generator().manual_seed(1234)
    for name, (sc, act_s, ga, act_g, gd) in GATE_CASES.items():
        g = Gate(sc, [fn[a] for a in act_s], ga, [fn[a] for a in act_g], gd)
        x = torch.randn(9, g.irreps_in.dim, generator=gen)
        out64 = g(x.double())
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), x=_np(x), out_f64=_np(out64))
        meta["cases"][name] = {"irreps_scalars": sc, "act_scalars": act_s, "irreps_gates": ga, "act_gates": act_g,
                               "irreps_gated": gd, "irreps_in": str(g.irreps_in), "irreps_out": str(g.irreps_out)}


ACTIVATION_CASES = {
    "activation_mixed": ("16x0e+8x0o+4x1e", ["silu", "tanh", None]),
    "activation_abs": ("8x0o", ["abs"]),
    "activation_identity": ("4x0e+4x1o", [None, None]),
    "activation_relu_sigmoid": ("5x0e+3x0e+2x2e", ["relu", "sigmoid", None]),
}


def activation_cases(meta):
    """Activation.forward of the reference on seeded rows (e3nn/nn/_activation.py:80-111)."""
    from e3nn.nn import Activation

    fn = {"silu": torch.nn.functional.silu, "tanh": torch.tanh, "sigmoid": torch.sigmoid, "abs": torch.abs,
          "relu": torch.relu, None: None}
    gen = torch.Generator().manual_seed(4242)
    for name, (irreps, acts) in ACTIVATION_CASES.items():
        a = Activation(irreps, [fn[n] for n in acts])
        x = torch.randn(7, a.irreps_in.dim, generator=gen)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), x=_np(x), out_f64=_np(a(x.double())))
        meta["cases"][name] = {"irreps_in": irreps, "acts": acts, "irreps_out": str(a.irreps_out)}


def radial_basis_cases(meta):
    """soft_one_hot_linspace for every basis / cutoff flag and smooth_cutoff, on seeded radii in (0, 6)."""
    from e3nn.math import soft_one_hot_linspace
    from e3nn.nn.models.gate_points_2101 import smooth_cutoff

    gen = torch.Generator().manual_seed(4321)
    r = torch.rand(64, generator=gen, dtype=torch.float64) * 6.0 + 1e-3
    out = {"r": _np(r), "smooth_cutoff": _np(smooth_cutoff(r / 5.0))}
    for basis in ("gaussian", "cosine", "smooth_finite", "fourier", "bessel"):
        for cutoff in (False, True):
            out[f"{basis}_{int(cutoff)}"] = _np(soft_one_hot_linspace(r, 0.5, 5.0, 8, basis=basis, cutoff=cutoff))
    np.savez_compressed(os.path.join(HERE, "radial_bases.npz"), **out)
    meta["cases"]["radial_bases"] = {"start": 0.5, "end": 5.0, "number": 8}


def _tp_case(meta, name, tp_factory, Z, shared, weight_scale=None, norm_kwargs=None):
    tp32 = tp_factory()
    x1 = torch.randn(Z, tp32.irreps_in1.dim)
    x2 = torch.randn(Z, tp32.irreps_in2.dim)
    w = torch.randn(tp32.weight_numel) if shared else torch.randn(Z, tp32.weight_numel)
    if weight_scale is not None:
        w = w * weight_scale(tp32)
    torch.set_default_dtype(torch.float64)
    tp64 = tp_factory()
    torch.set_default_dtype(torch.float32)
    out64 = tp64(x1.double(), x2.double(), w.double())
    out32 = tp32(x1, x2, w)
    np.savez_compressed(
        os.path.join(HERE, f"{name}.npz"), x1=_np(x1), x2=_np(x2), w=_np(w), out_f64=_np(out64), out_f32=_np(out32)
    )
    meta["cases"][name] = {
        "irreps_in1": str(tp32.irreps_in1),
        "irreps_in2": str(tp32.irreps_in2),
        "irreps_out": str(tp32.irreps_out),
        "instructions": [
            [i.i_in1, i.i_in2, i.i_out, i.connection_mode, bool(i.has_weight), float(i.path_weight)]
            for i in tp32.instructions
        ],
        "weight_numel": tp32.weight_numel,
        "shared_weights": shared,
        "output_mask": _np(tp32.output_mask).astype(int).tolist(),
        "norm_kwargs": norm_kwargs or {},
    }



def uuu_cases(meta):
    """'uuu' paths: the reference's ElementwiseTensorProduct (no weights) and a weighted mix with 'uvu' / 'uvw'."""
    from e3nn import o3

    torch.manual_seed(7)
    _tp_case(meta, "tp_elementwise", lambda: o3.ElementwiseTensorProduct("4x0e+3x1o+2x2e+5x1e", "4x0e+3x1o+2x1o+5x2e"), 16, True)

    def mixed():
        return o3.TensorProduct(
            "4x0e+3x1o+2x2e", "4x0e+3x1o+1x1o+3x0e", "4x0e+3x1o+3x1e+2x2e",
            [(0, 0, 0, "uuu", True), (1, 3, 1, "uuu", True), (1, 1, 2, "uuu", False), (1, 1, 2, "uuu", True),
             (2, 0, 3, "uvu", True), (1, 2, 0, "uvw", True), (1, 1, 3, "uvw", True, 0.5)],
            internal_weights=False, shared_weights=True,
        )

    _tp_case(meta, "tp_uuu_mixed_shared", mixed, 16, True)

    def unshared():
        return o3.TensorProduct(
            "3x0e+3x1o", "3x1o+3x2e", "3x1o+3x1e+3x0e",
            [(0, 0, 0, "uuu", True), (1, 0, 1, "uuu", True), (1, 0, 2, "uuu", True), (1, 1, 0, "uuu", True)],
            internal_weights=False, shared_weights=False,
        )

    _tp_case(meta, "tp_uuu_unshared", unshared, 16, False)
    # 'uvuv' paths: the reference's FullTensorProduct (no weights, sorted output) and a weighted mix
    _tp_case(meta, "tp_full", lambda: o3.FullTensorProduct("2x0e+3x1o+1x2e", "2x0e+2x1o+1x1e"), 16, True)

    def uvuv_mixed():
        return o3.TensorProduct(
            "2x0e+3x1o", "2x1o+4x0e", "6x0e+6x1e+3x1o+8x0e",
            [(1, 0, 0, "uvuv", True), (1, 0, 1, "uvuv", False), (1, 1, 2, "uvu", True), (0, 1, 3, "uvuv", True, 2.0),
             (1, 0, 3, "uvw", True)],
            internal_weights=False, shared_weights=False,
        )

    _tp_case(meta, "tp_uvuv_mixed_unshared", uvuv_mixed, 16, False)

    # the remaining connection modes: 'uvv', 'uuw', 'uvu<v', 'u<vw' (weighted and not), shared and per-row weights
    def rest(shared):
        return lambda: o3.TensorProduct(
            "4x0e+4x1o+1x1o", "4x1o+4x0e+3x1e", "4x1o+5x0e+6x1e+1x2e+3x1o+6x0e",
            [(0, 0, 0, "uvv", True), (1, 0, 1, "uuw", True), (1, 0, 2, "uvu<v", True), (1, 0, 1, "u<vw", True, 0.7),
             (1, 0, 3, "uuw", False), (4 - 2, 2, 4, "uvv", False), (0, 1, 5, "uvu<v", False)],
            internal_weights=False, shared_weights=shared,
        )

    _tp_case(meta, "tp_rest_shared", rest(True), 16, True)
    _tp_case(meta, "tp_rest_unshared", rest(False), 16, False)

    # TensorSquare: one input, unweighted (full) and weighted (fully connected) forms
    for name, args in (("square_full", ("2x0e+3x1o+2x2e",)), ("square_connected", ("2x0e+3x1o+2x2e", "4x0e+3x1o+2x2e+1x1e"))):
        sq32 = o3.TensorSquare(*args, internal_weights=False) if len(args) > 1 else o3.TensorSquare(*args)
        x = torch.randn(16, sq32.irreps_in.dim)
        w = torch.randn(sq32.weight_numel)
        torch.set_default_dtype(torch.float64)
        sq64 = o3.TensorSquare(*args, internal_weights=False) if len(args) > 1 else o3.TensorSquare(*args)
        torch.set_default_dtype(torch.float32)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), x=_np(x), w=_np(w), out_f64=_np(sq64(x.double(), w.double())),
                            out_f32=_np(sq32(x, w)))
        meta["cases"][name] = {
            "args": list(args), "irreps_out": str(sq32.irreps_out), "weight_numel": sq32.weight_numel,
            "instructions": [[i.i_in1, i.i_in2, i.i_out, i.connection_mode, bool(i.has_weight), float(i.path_weight)]
                             for i in sq32.instructions],
        }


def main():
    if "--only-uuu" in sys.argv:
        _import_reference()
        with open(os.path.join(HERE, "meta.json")) as f:
            meta = json.load(f)
        uuu_cases(meta)
        with open(os.path.join(HERE, "meta.json"), "w") as f:
            json.dump(meta, f, indent=1)
        print("'uuu' golden vectors written to", HERE)
        return
    if "--only-radial-bases" in sys.argv:
        _import_reference()
        with open(os.path.join(HERE, "meta.json")) as f:
            meta = json.load(f)
        radial_basis_cases(meta)
        with open(os.path.join(HERE, "meta.json"), "w") as f:
            json.dump(meta, f, indent=1)
        print("radial basis golden vectors written to", HERE)
        return
    if "--only-activation" in sys.argv:
        _import_reference()
        with open(os.path.join(HERE, "meta.json")) as f:
            meta = json.load(f)
        activation_cases(meta)
        with open(os.path.join(HERE, "meta.json"), "w") as f:
            json.dump(meta, f, indent=1)
        print("activation golden vectors written to", HERE)
        return
    if "--only-gate" in sys.argv:
        _import_reference()
        with open(os.path.join(HERE, "meta.json")) as f:
            meta = json.load(f)
        gate_cases(meta)
        with open(os.path.join(HERE, "meta.json"), "w") as f:
            json.dump(meta, f, indent=1)
        print("gate golden vectors written to", HERE)
        return
    e3nn, o3 = _import_reference()
    from e3nn.math import bessel
    from e3nn.nn import FullyConnectedNet

    torch.manual_seed(0)
    meta = {"e3nn_version": e3nn.__version__, "torch": torch.__version__, "cases": {}}

    # ---- Clebsch-Gordan -------------------------------------------------------------
    cg = {}
    for l1 in range(5):
        for l2 in range(5):
            for l3 in range(abs(l1 - l2), min(l1 + l2, 4) + 1):
                cg[f"{l1}_{l2}_{l3}"] = _np(o3.wigner_3j(l1, l2, l3, dtype=torch.float64))
    for t in [(5, 1, 4), (6, 1, 5), (5, 5, 6), (6, 6, 6)]:
        cg["%d_%d_%d" % t] = _np(o3.wigner_3j(*t, dtype=torch.float64))
    np.savez_compressed(os.path.join(HERE, "wigner_3j.npz"), **cg)

    # ---- spherical harmonics ----------------------------------------------------------
    vec = torch.randn(48, 3)
    vec[0] = 0.0  # zero vector: Y0 = 1, rest 0 when normalize=True
    vec[1] = torch.tensor([0.0, 1.0, 0.0])
    vec[2] = torch.tensor([1.0, 0.0, 0.0])
    vec[3] = torch.tensor([0.0, 0.0, -2.5])
    sh = {"vec": _np(vec)}
    for norm in ("component", "integral", "norm"):
        for normalize in (True, False):
            for lmax in (3, 6):
                ls = list(range(lmax + 1))
                o64, o32 = _run_both(
                    lambda dt, v: o3.spherical_harmonics(ls, v, normalize, norm), vec
                )
                sh[f"l{lmax}_{norm}_{int(normalize)}_f64"] = o64
                sh[f"l{lmax}_{norm}_{int(normalize)}_f32"] = o32
    o64, _ = _run_both(lambda dt, v: o3.spherical_harmonics([2, 0, 3, 2], v, True, "norm"), vec)
    sh["ls_2_0_3_2_norm_1_f64"] = o64
    o64, _ = _run_both(lambda dt, v: o3.spherical_harmonics(list(range(9)), v, True, "component"), vec)
    sh["l8_component_1_f64"] = o64
    np.savez_compressed(os.path.join(HERE, "spherical_harmonics.npz"), **sh)

    # ---- tensor products --------------------------------------------------------------
    def tp_case(name, tp_factory, Z, shared, weight_scale=None, norm_kwargs=None):
        _tp_case(meta, name, tp_factory, Z, shared, weight_scale, norm_kwargs)

    def fctp(a, b, c):
        return lambda: o3.FullyConnectedTensorProduct(a, b, c, internal_weights=False, shared_weights=True)

    def conv_tp(node, edge, keep):
        def make():
            mid, ins = conv_layout(o3, node, edge, keep)
            return o3.TensorProduct(node, edge, mid, ins, internal_weights=False, shared_weights=False)

        return make

    tp_case("tp_cfg1_uvw", fctp("32x0e+32x1o+32x2e", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e"), 24, True)
    tp_case("tp_cfg4_uvw", fctp("128x0e+64x1o+32x2e", "0e+1o+2e+3o", "128x0e+64x1o+32x2e"), 12, True)
    tp_case("tp_small_uvw", fctp("3x0e+2x1o+4x2e+1x1e", "2x0e+3x1o+1x2e", "5x0e+2x1o+3x2e+2x1e+1x3o"), 16, True)
    all_l2 = "0e+0o+1e+1o+2e+2o"
    tp_case("tp_cfg3_uvu_15", conv_tp("64x0e+64x1o+64x2e", "0e+1o+2e", all_l2), 12, False)
    tp_case("tp_cfg3_uvu_11", conv_tp("64x0e+64x1o+64x2e", "0e+1o+2e", "0e+1o+2e"), 12, False)
    tp_case("tp_cfg5_uvu_23", conv_tp("64x0e+64x1o+64x2e+64x3o", "0e+1o+2e+3o", "0e+1o+2e+3o"), 8, False)
    tp_case("tp_small_uvu", conv_tp("3x0e+5x1o+2x2e+4x1e", "0e+1o+2e", all_l2), 16, False)

    def general_uvu():
        # 'uvu' with in2 multiplicities > 1, two paths into one output, an unweighted path,
        # a custom path weight and an output nothing writes to.
        return o3.TensorProduct(
            "4x0e+3x1o+2x2e", "2x0e+3x1o", "4x0e+3x1o+3x1e+2x2e+5x3e",
            [
                (0, 0, 0, "uvu", True), (1, 1, 0, "uvw", True), (1, 0, 1, "uvu", True), (1, 1, 2, "uvu", False),
                (2, 1, 1, "uvw", True, 2.5), (2, 0, 3, "uvu", True), (1, 1, 3, "uvw", True),
            ],
            internal_weights=False, shared_weights=True,
        )

    tp_case("tp_mixed_shared", general_uvu, 16, True)

    def general_uvu_unshared():
        return o3.TensorProduct(
            "4x0e+3x1o+2x2e", "2x0e+3x1o", "4x0e+3x1o+2x2e",
            [(0, 0, 0, "uvu", True), (1, 0, 1, "uvu", True), (0, 1, 1, "uvw", True), (2, 0, 2, "uvu", True),
             (1, 1, 2, "uvw", True)],
            internal_weights=False, shared_weights=False, irrep_normalization="norm", path_normalization="path",
        )

    tp_case("tp_mixed_unshared", general_uvu_unshared, 16, False,
            norm_kwargs={"irrep_normalization": "norm", "path_normalization": "path"})

    # ---- Linear ----------------------------------------------------------------------
    def lin_case(name, irreps_in, irreps_out, Z, biases=False):
        torch.set_default_dtype(torch.float64)
        lin = o3.Linear(irreps_in, irreps_out, biases=biases)
        torch.set_default_dtype(torch.float32)
        x = torch.randn(Z, lin.irreps_in.dim)
        w = torch.randn(lin.weight_numel)
        b = torch.randn(lin.bias_numel)
        out64 = lin(x.double(), w.double(), b.double())
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), x=_np(x), w=_np(w), b=_np(b), out_f64=_np(out64))
        meta["cases"][name] = {
            "irreps_in": str(lin.irreps_in),
            "irreps_out": str(lin.irreps_out),
            "instructions": [[i.i_in, i.i_out, list(i.path_shape), float(i.path_weight)] for i in lin.instructions],
            "weight_numel": lin.weight_numel,
            "bias_numel": lin.bias_numel,
            "biases": bool(biases),
            "output_mask": _np(lin.output_mask).astype(int).tolist(),
        }

    lin_case("linear_cfg4", "128x0e+64x1o+32x2e", "128x0e+64x1o+32x2e", 12)
    mid5, _ = conv_layout(o3, "64x0e+64x1o+64x2e+64x3o", "0e+1o+2e+3o", "0e+1o+2e+3o")
    lin_case("linear_cfg5", str(mid5), "64x0e+64x1o+64x2e+64x3o", 6)
    lin_case("linear_small_bias", "3x0e+2x1o+4x0e+1x2e", "5x0e+2x1o+3x1o+2x0e+1x3o", 16, biases=True)

    # ---- radial network --------------------------------------------------------------
    r = torch.rand(32) * 5.0
    r[0] = 0.0
    torch.set_default_dtype(torch.float64)
    fc = FullyConnectedNet([8, 64, 96], torch.nn.functional.silu)
    torch.set_default_dtype(torch.float32)
    b64 = bessel(r.double(), 8, 5.0)
    out64 = fc(b64)
    np.savez_compressed(
        os.path.join(HERE, "radial.npz"),
        r=_np(r), bessel_f64=_np(b64), w0=_np(fc.layer0.weight), w1=_np(fc.layer1.weight), out_f64=_np(out64),
        silu_cst=np.array(fc.layer0.act.cst),
    )

    # ---- fused convolution step: gather -> SH -> uvu -> scatter -> Linear -----------------
    N, E = 10, 40
    mid, ins = conv_layout(o3, "8x0e+8x1o+8x2e", "0e+1o+2e", all_l2)
    torch.set_default_dtype(torch.float64)
    tp = o3.TensorProduct("8x0e+8x1o+8x2e", "0e+1o+2e", mid, ins, internal_weights=False, shared_weights=False)
    lin = o3.Linear(mid, "8x0e+8x1o+8x2e")
    torch.set_default_dtype(torch.float32)
    node_x = torch.randn(N, 72)
    vec = torch.randn(E, 3)
    src = torch.randint(0, N, (E,))
    dst = torch.randint(0, N - 2, (E,))  # nodes N-2, N-1 receive nothing
    w = torch.randn(E, tp.weight_numel)
    lw = torch.randn(lin.weight_numel)
    y = o3.spherical_harmonics([0, 1, 2], vec.double(), True, "component")
    msg = tp(node_x.double()[src], y, w.double())
    agg = torch.zeros(N, mid.dim, dtype=torch.float64).index_add_(0, dst, msg) / 4.0 ** 0.5
    out = lin(agg, lw.double())
    np.savez_compressed(
        os.path.join(HERE, "conv_small.npz"),
        node_x=_np(node_x), vec=_np(vec), src=_np(src), dst=_np(dst), w=_np(w), lin_w=_np(lw),
        msg_f64=_np(msg), agg_f64=_np(agg), out_f64=_np(out),
    )
    meta["cases"]["conv_small"] = {
        "irreps_node": "8x0e+8x1o+8x2e", "irreps_edge": "0e+1o+2e", "irreps_mid": str(mid),
        "instructions": [list(i) for i in ins], "num_nodes": N, "scale": 0.5,
    }

    gate_cases(meta)
    radial_basis_cases(meta)

    with open(os.path.join(HERE, "meta.json"), "w") as f:
        json.dump(meta, f, indent=1)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
