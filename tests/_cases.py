"""Layouts used by the GPU property tests (seeded, so they can be pre-built without a GPU)."""
import random

from e3nn_b200 import layouts, o3


def random_conv_layouts(n=4, seed=0):
    rng = random.Random(seed)
    out = []
    for _ in range(n):
        irreps = []
        for _ in range(rng.randint(1, 4)):
            l = rng.randint(0, 3)
            irreps.append((rng.choice([1, 2, 3, 5, 8, 16, 33]), (l, rng.choice([-1, 1]))))
        node = o3.Irreps(irreps)
        lmax = rng.randint(1, 3)
        edge = o3.Irreps.spherical_harmonics(lmax)
        keep = o3.Irreps([(1, ir) for ir in o3.Irrep.iterator(3)])
        out.append((str(node), str(edge), str(keep)))
    return out


def conv_tps():
    return [layouts.conv_tensor_product(*t) for t in random_conv_layouts()] + [
        layouts.conv_tensor_product("8x0e+8x1o+8x2e", "0e+1o+2e", layouts.ALL_L2),
        layouts.conv_tensor_product("16x0e+16x1o+16x2e+16x3o", "0e+1o+2e+3o", "0e+1o+2e+3o"),
    ]


# layouts that exercise the planner of the post-coupling tensor-core kernel: merged output irreps, slabs of unequal
# width, blocks whose components are all live at once (several 32-channel chunks), odd-parity irreps, a scalar-only
# second operand
UVW_TC_EXTRA_LAYOUTS = [
    ("64x0e+64x1o+64x2e", "0e+1o+2e", "48x0e+32x1o+16x2e"),
    ("96x0e+32x1e+32x2e+32x3o", "0e+1o+2e+3o", "64x0e+32x1o+32x2e+16x3o"),
    ("32x0e+32x1o", "0e+1o", "256x0e+16x1o"),
    ("64x0e+64x1o+64x2e+64x3o", "0e", "64x0e+64x1o+64x2e+64x3o"),
]


def prebuild():
    from e3nn_b200 import prebuild as pb

    for tp in conv_tps():
        tp._uvu_module()
    # layouts of the tensor-core tests
    for layout in UVW_TC_EXTRA_LAYOUTS:
        pb._build_tp(o3.FullyConnectedTensorProduct(*layout, math_mode="tf32"))
    for layout in [("32x0e+32x1o+32x2e", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e"),
                   ("128x0e+64x1o+32x2e", "0e+1o+2e+3o", "128x0e+64x1o+32x2e")]:
        pb._build_tp(o3.FullyConnectedTensorProduct(*layout, math_mode="tf32x3"))
        # the derived product that gives the gradient w.r.t. the first operand in the tensor-core modes
        for mode in ("tf32", "tf32x3"):
            pb._build_tp(o3.FullyConnectedTensorProduct(*layout, math_mode=mode)._vjp_module(0))
    pb._build_linear(o3.Linear("64x0e+64x1o+64x2e+64x3o", "256x0e+64x1o+64x2e+64x3o", math_mode="tf32x3"))   # Linear -> Gate
    pb._build_linear(o3.Linear("16x0e+8x1o+4x2e", "8x0e+8x1o+4x2e"))
    pb._build_linear(o3.Linear("64x0e+32x1o+32x2e", "32x0e+64x1o+32x2e"))
    for mode in ("fp32", "tf32x3", "tf32"):
        pb._build_linear(o3.Linear("128x0e+128x1o+256x2e+128x3o", "64x0e+64x1o+32x2e+32x3o", math_mode=mode))
    pb._build_tp(o3.ElementwiseTensorProduct("4x0e+3x1o+2x2e+5x1e", "4x0e+3x1o+2x1o+5x2e"))
    pb._build_tp(o3.ElementwiseTensorProduct("5x1o+5x1e", "10x1e", ["0e", "0o"]))
    pb._build_tp(o3.FullTensorProduct("2x0e+3x1o+1x2e", "2x0e+2x1o+1x1e"))
    pb._build_tp(o3.TensorSquare("2x0e+3x1o+2x2e"))
    pb._build_tp(o3.TensorSquare("2x0e+3x1o+2x2e", "4x0e+3x1o+2x2e+1x1e"))
    pb._build_tp(o3.Norm("5x0e+4x1o+3x2e+2x3o").tp)
