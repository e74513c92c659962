"""The irreps layouts of the benchmark configurations, and pre-building of their kernel modules."""
from __future__ import annotations

from typing import List, Tuple

from .o3._irreps import Irrep, Irreps
from .o3._tensor_product import TensorProduct


def conv_uvu_layout(irreps_node, irreps_edge, irreps_keep) -> Tuple[Irreps, List[tuple]]:
    """Instruction list of the reference's ``Convolution`` (``e3nn/nn/models/v2106/points_convolution.py:60-76``):
    one 'uvu' path and one output slot per allowed (node irrep, edge irrep, output irrep), output
    slots sorted by (l, p).  ``irreps_keep``: output irreps to keep (0e is always kept)."""
    irreps_node, irreps_edge, irreps_keep = Irreps(irreps_node), Irreps(irreps_edge), Irreps(irreps_keep)
    mid, ins = [], []
    for i, (mul, ir_in) in enumerate(irreps_node):
        for j, (_, ir_edge) in enumerate(irreps_edge):
            for ir_out in ir_in * ir_edge:
                if ir_out in irreps_keep or ir_out == Irrep(0, 1):
                    ins.append((i, j, len(mid), "uvu", True))
                    mid.append((mul, ir_out))
    mid, p, _ = Irreps(mid).sort()
    return mid, [(a, b, p[c], mode, train) for a, b, c, mode, train in ins]


def conv_tensor_product(irreps_node, irreps_edge, irreps_keep) -> TensorProduct:
    mid, ins = conv_uvu_layout(irreps_node, irreps_edge, irreps_keep)
    return TensorProduct(irreps_node, irreps_edge, mid, ins, internal_weights=False, shared_weights=False)


ALL_L2 = "0e+0o+1e+1o+2e+2o"

# name -> (node irreps, edge irreps, kept output irreps)
BENCH_CONV_LAYOUTS = {
    "cfg3_15": ("64x0e+64x1o+64x2e", "0e+1o+2e", ALL_L2),
    "cfg3_11": ("64x0e+64x1o+64x2e", "0e+1o+2e", "0e+1o+2e"),
    "cfg5_23": ("64x0e+64x1o+64x2e+64x3o", "0e+1o+2e+3o", "0e+1o+2e+3o"),
}


def bench_conv_tp(name: str) -> TensorProduct:
    return conv_tensor_product(*BENCH_CONV_LAYOUTS[name])
