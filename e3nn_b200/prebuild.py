"""Ahead-of-time build of the core library and of the layout modules a deployment needs.

``python -m e3nn_b200.prebuild`` builds ``libe3nn_b200.so`` and the modules of the benchmark
layouts; ``prebuild_cases(path)`` additionally builds every 'uvu' layout listed in a JSON file of
cases (the format of ``tests/golden/meta.json``), so that a machine without nvcc can load them.
"""
from __future__ import annotations

import json
from concurrent.futures import ThreadPoolExecutor
from typing import Iterable, List

from . import _build, _lib
from .layouts import BENCH_CONV_LAYOUTS, bench_conv_tp
from .o3._tensor_product import TensorProduct


def _build_tp(tp: TensorProduct) -> str:
    """Every generated module a TensorProduct can use: 'uvu' layout module, tf32 and fp32 tensor-core modules."""
    from .codegen import tc_gemm, uvw_post, uvw_tc

    paths = []
    if tp._has_uvu:
        paths.append(tp._uvu_module().path)
    for n in tp._uuu_ids:
        paths.append(tp._uuu_sub(n)._uvu_module().path)
    if tp._uvw_ids and not tp._has_uvu:
        if uvw_post.plan_groups(tp._spec) is not None or uvw_tc.plan_groups(tp._spec) is not None:
            paths.append(_lib.uvw_tc_module(tp._spec).path)
        gs = tc_gemm.uvw_gemm_spec(tp._spec)
        if gs is not None:
            paths.append(_lib.tc_gemm_module(gs).path)
    return ";".join(paths)


def _build_linear(lin) -> str:
    paths = []
    for gs in (lin._tc_fwd, lin._tc_bwd):
        if gs is not None:
            paths.append(_lib.tc_gemm_module(gs).path)
    return ";".join(paths)


def prebuild_linears() -> List[str]:
    from .o3._linear import Linear

    lins = [
        Linear("128x0e+64x1o+32x2e", "128x0e+64x1o+32x2e"),
        Linear(bench_conv_tp("cfg5_23").irreps_out, "64x0e+64x1o+64x2e+64x3o"),
        Linear(bench_conv_tp("cfg3_15").irreps_out, "64x0e+64x1o+64x2e", math_mode="tf32x3"),
    ]
    with ThreadPoolExecutor(max_workers=4) as pool:
        return list(pool.map(_build_linear, lins))


def prebuild_bench_layouts() -> List[str]:
    tps = [bench_conv_tp(name) for name in BENCH_CONV_LAYOUTS]
    with ThreadPoolExecutor(max_workers=4) as pool:
        return list(pool.map(_build_tp, tps))


def tps_from_cases(path: str) -> Iterable[TensorProduct]:
    with open(path) as f:
        cases = json.load(f)["cases"]
    for name, m in cases.items():
        if "irreps_in1" not in m:
            continue
        ins = [tuple(i[:5]) for i in m["instructions"]]
        # path weights in the file are final coefficients; the layout key depends on them, so the
        # user-level instruction list (with its custom weights) has to be rebuilt by the caller for
        # exotic cases.  The golden cases only use default weights except where noted there.
        if name == "tp_mixed_shared":
            ins[4] = ins[4] + (2.5,)
        if name == "tp_uuu_mixed_shared":
            ins[6] = ins[6] + (0.5,)
        if name == "tp_uvuv_mixed_unshared":
            ins[3] = ins[3] + (2.0,)
        if name in ("tp_rest_shared", "tp_rest_unshared"):
            ins[3] = ins[3] + (0.7,)
        yield TensorProduct(m["irreps_in1"], m["irreps_in2"], m["irreps_out"], ins, internal_weights=False,
                            shared_weights=m["shared_weights"], **m.get("norm_kwargs", {}))


def prebuild_cases(path: str) -> List[str]:
    tps = list(tps_from_cases(path))
    with ThreadPoolExecutor(max_workers=4) as pool:
        return list(pool.map(_build_tp, tps))


def prebuild_radial() -> List[str]:
    """Tensor-core modules of the 64 -> weight_numel radial layers of the benchmark interaction block."""
    from .nn._fc import _Layer

    out = []
    for wn in (bench_conv_tp("cfg5_23").weight_numel,):
        layer = _Layer(64, wn, None, 1.0, 1, 1, "tf32x3")
        for gs in layer._tc_specs():
            if gs is not None:
                out.append(_lib.tc_gemm_module(gs).path)
    return out


def main() -> None:
    print(_build.build_core())
    for so in prebuild_bench_layouts() + prebuild_linears() + prebuild_radial():
        print(so)


if __name__ == "__main__":
    main()
