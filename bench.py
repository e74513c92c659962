"""Throughput of the e3nn message-passing hot path on B200, one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Workloads (synthetic, seeded; shapes and distributions of the benchmark configurations):
  conv_l2_15   fused gather -> SH(lmax 2) -> 'uvu' (15 paths, 64 channels) -> per-destination sum;
               65,536 nodes, 2,097,152 edges, in-degree 32, uniform random sources, per-edge weights.
  conv_l2_11   same graph, the 11-path layout (outputs restricted to the node irreps).
  conv_l3_23   the 'uvu' l<=3 layout (23 paths, 64x0e+64x1o+64x2e+64x3o), same graph shape.
  sh_l3        spherical harmonics lmax 3 on 4,194,304 edge vectors.
  gate         Gate non-linearity (64 scalars, 192 gates, 64x1o+64x2e+64x3o gated) on 1,048,576 rows, forward.
  interaction_l3  one NequIP-style interaction block, forward + gradient w.r.t. positions: 262,144 atoms uniform in
               a periodic cube at 0.05 / A^3, 5 A cutoff (~26 neighbours), features 64x0e+64x1o+64x2e+64x3o,
               SH lmax 3, Bessel(8) -> 64 -> 1472 radial MLP, 23-path 'uvu', scatter / sqrt(n), Linear.
  uvw_fctp     FullyConnectedTensorProduct 128x0e+64x1o+32x2e (x) 0e+1o+2e+3o -> same, shared weights,
               1,048,576 rows, tcgen05 tf32 kernel, followed by o3.Linear (fp32) on the output.

A "step" is one pass of the hot path over the whole graph.  `value` is timed with CUDA events on the
launching stream with every input resident in HBM (inputs are far larger than L2, nothing is cached
between steps); `e2e` runs the same step through the public Python API from pinned host buffers,
copies included.  With --gpus N (launched by torchrun) destination rows are split into N contiguous
ranges, each rank owns the features of its own rows and all-gathers the source features every step
(strong scaling; NCCL).  `--impl reference` times the CPU oracle (a restatement of e3nn's own
arithmetic with torch CPU operators, all host threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    # name: (layout, nodes, in-degree)
    "conv_l2_15": ("cfg3_15", 65536, 32),
    "conv_l2_11": ("cfg3_11", 65536, 32),
    "conv_l3_23": ("cfg5_23", 65536, 32),
}
DEFAULT_WORKLOAD = "interaction_l3"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------- workload
def make_graph(layout: str, nodes: int, degree: int, rank: int, world: int, device):
    """This rank's shard: destination rows [n0, n1), their edges (already sorted by destination)."""
    from e3nn_b200 import layouts

    tp = layouts.bench_conv_tp(layout)
    n0, n1 = nodes * rank // world, nodes * (rank + 1) // world
    n_local = n1 - n0
    e_local = n_local * degree
    gen = torch.Generator(device=device).manual_seed(1234 + rank)
    data = {
        "tp": tp, "nodes": nodes, "n0": n0, "n_local": n_local, "e_local": e_local, "degree": degree,
        "node_x_local": torch.randn(n_local, tp.irreps_in1.dim, device=device, generator=gen),
        "vec": torch.nn.functional.normalize(torch.randn(e_local, 3, device=device, generator=gen), dim=-1),
        "src": torch.randint(0, nodes, (e_local,), device=device, generator=gen),
        "rowptr": torch.arange(0, e_local + 1, degree, device=device, dtype=torch.int64),
        "w": torch.randn(e_local, tp.weight_numel, device=device, generator=gen),
    }
    return data


def conv_step(d, node_x_full, world):
    import e3nn_b200

    if world > 1:
        torch.distributed.all_gather_into_tensor(node_x_full, d["node_x_local"])
    return e3nn_b200.conv_uvu(d["tp"], node_x_full, d["vec"], d["src"], d["rowptr"], d["w"],
                              scale=d["degree"] ** -0.5, edge_attr_is_vector=True)


def algorithmic_bytes_per_edge(tp, nodes, edges):
    """Unique bytes the fused step must move: per edge weights + vector + int64 src/dst,
    per node one read of its features and one write of its output row."""
    per_edge = 4 * tp.weight_numel + 12 + 16
    per_node = 4 * tp.irreps_in1.dim + 4 * tp.irreps_out.dim
    return per_edge + per_node * nodes / edges


def run_ours(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("bench.py --gpus N>1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        from e3nn_b200 import sharding

        sharding.init_process_group("nccl", device, timeout_s=600.0)

    if args.workload == "sh_l3":
        return run_sh(args, rank, world, device)
    if args.workload == "gate":
        return run_gate(args, rank, world, device)
    if args.workload == "uvw_fctp":
        return run_uvw(args, rank, world, device)
    if args.workload == "uvw_cfg1":
        return run_uvw_cfg1(args, rank, world, device)
    if args.workload == "interaction_l3":
        return run_interaction(args, rank, world, device)
    if args.workload == "conv_train_l3_23":
        return run_conv_train(args, rank, world, device)
    layout, nodes, degree = WORKLOADS[args.workload]
    if args.nodes > 0:
        nodes = args.nodes
    d = make_graph(layout, nodes, degree, rank, world, device)
    tp = d["tp"]
    node_x_full = torch.empty(nodes, tp.irreps_in1.dim, device=device) if world > 1 else d["node_x_local"]
    edges_total = nodes * degree

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        out = conv_step(d, node_x_full, world)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kernel_ms = []
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        out = conv_step(d, node_x_full, world)
    stop.record()
    barrier()
    ms_total = start.elapsed_time(stop)
    clocks = sampler.stop() if rank == 0 else None
    # dominant kernel alone (same launch, events directly around it), for the roofline
    for _ in range(max(3, min(args.steps, 10))):
        k0.record()
        out = conv_step(d, node_x_full, 1)
        k1.record()
        torch.cuda.synchronize()
        kernel_ms.append(k0.elapsed_time(k1))
    t = torch.tensor([ms_total], device=device)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms_step = t.item() / args.steps

    # ---- end to end from pinned host memory through the public API
    if args.skip_e2e:
        return finish(args, rank, world, d, tp, nodes, degree, edges_total, ms_step, kernel_ms, clocks, None)
    e2e_steps = max(1, min(args.steps, 3))
    host = {k: d[k].cpu().pin_memory() for k in ("node_x_local", "vec", "src", "rowptr", "w")}
    out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = out_host.numel() * out_host.element_size()

    def e2e_step():
        import e3nn_b200

        dev = {k: v.to(device, non_blocking=True) for k, v in host.items()}
        nx = dev["node_x_local"]
        if world > 1:
            torch.distributed.all_gather_into_tensor(node_x_full, nx)
            nx = node_x_full
        o = e3nn_b200.conv_uvu(tp, nx, dev["vec"], dev["src"], dev["rowptr"], dev["w"], scale=degree ** -0.5,
                               edge_attr_is_vector=True)
        out_host.copy_(o, non_blocking=True)

    del d["w"], d["vec"], d["src"]
    torch.cuda.empty_cache()
    e2e_step()
    barrier()
    t0 = time.perf_counter()
    start.record()
    for _ in range(e2e_steps):
        e2e_step()
    stop.record()
    barrier()
    t = torch.tensor([start.elapsed_time(stop)], device=device)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    e2e_ms = t.item() / e2e_steps

    e2e = {"value": edges_total / (e2e_ms * 1e-3), "unit": "edges/s", "h2d_bytes_per_step": h2d * world,
           "d2h_bytes_per_step": d2h * world, "steps": e2e_steps}
    return finish(args, rank, world, d, tp, nodes, degree, edges_total, ms_step, kernel_ms, clocks, e2e)


def finish(args, rank, world, d, tp, nodes, degree, edges_total, ms_step, kernel_ms, clocks, e2e):
    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        return
    peak, peak_kind = measured_peaks()
    kernel_ms.sort()
    k_ms = kernel_ms[len(kernel_ms) // 2]
    bytes_per_launch = algorithmic_bytes_per_edge(tp, nodes, edges_total) * d["e_local"]
    achieved = bytes_per_launch / (k_ms * 1e-3) / 1e9
    traffic = None
    line = {
        "metric": "TP edges/sec (fused SH + uvu + scatter, fp32)",
        "value": edges_total / (ms_step * 1e-3),
        "unit": "edges/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {
            "workload": args.workload, "layout": f"{tp.irreps_in1} x {tp.irreps_in2} -> {len(tp.instructions)} uvu paths",
            "nodes": nodes, "edges": edges_total, "in_degree": degree, "weight_numel": tp.weight_numel,
            "out_dim": tp.irreps_out.dim, "l2": "inputs (%.1f GB/step) far larger than the 126 MB L2" % (bytes_per_launch / 1e9),
            "parallelism": f"dst-range x{world}" + (" + allgather(node features)" if world > 1 else ""),
        },
        "roofline": {
            "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": traffic, "peak_kind": f"of {peak_kind}", "kernel": "conv_fwd_tma_kernel",
            "kernel_ms": k_ms, "algorithmic_bytes_per_edge": algorithmic_bytes_per_edge(tp, nodes, edges_total),
        },
        "e2e": e2e,
        "gpu_launches": args.steps * 1,
        "clocks": clocks,
    }
    if world == 1 and not args.skip_cpu:
        line["cpu_baseline"] = cpu_baseline(args.workload)
    print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


def run_sh(args, rank, world, device):
    from e3nn_b200 import o3

    n_total = 4_194_304
    n = n_total // world
    gen = torch.Generator(device=device).manual_seed(rank)
    vec = torch.randn(n, 3, device=device, generator=gen)
    sh = o3.SphericalHarmonics("0e+1o+2e+3o", True, "component")
    for _ in range(args.warmup):
        out = sh(vec)
    torch.cuda.synchronize()
    flush = torch.empty(64 * 1024 * 1024, device=device)  # 256 MB > L2
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(args.steps):
        flush.zero_()
        start.record()
        out = sh(vec)
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop))
    times.sort()
    ms = times[len(times) // 2]
    if rank != 0:
        return
    peak, peak_kind = measured_peaks()
    achieved = 76.0 * n / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "SH edges/sec (lmax 3, fp32)", "value": n_total / (ms * 1e-3), "unit": "edges/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "sh_l3", "edges": n_total, "l2": "256 MB buffer written between timed launches"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_kind": f"of {peak_kind}", "kernel": "sh_fwd_kernel<3>"},
        "gpu_launches": args.steps,
    }), flush=True)


def run_gate(args, rank, world, device):
    """Linear then Gate after an l <= 3 block: the Linear maps 64x0e+64x1o+64x2e+64x3o to the Gate's input
    (64 scalars (silu), 192 gates (sigmoid), 64x1o+64x2e+64x3o gated).  Reported: the Gate kernel alone (value,
    roofline), the Linear alone, the two in sequence, and the pair with the Gate as the Linear's epilogue."""
    from e3nn_b200 import nn as bnn
    from e3nn_b200 import o3

    rows_total = args.nodes if args.nodes > 0 else 1_048_576
    rows = rows_total // world
    gate = bnn.Gate("64x0e", [torch.nn.functional.silu], "192x0e", [torch.sigmoid], "64x1o+64x2e+64x3o").to(device)
    lin = o3.Linear("64x0e+64x1o+64x2e+64x3o", gate.irreps_in, math_mode="tf32x3").to(device)   # tensor cores, hi/lo-split tf32
    fused = bnn.LinearGate(lin, gate, fuse=True).to(device)
    gen = torch.Generator(device=device).manual_seed(rank)
    x = torch.randn(rows, gate.irreps_in.dim, device=device, generator=gen)
    h = torch.randn(rows, lin.irreps_in.dim, device=device, generator=gen)
    with torch.no_grad():
        for _ in range(args.warmup):
            out = gate(x)
            fused(h)
            gate(lin(h))
        torch.cuda.synchronize()
        ms = _median_launch_ms(lambda: gate(x), args.steps)
        ms_lin = _median_launch_ms(lambda: lin(h), args.steps)
        ms_two = _median_launch_ms(lambda: gate(lin(h)), args.steps)
        ms_fused = _median_launch_ms(lambda: fused(h), args.steps)
    if rank != 0:
        return
    peak, peak_kind = measured_peaks()
    nbytes = 4.0 * rows * (gate.irreps_in.dim + gate.irreps_out.dim)
    achieved = nbytes / (ms * 1e-3) / 1e9
    fused_bytes = 4.0 * rows * (lin.irreps_in.dim + gate.irreps_out.dim + 2 * fused.n_slots)
    two_bytes = 4.0 * rows * (lin.irreps_in.dim + 2 * gate.irreps_in.dim + gate.irreps_out.dim)
    print(json.dumps({
        "metric": "Gate rows/sec (l<=3, fp32)", "value": rows_total / (ms * 1e-3), "unit": "rows/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "gate", "rows": rows_total, "irreps_in": str(gate.irreps_in), "irreps_out": str(gate.irreps_out),
                   "l2": "rows in + out (%.1f GB) far larger than the 126 MB L2" % (nbytes / 1e9),
                   "linear_ms": ms_lin, "linear_then_gate_ms": ms_two, "linear_gate_fused_ms": ms_fused,
                   "linear_then_gate_bytes": two_bytes, "linear_gate_fused_bytes": fused_bytes,
                   "fused_hbm_frac": fused_bytes / (ms_fused * 1e-3) / 1e9 / peak},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_kind": f"of {peak_kind}", "kernel": "gate_fwd_kernel"},
        "gpu_launches": args.steps,
    }), flush=True)


# DRAM bytes per edge of conv_bwd_x_tma_kernel (layout l3_23), ncu capture of this workload (65,536 nodes x 32 edges)
NCU_CONV_BWD_X_L3_TRAFFIC_PER_EDGE = 13727


def run_conv_train(args, rank, world, device):
    """Fused convolution of a hidden layer in training: forward, then the gradients w.r.t. the per-edge weights,
    the edge vectors and the node features (layout l3_23, 65,536 nodes x 32 incoming edges; one GPU, or N
    independent replicas).  `roofline` is reported on the node-feature gradient kernel, timed alone."""
    import e3nn_b200
    from e3nn_b200 import _lib

    layout, nodes, degree = WORKLOADS["conv_l3_23"]
    if args.nodes > 0:
        nodes = args.nodes
    d = make_graph(layout, nodes, degree, 0, 1, device)
    tp, E = d["tp"], nodes * degree
    x = d["node_x_local"].requires_grad_(True)
    w = d["w"].requires_grad_(True)
    vec = d["vec"].requires_grad_(True)
    g = torch.randn(nodes, tp.irreps_out.dim, device=device)
    scale = degree ** -0.5

    def step():
        x.grad = w.grad = vec.grad = None
        out = e3nn_b200.conv_uvu(tp, x, vec, d["src"], d["rowptr"], w, scale=scale, edge_attr_is_vector=True)
        out.backward(g)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    torch.cuda.synchronize()
    t = torch.tensor([start.elapsed_time(stop)], device=device)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    # the node-feature gradient kernel alone, through the C ABI (the table is zeroed outside the events)
    x.grad = w.grad = vec.grad = None
    torch.cuda.empty_cache()
    mod = tp._uvu_module()
    gx = torch.empty(nodes, tp.irreps_in1.dim, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    P = _lib._ptr
    kernel_ms = []
    for _ in range(max(3, min(args.steps, 10))):
        gx.zero_()
        start.record()
        rc = mod.lib.e3b_conv_bwd_x(P(vec), 1, P(d["src"]), P(d["rowptr"]), None, P(w), P(g), P(gx), nodes, nodes, E, scale,
                                    P(status), _lib.stream_ptr())
        stop.record()
        torch.cuda.synchronize()
        if rc != 0 or int(status.item()) != 0:
            raise RuntimeError("conv_bwd_x failed: rc %d status %d" % (rc, int(status.item())))
        kernel_ms.append(start.elapsed_time(stop))
    if rank != 0:
        return
    kernel_ms.sort()
    k_ms = kernel_ms[len(kernel_ms) // 2]
    peak, peak_kind = measured_peaks()
    # per edge: the weight row, the vector, the source index, read + write of one gradient row; per node its cotangent
    per_edge = 4 * tp.weight_numel + 12 + 8 + 8 * tp.irreps_in1.dim + 4 * tp.irreps_out.dim / degree
    achieved = per_edge * E / (k_ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "TP edges/sec (fused SH + uvu + scatter, forward + all gradients, fp32)",
        "value": world * E / (ms_step * 1e-3), "unit": "edges/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "conv_train_l3_23", "nodes": nodes, "edges": E, "in_degree": degree,
                   "layout": f"{tp.irreps_in1} x {tp.irreps_in2} -> {len(tp.instructions)} uvu paths",
                   "parallelism": "replicas only" if world > 1 else "single GPU",
                   "l2": "per-edge weights (%.1f GB) far larger than the 126 MB L2" % (4e-9 * tp.weight_numel * E)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_CONV_BWD_X_L3_TRAFFIC_PER_EDGE * E, "peak_kind": f"of {peak_kind}",
                     "kernel": "conv_bwd_x_tma_kernel", "kernel_ms": k_ms, "algorithmic_bytes_per_edge": per_edge},
        "gpu_launches": args.steps * 3, "clocks": clocks,
    }), flush=True)


def measure_tf32_peak(device) -> float:
    """Dense tf32 matmul throughput of this GPU in TFLOP/s: torch.matmul on 8192^3 with tf32 allowed, best of 10
    (the burst figure, measured the way the bf16 figure of MEASURED_PEAKS.json was)."""
    n = 8192
    a = torch.randn(n, n, device=device)
    b = torch.randn(n, n, device=device)
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        for _ in range(3):
            a @ b
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = float("inf")
        for _ in range(10):
            start.record()
            a @ b
            stop.record()
            torch.cuda.synchronize()
            best = min(best, start.elapsed_time(stop))
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    return 2.0 * n ** 3 / (best * 1e-3) / 1e12


def _median_launch_ms(fn, launches: int, flush=None):
    """Median CUDA-event time of one launch of `fn` (events on the current stream directly around the call)."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ts = []
    for _ in range(launches):
        if flush is not None:
            flush.zero_()
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        ts.append(start.elapsed_time(stop))
    ts.sort()
    return ts[len(ts) // 2]


def secondary_workloads(device, tf32_peak: float):
    """The other configurations of the path, one compact record each, timed through the C ABI with outputs
    allocated beforehand: spherical harmonics of 4,194,304 vectors, the fused convolution on the 15- and 11-path
    l <= 2 layouts (65,536 nodes x 32 edges), the 1,048,576-row fully connected product + Linear, and the
    10,000-row product.  Inputs are far larger than L2 except where `l2` says otherwise."""
    from e3nn_b200 import _lib, layouts, o3

    peak, peak_kind = measured_peaks()
    P, core = _lib._ptr, _lib.core()
    out = []
    gen = torch.Generator(device=device).manual_seed(7)
    status = torch.zeros(1, dtype=torch.int32, device=device)

    # ---- spherical harmonics, lmax 3, normalize, 'component'
    n = 4_194_304
    vec = torch.randn(n, 3, device=device, generator=gen)
    y = torch.empty(n, 16, device=device)
    flush = torch.empty(64 * 1024 * 1024, device=device)   # 256 MB, written between launches

    def sh():
        rc = core.e3b_sh_fwd(P(vec), P(y), n, 3, 1, 0, _lib.stream_ptr())
        assert rc == 0
    for _ in range(3):
        sh()
    ms = _median_launch_ms(sh, 50, flush)
    out.append({"workload": "sh_l3", "metric": "SH edges/sec (lmax 3, fp32)", "value": n / (ms * 1e-3), "unit": "edges/s",
                "kernel": "sh_fwd_kernel<3>", "kernel_ms": ms, "launches": 50, "l2": "256 MB written between launches",
                "roofline": {"bound": "hbm", "achieved": 76.0 * n / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                             "frac": 76.0 * n / (ms * 1e-3) / 1e9 / peak, "peak_kind": f"of {peak_kind}"}})
    del vec, y

    # ---- fused convolution, l <= 2 layouts
    for name in ("conv_l2_15", "conv_l2_11"):
        layout, nodes, degree = WORKLOADS[name]
        d = make_graph(layout, nodes, degree, 0, 1, device)
        tp, E = d["tp"], nodes * degree
        mod = tp._uvu_module()
        res = torch.empty(nodes, tp.irreps_out.dim, device=device)

        def conv():
            rc = mod.lib.e3b_conv_fwd(P(d["node_x_local"]), P(d["vec"]), 1, P(d["src"]), P(d["rowptr"]), None, P(d["w"]),
                                      P(res), nodes, nodes, E, degree ** -0.5, P(status), _lib.stream_ptr())
            assert rc == 0
        for _ in range(3):
            conv()
        ms = _median_launch_ms(conv, 20)
        per_edge = algorithmic_bytes_per_edge(tp, nodes, E)
        out.append({"workload": name, "metric": "TP edges/sec (fused SH + uvu + scatter, fp32)", "value": E / (ms * 1e-3),
                    "unit": "edges/s", "kernel": "conv_fwd_tma_kernel", "kernel_ms": ms, "launches": 20,
                    "paths": len(tp.instructions), "l2": "per-edge weights (%.1f GB) far larger than L2" % (4e-9 * tp.weight_numel * E),
                    "roofline": {"bound": "hbm", "achieved": per_edge * E / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                                 "frac": per_edge * E / (ms * 1e-3) / 1e9 / peak, "peak_kind": f"of {peak_kind}",
                                 "algorithmic_bytes_per_edge": per_edge}})
        del d, res
    torch.cuda.empty_cache()

    # ---- fully connected product + Linear, 1,048,576 rows (tensor cores, plain tf32)
    rows = 1_048_576
    tp = o3.FullyConnectedTensorProduct("128x0e+64x1o+32x2e", "0e+1o+2e+3o", "128x0e+64x1o+32x2e", math_mode="tf32").to(device)
    lin = o3.Linear(tp.irreps_out, tp.irreps_out, math_mode="tf32").to(device)
    fused = o3.TensorProductLinear(tp, lin)      # the Linear folded into the product's weights: one product kernel
    with torch.no_grad():
        for view in tp.weight_views():
            view.div_((view.shape[0] * view.shape[1]) ** 0.5)
        x = torch.randn(rows, tp.irreps_in1.dim, device=device, generator=gen)
        y2 = torch.randn(rows, tp.irreps_in2.dim, device=device, generator=gen)
        for _ in range(3):
            lin(tp(x, y2))
            fused(x, y2)
        ms_tp = _median_launch_ms(lambda: tp(x, y2), 10)
        ms_two = _median_launch_ms(lambda: lin(tp(x, y2)), 10)
        ms_both = _median_launch_ms(lambda: fused(x, y2), 10)
    tf = 282_624.0 * rows / (ms_tp * 1e-3) / 1e12
    tf_both = (282_624.0 + 67_584.0) * rows / (ms_both * 1e-3) / 1e12
    out.append({"workload": "uvw_fctp", "metric": "uvw TP rows/sec (tf32 tensor cores) + Linear", "value": rows / (ms_both * 1e-3),
                "unit": "rows/s", "kernel": "uvw_post_kernel", "kernel_ms": ms_tp, "tp_plus_linear_ms": ms_both,
                "tp_then_linear_two_kernels_ms": ms_two, "launches": 10,
                "fusion": "Linear folded into the product's weights (W' = W_p L_o, 4.5 MFLOP per call), one product kernel",
                "roofline": {"bound": "tensor", "achieved": tf, "peak": tf32_peak, "unit": "TFLOP/s", "frac": tf / tf32_peak,
                             "peak_kind": "tf32 matmul measured in this run",
                             "tp_plus_linear_tflops_of_the_two_module_count": tf_both,
                             "tp_plus_linear_frac": tf_both / tf32_peak,
                             "hbm_frac_tp": 3904.0 * rows / (ms_tp * 1e-3) / 1e9 / peak,
                             "hbm_frac_tp_plus_linear": 3904.0 * rows / (ms_both * 1e-3) / 1e9 / peak}})
    del x, y2, tp, lin, fused
    torch.cuda.empty_cache()

    # ---- the 10,000-row product (23 MB of operands: a latency figure)
    tp = o3.FullyConnectedTensorProduct("32x0e+32x1o+32x2e", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e").to(device)
    with torch.no_grad():
        x = torch.randn(10_000, tp.irreps_in1.dim, device=device, generator=gen)
        y2 = torch.randn(10_000, tp.irreps_in2.dim, device=device, generator=gen)
        for _ in range(3):
            tp(x, y2)
        ms = _median_launch_ms(lambda: tp(x, y2), 50)
    out.append({"workload": "uvw_cfg1", "metric": "uvw TP rows/sec (10,000 rows, fp32)", "value": 10_000 / (ms * 1e-3),
                "unit": "rows/s", "kernel": "dense_fwd_kernel", "kernel_ms": ms, "launches": 50,
                "l2": "operands are L2 resident: launch latency, not bandwidth"})
    del x, y2, tp, flush
    torch.cuda.empty_cache()
    return out


def interaction_problem(n_atoms: int, seed: int = 0, device=None):
    """Positions and neighbour list of benchmark case 5 (interaction block) at `n_atoms` (host tensors, edges sorted by destination).

    With `device` the list is built by the device cell list (timed with a synchronisation on both sides, after
    one untimed call); without it by the host k-d tree (the CPU arms)."""
    from e3nn_b200 import nn as bnn

    box = (n_atoms / 0.05) ** (1.0 / 3.0)
    gen = torch.Generator().manual_seed(seed)
    pos = torch.rand(n_atoms, 3, generator=gen) * box
    if device is None:
        t0 = time.perf_counter()
        src, dst, shift = bnn.radius_graph_pbc(pos, box, 5.0)
        return box, pos, src, dst, shift, time.perf_counter() - t0
    pos_d = pos.to(device)
    bnn.neighbor_list_pbc(pos_d, box, 5.0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    src, dst, shift, _ = bnn.neighbor_list_pbc(pos_d, box, 5.0)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    return box, pos, src.cpu(), dst.cpu(), shift.cpu(), dt


# DRAM bytes per edge of conv_bwd_tma_kernel (layout l3_23) from an ncu capture of a 16,384-atom case
NCU_CONV_BWD_L3_TRAFFIC_PER_EDGE = 15718


def run_interaction(args, rank, world, device):
    """benchmark case 5 (interaction block): interaction block, forward + gradient w.r.t. positions.

    N GPUs: destination atoms are split into N contiguous ranges balanced by edge count; a rank owns the
    features of its atoms, all-gathers all source features every step (NCCL), evaluates its own output rows
    and its part of the loss; the position gradients of the ranks are summed with one all-reduce."""
    import e3nn_b200
    from e3nn_b200 import nn as bnn
    from e3nn_b200 import sharding

    n_atoms = args.nodes if args.nodes > 0 else 262_144
    secondary = tf32_peak = None
    if world == 1 and not args.skip_secondary:
        # the other configurations and the tf32 peak, measured before the large problem is resident
        tf32_peak = measure_tf32_peak(device)
        secondary = secondary_workloads(device, tf32_peak)
        torch.cuda.empty_cache()
    box, pos_host, src, dst, shift, t_graph = interaction_problem(n_atoms, device=device)
    E = src.numel()
    rowptr_host = torch.zeros(n_atoms + 1, dtype=torch.int64)
    rowptr_host[1:] = torch.cumsum(torch.bincount(dst, minlength=n_atoms), 0)
    bounds = sharding.partition_rows_by_edges(rowptr_host, world)
    n0, n1, e0, e1, rowptr_local = sharding.local_shard(rowptr_host, bounds, rank)
    torch.manual_seed(0)
    block = bnn.InteractionBlock("64x0e+64x1o+64x2e+64x3o", 3, num_basis=8, hidden=64, r_max=5.0,
                                 num_neighbors=E / n_atoms).to(device)
    for prm in block.parameters():
        prm.requires_grad_(False)
    gen = torch.Generator().manual_seed(1)
    node_x_host = torch.randn(n_atoms, 1024, generator=gen)
    G_host = torch.randn(n_atoms, 1024, generator=gen)
    x_local = node_x_host[n0:n1].to(device)
    G = G_host[n0:n1].to(device)
    # local edges: destinations re-based to the rank's rows, sources stay global (they index the gathered features)
    src_d, dst_glob, shift_d = src[e0:e1].to(device), dst[e0:e1].to(device), shift[e0:e1].to(device)
    rowptr = rowptr_local.to(device)
    pos_d = pos_host.to(device)
    x_full = torch.empty(n_atoms, 1024, device=device) if world > 1 else x_local
    tp = block.tp
    if world > 1:
        # the feature all-gather overlaps the radial layer: that layer's persistent kernel leaves the collective's SMs alone
        block.overlap_reserved_sms = sharding.OVERLAP_SMS

    def forward(p, xs, before_conv=None, phase_mark=None):
        # the block's own forward: global indices into the (replicated) positions and the gathered features,
        # the rank's local CSR -> the rank's output rows
        return block(p, xs, src_d, dst_glob, rowptr, shift_d, before_conv=before_conv, phase_mark=phase_mark)

    def step(p_in, phase_mark=None, keep=None):
        mark = phase_mark if phase_mark is not None else (lambda name: None)
        mark("start")
        wait = None
        if world > 1:
            # asynchronous: the transfer overlaps the edge embedding and the radial layers, which do not read features
            _, wait = sharding.all_gather_rows(x_local, bounds, out=x_full, async_op=True)
        p = p_in.detach().requires_grad_(True)
        out = forward(p, x_full, wait, phase_mark)
        loss = torch.dot(out.reshape(-1), G.reshape(-1))      # sum(out * G) without materialising the product
        mark("loss")
        loss.backward()
        mark("bwd_embed")
        if world > 1:
            torch.distributed.all_reduce(p.grad)
        mark("allreduce")
        if keep is not None:
            keep["out"] = out.detach()
        return p.grad

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        g = step(pos_d)
    barrier()
    sampler = ClockSampler(device.index or 0)
    if rank == 0:
        sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        g = step(pos_d)
    stop.record()
    barrier()
    t = torch.tensor([start.elapsed_time(stop)], device=device)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    clocks = sampler.stop() if rank == 0 else None

    # ---- what the step computed, reduced over the ranks (the same numbers at every N), and the phases of one step
    keep = {}
    marks = []

    def phase_mark(name):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        marks.append((name, ev))

    g = step(pos_d, phase_mark, keep)
    torch.cuda.synchronize()
    sums = torch.stack([keep["out"].double().pow(2).sum(), torch.tensor(float(keep["out"].numel()), device=device, dtype=torch.float64)])
    if world > 1:
        torch.distributed.all_reduce(sums)
    check = {"out_rms": (sums[0] / sums[1]).sqrt().item(), "dpos_rms": g.double().pow(2).mean().sqrt().item(),
             "dpos_abs_sum": g.double().abs().sum().item(), "dpos_sum": g.double().sum(0).abs().max().item()}
    phase_ms = {}
    for (_, e_prev), (name, e_now) in zip(marks, marks[1:]):
        phase_ms[name] = phase_ms.get(name, 0.0) + e_prev.elapsed_time(e_now)
    del keep, marks
    status_word = e3nn_b200.last_status_code()

    # ---- the same step with every contraction in strict fp32 (CUDA-core Linear, library fp32 GEMM for the radial
    # layer): the arithmetic mode whose error stays inside 1e-5 x RMS, reported beside the tensor-core default
    fp32_ms = None
    if world == 1 and not args.skip_secondary:
        block32 = bnn.InteractionBlock("64x0e+64x1o+64x2e+64x3o", 3, num_basis=8, hidden=64, r_max=5.0, num_neighbors=E / n_atoms,
                                       linear_math_mode="fp32", radial_math_mode="fp32").to(device)
        block32.load_state_dict(block.state_dict())
        for prm in block32.parameters():
            prm.requires_grad_(False)

        def step32():
            p = pos_d.detach().requires_grad_(True)
            torch.dot(block32(p, x_full, src_d, dst_glob, rowptr, shift_d).reshape(-1), G.reshape(-1)).backward()
            return p.grad

        step32()
        torch.cuda.synchronize()
        start.record()
        for _ in range(2):
            step32()
        stop.record()
        torch.cuda.synchronize()
        fp32_ms = start.elapsed_time(stop) / 2
        del block32
        torch.cuda.empty_cache()

    # ---- dominant kernel alone (conv_bwd) and the forward convolution, events directly around the launches
    mod = tp._uvu_module()
    with torch.no_grad():
        edge_vec = (pos_d[src_d] - pos_d[dst_glob] + shift_d).contiguous()
        w = block.edge_weights(edge_vec).contiguous()
    e_loc, n_loc = e1 - e0, n1 - n0
    gout = torch.randn(n_loc, tp.irreps_out.dim, device=device)
    gw, gvec = torch.empty_like(w), torch.empty_like(edge_vec)
    out_mid = torch.empty(n_loc, tp.irreps_out.dim, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    stream = torch.cuda.current_stream().cuda_stream
    scale = float(block.num_neighbors ** -0.5)

    def launch_bwd():
        rc = mod.lib.e3b_conv_bwd(x_full.data_ptr(), edge_vec.data_ptr(), 1, src_d.data_ptr(), rowptr.data_ptr(), None,
                                  w.data_ptr(), gout.data_ptr(), gw.data_ptr(), gvec.data_ptr(), n_loc, n_atoms, e_loc,
                                  scale, status.data_ptr(), stream)
        assert rc == 0

    def launch_fwd():
        rc = mod.lib.e3b_conv_fwd(x_full.data_ptr(), edge_vec.data_ptr(), 1, src_d.data_ptr(), rowptr.data_ptr(), None,
                                  w.data_ptr(), out_mid.data_ptr(), n_loc, n_atoms, e_loc, scale, status.data_ptr(), stream)
        assert rc == 0

    def median_ms(fn, n=5):
        ts = []
        for _ in range(n):
            start.record()
            fn()
            stop.record()
            torch.cuda.synchronize()
            ts.append(start.elapsed_time(stop))
        ts.sort()
        return ts[len(ts) // 2]

    launch_bwd(); launch_fwd()
    torch.cuda.synchronize()
    bwd_ms, fwd_ms = median_ms(launch_bwd), median_ms(launch_fwd)
    del gw, gvec, gout, out_mid, w
    torch.cuda.empty_cache()

    # ---- end to end: positions and features from pinned host memory, neighbour list built on the device from the
    # uploaded positions every step (as a simulation whose atoms move would), gradient back to the host.  The rank's
    # row and edge ranges are those of the set-up partition (the positions do not change between steps).
    e2e = None
    if not args.skip_e2e:
        host = {"pos": pos_host.pin_memory(), "x": node_x_host[n0:n1].contiguous().pin_memory()}
        grad_host = torch.empty(n_atoms, 3).pin_memory()

        copy_stream = torch.cuda.Stream(device=device)
        # two device buffers for the feature rows: the rows of step k + 1 are uploaded (copy engine, second stream)
        # while step k computes, as a loader that prefetches its next batch does; every step still uploads its
        # 1.07 GB from pinned host memory inside the timed region
        x_bufs = [torch.empty(n1 - n0, 1024, device=device) for _ in range(2)]
        x_ready = [None, None]
        state = {"k": 0}

        def enqueue_upload(i):
            copy_stream.wait_stream(torch.cuda.current_stream())     # the buffer's last reader (the step before) is done
            with torch.cuda.stream(copy_stream):
                x_bufs[i].copy_(host["x"], non_blocking=True)
                x_ready[i] = torch.cuda.Event()
                x_ready[i].record(copy_stream)

        enqueue_upload(0)

        def e2e_step():
            # the positions are needed first (neighbour list, edge embedding): main stream.  The feature rows (the bulk
            # of the bytes) are not read before the convolution; sharded, the all-gather of the rows that were uploaded
            # during the previous step runs on the second stream under the edge embedding and the radial layer
            k = state["k"]
            state["k"] = k + 1
            x_dev, uploaded = x_bufs[k % 2], x_ready[k % 2]
            pos_up = host["pos"].to(device, non_blocking=True)
            # every atom is binned, but only this rank's destination rows are walked: the list costs 1 / world of the full one
            s_loc, d_loc, sh_loc, rp_loc = bnn.neighbor_list_pbc(pos_up, box, 5.0, rows=(n0, n1))
            gather_wait = None
            xs = x_dev
            if world > 1:
                copy_stream.wait_stream(torch.cuda.current_stream())     # x_full's last reader (the step before) is done
                with torch.cuda.stream(copy_stream):
                    copy_stream.wait_event(uploaded)
                    _, gather_wait = sharding.all_gather_rows(x_dev, bounds, out=x_full, async_op=True)
                xs = x_full
            enqueue_upload((k + 1) % 2)          # next step's rows: into the buffer the previous step has finished with

            def wait():
                torch.cuda.current_stream().wait_event(uploaded)
                if gather_wait is not None:
                    gather_wait()

            p = pos_up.requires_grad_(True)
            torch.dot(block(p, xs, s_loc, d_loc, rp_loc, sh_loc, before_conv=wait).reshape(-1), G.reshape(-1)).backward()
            if world > 1:
                torch.distributed.all_reduce(p.grad)
            grad_host.copy_(p.grad, non_blocking=True)

        e2e_step()
        barrier()
        n_e2e = max(1, min(args.steps, 3))
        start.record()
        for _ in range(n_e2e):
            e2e_step()
        stop.record()
        barrier()
        t = torch.tensor([start.elapsed_time(stop)], device=device)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        e2e_ms = t.item() / n_e2e
        torch.cuda.synchronize()
        # the gradient that came back to the host against the one of the resident step (same positions and features)
        e2e_diff = ((grad_host.to(device) - g).abs().max() / g.abs().max()).item()
        e2e = {"value": E / (e2e_ms * 1e-3), "unit": "edges/s", "steps": n_e2e, "max_rel_diff_vs_resident_step": e2e_diff,
               "h2d_bytes_per_step": sum(v.numel() * v.element_size() for v in host.values()) * world,
               "d2h_bytes_per_step": grad_host.numel() * 4 * world}
    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        return
    peak, peak_kind = measured_peaks()
    wn, d1, dmid = tp.weight_numel, tp.irreps_in1.dim, tp.irreps_out.dim
    # algorithmic bytes of the two convolution kernels on this rank's shard
    bwd_bytes = e_loc * (2 * 4 * wn + 12 + 12 + 8) + n_loc * 4 * dmid + n_atoms * 4 * d1
    fwd_bytes = e_loc * (4 * wn + 12 + 8) + n_loc * 4 * dmid + n_atoms * 4 * d1
    achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9
    line = {
        "metric": "TP edges/sec (uvu l<=3, fp32): interaction block forward + gradient w.r.t. positions",
        "value": E / (ms_step * 1e-3), "unit": "edges/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32 (uvu, SH, scatter); tensor cores with hi/lo-split tf32 operands (Linear, 64->1472 radial layer)",
        "data": "synthetic",
        "config": {"workload": "interaction_l3", "atoms": n_atoms, "edges": E, "neighbours_per_atom": E / n_atoms,
                   "box": box, "cutoff": 5.0, "atoms_per_s": n_atoms / (ms_step * 1e-3),
                   "neighbour_list_s_device": t_graph, "weight_numel": wn, "mid_dim": dmid,
                   "conv_fwd_ms": fwd_ms, "conv_fwd_hbm_frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak,
                   "per_edge_weights": "materialised in HBM (%.1f GB per rank), radial network not fused yet" % (e_loc * wn * 4 / 1e9),
                   "l2": "per-edge weights and their gradient (2 x %.1f GB) far larger than the 126 MB L2" % (e_loc * wn * 4 / 1e9),
                   "parallelism": f"dst-range x{world}" + (" + allgather(node features) + allreduce(dpos)" if world > 1 else "")},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_CONV_BWD_L3_TRAFFIC_PER_EDGE * e_loc,
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch on 428,990 edges "
                                       "(15,718 B/edge), scaled by the edge count",
                     "peak_kind": f"of {peak_kind}", "kernel": "conv_bwd_tma_kernel", "kernel_ms": bwd_ms,
                     "algorithmic_bytes_per_launch": bwd_bytes},
        "e2e": e2e,
        "gpu_launches": args.steps * 12,
        "clocks": clocks,
        "check": check,
        "phase_ms": phase_ms,
        "kernel_status": status_word,
    }
    if clocks and clocks.get("sm_mhz"):
        line["ms_per_step_x_sm_ghz"] = ms_step * clocks["sm_mhz"] * 1e-3   # for comparing N against N at different clocks
    if fp32_ms is not None:
        line["fp32_mode_ms_per_step"] = fp32_ms     # Linear and radial layer in strict fp32 instead of hi/lo-split tf32
    if tf32_peak is not None:
        line["tf32_peak_tflops"] = tf32_peak
    if secondary is not None:
        line["secondary"] = secondary
    if world == 1 and not args.skip_cpu:
        line["cpu_baseline"] = cpu_interaction_baseline()
    print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


def import_reference():
    """The unmodified e3nn installed in ``baseline/_ref`` (by ``baseline/install_reference.py``, which
    ``__graft_entry__.build()`` runs where the sources exist), or None.  It travels to the GPU box with the repository."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not (os.path.isfile(os.path.join(ref, "e3nn", "__init__.py")) and os.path.isdir(os.path.join(ref, "opt_einsum_fx"))):
        return None
    if ref not in sys.path:
        sys.path.insert(0, ref)
    try:
        import e3nn
    except Exception:   # a dependency of the reference (sympy, scipy) is missing on this machine
        return None
    return e3nn


def _reference_dce(module):
    """Remove the dead outer-product nodes the reference's generated graph keeps when opt_einsum_fx is absent
    (that package would have removed them; outputs are bit-identical)."""
    gm = getattr(module, "_compiled_main_left_right", None)
    if gm is not None and hasattr(gm, "graph"):
        gm.graph.eliminate_dead_code()
        gm.recompile()
    return module


_REF_CACHE = {}


def reference_interaction_model():
    """The block of the default workload assembled from the reference's own modules (recipe of its ``Convolution``)."""
    if "interaction" in _REF_CACHE:
        return _REF_CACHE["interaction"]
    e3nn = import_reference()
    from e3nn import o3
    from e3nn.nn import FullyConnectedNet

    torch.manual_seed(0)
    node, sh = o3.Irreps("64x0e+64x1o+64x2e+64x3o"), o3.Irreps.spherical_harmonics(3)
    mid, ins = [], []
    for i, (mul, ir_in) in enumerate(node):
        for j, (_, ir_edge) in enumerate(sh):
            for ir_out in ir_in * ir_edge:
                if ir_out in node:
                    ins.append((i, j, len(mid), "uvu", True))
                    mid.append((mul, ir_out))
    mid, perm, _ = o3.Irreps(mid).sort()
    ins = [(a, b, perm[c], m, t) for a, b, c, m, t in ins]
    tp = _reference_dce(o3.TensorProduct(node, sh, mid, ins, internal_weights=False, shared_weights=False))
    fc = FullyConnectedNet([8, 64, tp.weight_numel], torch.nn.functional.silu)
    lin = o3.Linear(mid, node)
    for m in (fc, lin):
        for prm in m.parameters():
            prm.requires_grad_(False)
    _REF_CACHE["interaction"] = (e3nn, o3, sh, tp, fc, lin)
    return _REF_CACHE["interaction"]


def reference_interaction_sample(n_atoms: int, threads: int):
    """The reference itself (eager fp32, torch CPU, `threads` intra-op threads): forward + position gradient of the
    block on a smaller box of the same density.  Returns (edges, seconds)."""
    e3nn, o3, sh, tp, fc, lin = reference_interaction_model()
    from e3nn.math import bessel

    torch.set_num_threads(threads)
    box, pos, src, dst, shift, _ = interaction_problem(n_atoms, seed=3)
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(n_atoms, 1024, generator=gen)
    G = torch.randn(n_atoms, 1024, generator=gen)
    nn = src.numel() / n_atoms
    t0 = time.perf_counter()
    p = pos.clone().requires_grad_(True)
    vec = p[src] - p[dst] + shift
    w = fc(bessel(vec.norm(dim=1), 8, 5.0))
    msg = tp(x[src], o3.spherical_harmonics(sh, vec, True, "component"), w)
    mid = torch.zeros(n_atoms, msg.shape[1]).index_add_(0, dst, msg) / nn ** 0.5
    (lin(mid) * G).sum().backward()
    assert p.grad is not None
    return src.numel(), time.perf_counter() - t0


def cpu_interaction_sample(n_atoms: int, threads: int):
    """Oracle (fp32, torch CPU) forward + position gradient of the same block on a smaller box of the
    same density: returns (edges, seconds).  Only used when the reference is not installed."""
    from oracle import e3nn_oracle as orc

    torch.set_num_threads(threads)
    box, pos, src, dst, shift, _ = interaction_problem(n_atoms, seed=3)
    node, edge = "64x0e+64x1o+64x2e+64x3o", "0e+1o+2e+3o"
    mid, ins = orc.conv_uvu_layout(node, edge, [(0, 1), (1, -1), (2, 1), (3, -1)])
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(n_atoms, 1024, generator=gen)
    G = torch.randn(n_atoms, 1024, generator=gen)
    W0, W1 = torch.randn(8, 64, generator=gen), torch.randn(64, 1472, generator=gen)
    lw = torch.randn(sum(64 * 64 for _ in orc.linear_instructions(mid, node)), generator=gen)
    t0 = time.perf_counter()
    p = pos.clone().requires_grad_(True)
    out = orc.interaction_block(node, edge, mid, ins, node, p, x, src, dst, shift, [W0, W1], lw, 8, 5.0,
                                src.numel() / n_atoms, [0, 1, 2, 3], chunk=8192)
    (out * G).sum().backward()
    return src.numel(), time.perf_counter() - t0


def cpu_sample_atoms(t_warm: float) -> int:
    """Atoms of the CPU sample, the same rule in the `cpu_baseline` leg and in `--impl reference`: about 15 s of work
    per step judged from the 256-atom warm-up (`t_warm` seconds), between 512 and 2,048 atoms in steps of 256."""
    n = int(256 * 15.0 / max(t_warm, 1e-3)) // 256 * 256
    return max(512, min(2048, n))



def cpu_interaction_arm(steps: int, warmup: int):
    """(value edges/s, seconds per step, steps, cpu_baseline dict) of the CPU arm on the sample of `cpu_sample_atoms`."""
    threads = os.cpu_count() or 1
    ref = import_reference()
    fn, kind = (reference_interaction_sample, "reference") if ref is not None else (cpu_interaction_sample, "port")
    fn(256, threads)                         # first call: graph construction, allocator warm-up
    t_warm = fn(256, threads)[1]
    n_atoms = cpu_sample_atoms(t_warm)
    runs = [fn(n_atoms, threads) for _ in range(max(1, steps))]
    edges, t = runs[0][0], sum(r[1] for r in runs) / len(runs)
    what = ("e3nn 0.6.0 itself (eager fp32 torch-CPU, identity opt_einsum_fx stand-in, dead FX nodes removed)"
            if kind == "reference" else "fp32 torch-CPU oracle port (the reference is not installed in baseline/_ref)")
    base = {"value": edges / t, "unit": "edges/s", "cores": threads, "kind": kind,
            "sample": f"{n_atoms} atoms / {edges} edges at the same density, forward + position gradient, "
                      f"{what}, {t:.1f} s per step", "sample_atoms": n_atoms}
    return edges / t, t, len(runs), base


def cpu_interaction_baseline():
    return cpu_interaction_arm(steps=1, warmup=1)[3]


def run_uvw(args, rank, world, device):
    """benchmark case 4 (1,048,576-row fully connected product): rows are independent, so N GPUs run N replicas of rows/N each (no collective)."""
    from e3nn_b200 import o3

    rows_total = args.nodes if args.nodes > 0 else 1_048_576
    rows = rows_total // world
    tp = o3.FullyConnectedTensorProduct("128x0e+64x1o+32x2e", "0e+1o+2e+3o", "128x0e+64x1o+32x2e", math_mode="tf32").to(device)
    lin = o3.Linear(tp.irreps_out, tp.irreps_out, math_mode="tf32x3").to(device)
    fused = o3.TensorProductLinear(tp, lin)
    with torch.no_grad():
        for view in tp.weight_views():
            view.div_((view.shape[0] * view.shape[1]) ** 0.5)
    gen = torch.Generator(device=device).manual_seed(rank)
    x = torch.randn(rows, tp.irreps_in1.dim, device=device, generator=gen)
    y = torch.randn(rows, tp.irreps_in2.dim, device=device, generator=gen)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, n):
        ts = []
        for _ in range(n):
            start.record()
            r = fn()
            stop.record()
            torch.cuda.synchronize()
            ts.append(start.elapsed_time(stop))
        ts.sort()
        return ts[len(ts) // 2], r

    with torch.no_grad():
        for _ in range(args.warmup):
            out = lin(tp(x, y))
        torch.cuda.synchronize()
        ms_tp, mid = timed(lambda: tp(x, y), args.steps)
        ms_lin, out = timed(lambda: lin(mid), max(3, args.steps // 4))
        ms_two, out = timed(lambda: lin(tp(x, y)), args.steps)
        fused(x, y)
        ms_both, out = timed(lambda: fused(x, y), args.steps)
    if rank != 0:
        return
    peak, peak_kind = measured_peaks()
    flops_tp, flops_lin = 282_624.0, 67_584.0
    achieved_tf = flops_tp * rows / (ms_tp * 1e-3) / 1e12
    tf32_peak = measure_tf32_peak(device)        # torch.matmul with tf32 allowed, in this run, on this GPU
    print(json.dumps({
        "metric": "uvw TP rows/sec (tf32 tensor cores) + Linear", "value": rows_total / (ms_both * 1e-3), "unit": "rows/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_both, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "tf32 operands, f32 accumulate (TP); hi/lo-split tf32 operands (Linear)", "data": "synthetic",
        "config": {"workload": "uvw_fctp", "rows": rows_total, "tp_ms": ms_tp, "linear_ms": ms_lin, "tp_then_linear_ms": ms_two,
                   "tp_plus_linear_fused_ms": ms_both,
                   "l2": "inputs and outputs (4.1 GB) far larger than the 126 MB L2", "parallelism": f"replicas x{world}"},
        "roofline": {"bound": "tensor", "achieved": achieved_tf, "peak": tf32_peak, "unit": "TFLOP/s",
                     "frac": achieved_tf / tf32_peak, "traffic": None, "kernel": "uvw_post_kernel",
                     "peak_kind": "tf32 matmul (8192^3) measured in this run",
                     "hbm_achieved_gbs": 3904.0 * rows / (ms_tp * 1e-3) / 1e9, "hbm_peak_gbs": peak,
                     "hbm_frac": 3904.0 * rows / (ms_tp * 1e-3) / 1e9 / peak},
        "gpu_launches": args.steps * 4,
    }), flush=True)


def run_uvw_cfg1(args, rank, world, device):
    """benchmark case 1 (10,000-row fully connected product) (the reference's own CPU-runnable case): 10,000 rows of a 32-channel l <= 2 fully connected
    product.  23 MB of data and 0.7 GFLOP: the call is bound by launch latency, so the line reports the time of one
    call per arithmetic mode, and of a CUDA-graph replay of the fp32 call."""
    from e3nn_b200 import o3

    layout = ("32x0e+32x1o+32x2e", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e")
    rows = args.nodes if args.nodes > 0 else 10_000
    gen = torch.Generator(device=device).manual_seed(rank)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = {}
    with torch.no_grad():
        base = o3.FullyConnectedTensorProduct(*layout).to(device)
        x = torch.randn(rows, base.irreps_in1.dim, device=device, generator=gen)
        y = torch.randn(rows, base.irreps_in2.dim, device=device, generator=gen)
        for mode in ("fp32", "tf32x3", "tf32"):
            tp = o3.FullyConnectedTensorProduct(*layout, math_mode=mode).to(device)
            tp.load_state_dict(base.state_dict())
            for _ in range(max(3, args.warmup)):
                tp(x, y)
            torch.cuda.synchronize()
            ts = []
            for _ in range(max(20, args.steps)):
                start.record()
                tp(x, y)
                stop.record()
                torch.cuda.synchronize()
                ts.append(start.elapsed_time(stop))
            ts.sort()
            times[mode] = ts[len(ts) // 2]
        # the fp32 call captured in a CUDA graph (what a caller with a fixed batch would replay)
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            base(x, y)
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(graph):
            out = base(x, y)
        graph.replay()
        torch.cuda.synchronize()
        n = 50
        start.record()
        for _ in range(n):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        times["fp32_graph_replay"] = start.elapsed_time(stop) / n
    if rank != 0:
        return
    peak, peak_kind = measured_peaks()
    ms = times["fp32"]
    nbytes = 4.0 * rows * (base.irreps_in1.dim + base.irreps_in2.dim + base.irreps_out.dim)
    print(json.dumps({
        "metric": "uvw TP rows/sec (config 1, fp32)", "value": world * rows / (ms * 1e-3), "unit": "rows/s", "n_gpus": world,
        "steps": max(20, args.steps), "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "uvw_cfg1", "rows": rows, "ms_per_call": times, "parallelism": f"replicas x{world}",
                   "l2": "23 MB of operands, L2 resident: a latency measurement, not a bandwidth one"},
        "roofline": {"bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": nbytes / (ms * 1e-3) / 1e9 / peak, "traffic": None, "peak_kind": f"of {peak_kind}",
                     "kernel": "dense_fwd_kernel", "note": "launch bound (3 launches, one per output irrep)"},
        "gpu_launches": max(20, args.steps) * 3,
    }), flush=True)


# ------------------------------------------------------------------------------------------- CPU arm
def cpu_conv_sample(workload: str, sample_edges: int, threads: int):
    """One pass of the oracle over a sample of the workload: returns seconds."""
    from oracle import e3nn_oracle as orc

    layout, nodes, degree = WORKLOADS[workload]
    from e3nn_b200 import layouts

    node, edge, keep = layouts.BENCH_CONV_LAYOUTS[layout]
    keep_lp = [(l, p) for _, l, p in orc.parse_irreps(keep)]
    mid, ins = orc.conv_uvu_layout(node, edge, keep_lp)
    lmax = max(l for _, l, _ in orc.parse_irreps(edge))
    torch.set_num_threads(threads)
    gen = torch.Generator().manual_seed(0)
    n_dst = sample_edges // degree
    node_x = torch.randn(nodes, orc.irreps_dim(orc.parse_irreps(node)), generator=gen)
    vec = torch.randn(sample_edges, 3, generator=gen)
    src = torch.randint(0, nodes, (sample_edges,), generator=gen)
    dst = torch.arange(sample_edges) // degree
    wn = sum(m for m, _, _ in orc.parse_irreps(mid))
    w = torch.randn(sample_edges, wn, generator=gen)
    t0 = time.perf_counter()
    orc.conv_uvu(node, edge, mid, ins, node_x, vec, src, dst, w, n_dst, list(range(lmax + 1)), scale=degree ** -0.5,
                 chunk=16384)
    return time.perf_counter() - t0


def reference_conv_sample(workload: str, sample_edges: int, threads: int):
    """The reference itself on a sample of a fused-convolution workload: gather, spherical harmonics, its
    ``TensorProduct`` ('uvu', per-edge weights) and the scatter sum, in chunks of 16,384 edges.  Returns seconds."""
    layout, nodes, degree = WORKLOADS[workload]
    key = "conv_" + layout
    if key not in _REF_CACHE:
        import_reference()
        from e3nn import o3
        from e3nn_b200 import layouts

        node, edge, keep = layouts.BENCH_CONV_LAYOUTS[layout]
        node, edge, keep = o3.Irreps(node), o3.Irreps(edge), o3.Irreps(keep)
        mid, ins = [], []
        for i, (mul, ir_in) in enumerate(node):
            for j, (_, ir_edge) in enumerate(edge):
                for ir_out in ir_in * ir_edge:
                    if ir_out in keep or ir_out == o3.Irrep(0, 1):
                        ins.append((i, j, len(mid), "uvu", True))
                        mid.append((mul, ir_out))
        mid, perm, _ = o3.Irreps(mid).sort()
        ins = [(a, b, perm[c], m, t) for a, b, c, m, t in ins]
        tp = _reference_dce(o3.TensorProduct(node, edge, mid, ins, internal_weights=False, shared_weights=False))
        _REF_CACHE[key] = (o3, node, edge, tp)
    o3, node, edge, tp = _REF_CACHE[key]
    torch.set_num_threads(threads)
    gen = torch.Generator().manual_seed(0)
    n_dst = sample_edges // degree
    node_x = torch.randn(nodes, node.dim, generator=gen)
    vec = torch.randn(sample_edges, 3, generator=gen)
    src = torch.randint(0, nodes, (sample_edges,), generator=gen)
    dst = torch.arange(sample_edges) // degree
    w = torch.randn(sample_edges, tp.weight_numel, generator=gen)
    t0 = time.perf_counter()
    out = torch.zeros(n_dst, tp.irreps_out.dim)
    with torch.no_grad():
        for c0 in range(0, sample_edges, 16384):
            c1 = min(c0 + 16384, sample_edges)
            y = o3.spherical_harmonics(edge, vec[c0:c1], True, "component")
            out.index_add_(0, dst[c0:c1], tp(node_x[src[c0:c1]], y, w[c0:c1]))
        out *= degree ** -0.5
    return time.perf_counter() - t0


CPU_SAMPLE_EDGES = 262144


def cpu_conv_arm(workload: str, steps: int, warmup: int):
    threads = os.cpu_count() or 1
    fn, kind = (reference_conv_sample, "reference") if import_reference() is not None else (cpu_conv_sample, "port")
    for _ in range(warmup):
        fn(workload, 16384, threads)
    times = [fn(workload, CPU_SAMPLE_EDGES, threads) for _ in range(max(1, steps))]
    t = sum(times) / len(times)
    what = ("e3nn 0.6.0 itself (eager fp32 torch-CPU, identity opt_einsum_fx stand-in, dead FX nodes removed)"
            if kind == "reference" else "fp32 torch-CPU oracle port (the reference is not installed in baseline/_ref)")
    base = {"value": CPU_SAMPLE_EDGES / t, "unit": "edges/s", "cores": threads, "kind": kind,
            "sample": f"{CPU_SAMPLE_EDGES} edges of the same graph in chunks of 16384, {what}, {t:.1f} s per step"}
    return CPU_SAMPLE_EDGES / t, t, len(times), base


def cpu_baseline(workload: str):
    return cpu_conv_arm(workload, steps=1, warmup=1)[3]


def run_reference(args):
    """CPU arm: the reference's own implementation of the workload on the host cores, a bounded sample per step.
    Under torchrun only rank 0 works."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 3)), min(args.warmup, 1)
    if args.workload == "interaction_l3":
        value, t, steps, base = cpu_interaction_arm(steps, warmup)
        metric = "TP edges/sec (uvu l<=3, fp32): interaction block forward + gradient w.r.t. positions"
        config = {"workload": "interaction_l3", "atoms": 262144, "cutoff": 5.0, "sample_atoms": base["sample_atoms"]}
    else:
        workload = args.workload if args.workload in WORKLOADS else "conv_l2_15"
        layout, nodes, degree = WORKLOADS[workload]
        value, t, steps, base = cpu_conv_arm(workload, steps, warmup)
        metric = "TP edges/sec (fused SH + uvu + scatter, fp32)"
        config = {"workload": workload, "nodes": nodes, "edges": nodes * degree, "in_degree": degree,
                  "sample_edges": CPU_SAMPLE_EDGES}
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": value, "unit": "edges/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + ["sh_l3", "uvw_fctp", "interaction_l3", "gate", "conv_train_l3_23", "uvw_cfg1"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--nodes", type=int, default=0, help="override the node count (smaller graphs for profiling)")
    ap.add_argument("--skip-e2e", action="store_true", help="profiling runs: skip the host-buffer leg")
    ap.add_argument("--skip-cpu", action="store_true", help="profiling runs: skip the CPU baseline leg")
    ap.add_argument("--skip-secondary", action="store_true", help="profiling runs: skip the list of the other configurations")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
