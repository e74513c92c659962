"""Generator of the bulk-copy (TMA) pipelined version of the fused convolution kernel.

Same arithmetic as ``conv_fwd_kernel`` of ``uvu.py``, restructured for the two ceilings that kernel
hits on B200 (issue slots and exposed global-load latency):

* **one warp per edge, two channels per lane** (u = lane and lane + 32): all per-channel arithmetic
  is issued as packed ``FFMA2`` (``__ffma2_rn`` on ``float2``), halving the issue slots per edge;
* **asynchronous staging**: the per-edge weight row and the gathered source-feature row are brought
  into a shared-memory ring by ``cp.async.bulk`` (1-D TMA) copies that one lane of the team issues
  ``depth - 1`` edges ahead; completion is tracked by mbarriers (``complete_tx``), consumers read
  shared memory only.  A *team* of ``T`` warps shares a ring when the accumulators of all paths do
  not fit the registers of one warp; each warp of the team then owns a subset of the paths;
* **persistent teams** own contiguous destination ranges balanced by edge count, keep the
  accumulators of the current destination row in registers and write every output row once.

Eligibility: every live path has 64 channels, one multiplicity in x2 and a weight; irreps_in2 is
Y^0..Y^L (harmonics evaluated in the kernel); weight and feature rows are multiples of 16 bytes.
Every mbarrier wait is bounded; a wait that gives up raises the status word and the warp returns.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np

from ..o3._wigner import wigner_3j_numpy

SMEM_BUDGET = 200 * 1024
ACC_FLOATS_PER_WARP = 112   # accumulator registers (2 per output component) one warp may hold


def _f(v: float) -> str:
    return f"{np.float32(v):.9e}f"


def eligible(layout) -> bool:
    if layout.sh_lmax() is None or not layout.paths:
        return False
    if layout.d1 % 4 != 0 or layout.wn % 4 != 0 or layout.wn == 0:
        return False
    for p in layout.paths:
        if p.mul1 != 64 or p.mul2 != 1 or p.woff < 0:
            return False
    # every output slot written by exactly the channels of one path group; slots may take several paths
    return True


def _path_cost(p) -> int:
    c = wigner_3j_numpy(p.l1, p.l2, p.l3)
    nnz = int((c != 0).sum())
    pairs = int((np.abs(c).sum(axis=1) != 0).sum())
    return nnz + 2 * pairs + 2 * (2 * p.l3 + 1)


def split_paths(layout) -> List[List]:
    """Partition of the paths over the warps of a team (balanced by arithmetic cost)."""
    total_acc = 2 * sum(layout.spec.irreps_out[io].ir.dim for io in layout.out_used)
    T = max(1, -(-total_acc // ACC_FLOATS_PER_WARP))
    if T == 1:
        return [list(layout.paths)]
    # output slots (not paths) are the unit: a slot's accumulators live in one warp
    slots: Dict[int, List] = {}
    for p in layout.paths:
        slots.setdefault(p.io, []).append(p)
    items = sorted(slots.values(), key=lambda ps: -sum(_path_cost(p) for p in ps))
    groups: List[List] = [[] for _ in range(T)]
    load = [0] * T
    for ps in items:
        g = load.index(min(load))
        groups[g] += ps
        load[g] += sum(_path_cost(p) for p in ps)
    for g in groups:
        g.sort(key=lambda p: p.index)
    return groups


def _body(layout, paths, folded: bool) -> Tuple[List[str], str, str]:
    """(accumulator declarations, per-edge body, output stores) for one warp of a team.

    ``folded``: out_k += C_ijk ((x_i w) Y_j) with the constants in the multiply-adds (fewest instructions, the
    choice when the paths are split over a team); otherwise the coupling table t_ik = sum_j C_ijk Y_j is
    built per edge first (measured faster when one warp holds every path)."""
    spec = layout.spec
    o1 = spec.irreps_in1.offsets()
    oo = spec.irreps_out.offsets()
    decl, body, store = [], [], []
    slots = sorted({p.io for p in paths})
    acc: Dict[Tuple[int, int], str] = {}
    for io in slots:
        dim = spec.irreps_out[io].ir.dim
        for k in range(dim):
            a = acc[(io, k)] = f"A{len(acc)}"      # registers are shared by the roles: role-local numbering
            decl.append(a)
            store.append(f"orow[{oo[io]} + lane * {dim} + {k}] = {a}.x * scale; "
                         f"orow[{oo[io]} + (lane + 32) * {dim} + {k}] = {a}.y * scale; "
                         f"{a} = make_float2(0.0f, 0.0f);")
    for i1 in sorted({p.i1 for p in paths}):
        d = spec.irreps_in1[i1].ir.dim
        for i in range(d):
            body.append(f"const float2 X{i1}_{i} = make_float2(sx[{o1[i1]} + lane * {d} + {i}], sx[{o1[i1]} + (lane + 32) * {d} + {i}]);")
    if folded:
        for j in range(layout.d2):
            body.append(f"const float2 YY{j} = make_float2(Y[{j}], Y[{j}]);")
        for p in paths:
            # out_k += C_ijk * ((x_i w) Y_j): constants folded into the multiply-add, no per-edge coupling table
            c = wigner_3j_numpy(p.l1, p.l2, p.l3) * p.pw
            body.append(f"{{ // path {p.index}: l={p.l1} (x) l={p.l2} -> l={p.l3}")
            body.append(f"  const float2 Wp = make_float2(sw[{p.woff} + lane], sw[{p.woff} + lane + 32]);")
            for i in range(2 * p.l1 + 1):
                if not (c[i] != 0.0).any():
                    continue
                body.append(f"  {{ const float2 XW = __fmul2_rn(X{p.i1}_{i}, Wp);")
                for j in range(2 * p.l2 + 1):
                    ks = [(k, c[i, j, k]) for k in range(2 * p.l3 + 1) if c[i, j, k] != 0.0]
                    if not ks:
                        continue
                    body.append(f"    {{ const float2 P = __fmul2_rn(XW, YY{p.off2 + j});")
                    for k, v in ks:
                        body.append(f"      {acc[(p.io, k)]} = __ffma2_rn(make_float2({_f(v)}, {_f(v)}), P, {acc[(p.io, k)]});")
                    body.append("    }")
                body.append("  }")
            body.append("}")
    else:
        for p in paths:
            c = wigner_3j_numpy(p.l1, p.l2, p.l3) * p.pw
            body.append(f"{{ // path {p.index}: l={p.l1} (x) l={p.l2} -> l={p.l3}")
            names = {}
            for i in range(2 * p.l1 + 1):
                for k in range(2 * p.l3 + 1):
                    terms = [(j, c[i, j, k]) for j in range(2 * p.l2 + 1) if c[i, j, k] != 0.0]
                    if not terms:
                        continue
                    expr = " + ".join(f"{_f(v)} * Y[{p.off2 + j}]" for j, v in terms)
                    body.append(f"  const float t{i}_{k} = {expr}; const float2 T{i}_{k} = make_float2(t{i}_{k}, t{i}_{k});")
                    names[(i, k)] = f"T{i}_{k}"
            body.append(f"  const float2 Wp = make_float2(sw[{p.woff} + lane], sw[{p.woff} + lane + 32]);")
            for k in range(2 * p.l3 + 1):
                terms = [(names[(i, k)], f"X{p.i1}_{i}") for i in range(2 * p.l1 + 1) if (i, k) in names]
                if not terms:
                    continue
                expr = f"__fmul2_rn({terms[0][0]}, {terms[0][1]})"
                for t, x in terms[1:]:
                    expr = f"__ffma2_rn({t}, {x}, {expr})"
                body.append(f"  {acc[(p.io, k)]} = __ffma2_rn(Wp, {expr}, {acc[(p.io, k)]});")
            body.append("}")
    return decl, "\n".join(body), "\n".join(store)


def _indent(text: str, n: int) -> str:
    pad = " " * n
    return "\n".join(pad + line if line else line for line in text.split("\n"))


def emit(layout, depth: int = 0, max_warps: int = 16) -> Optional[Dict[str, str]]:
    """Kernel source and launch code for an eligible layout (None otherwise)."""
    if not eligible(layout):
        return None
    spec = layout.spec
    groups = split_paths(layout)
    T = len(groups)
    stage_w, stage_x = layout.wn * 4, layout.d1 * 4
    stage = (stage_w + stage_x + 127) // 128 * 128
    def teams_for(d: int) -> int:
        return max(1, min(SMEM_BUDGET // (d * stage + 32 * 20 * 4), max_warps // T, 8))

    if depth == 0:
        # four stages in flight unless three let one more team (more warps to issue from) fit in shared memory
        depth = 3 if teams_for(3) > teams_for(4) else 4
    teams = teams_for(depth)
    lmax = layout.sh_lmax()
    # outputs nobody writes (possible in hand-written layouts): zero-filled by warp 0 of the team
    zero_ranges = []
    for io, (mul, ir) in enumerate(spec.irreps_out):
        if io not in layout.out_used and mul * ir.dim > 0:
            zero_ranges.append((spec.irreps_out.offsets()[io], mul * ir.dim))
    zero_code = "\n".join(f"for (int c = lane; c < {n}; c += 32) orow[{off} + c] = 0.0f;" for off, n in zero_ranges)

    parts = [_body(layout, paths, folded=T > 1) for paths in groups]
    n_acc = max(len(p[0]) for p in parts)
    decl = "\n".join(f"float2 A{i} = make_float2(0.0f, 0.0f);" for i in range(n_acc))

    def switch(texts: List[str], pad: int) -> str:
        if T == 1:
            return _indent(texts[0], pad)
        lines = ["switch (tw) {"]
        for tw, text in enumerate(texts):
            lines.append(f"case {tw}: {{")
            lines.append(_indent(text, 4))
            lines.append("} break;")
        lines.append("default: break;")
        lines.append("}")
        return _indent("\n".join(lines), pad)

    stores = [p[2] + ("\n" + zero_code if tw == 0 and zero_code else "") for tw, p in enumerate(parts)]
    kernel = f"""
// ================================================================= bulk-copy pipelined fused convolution
constexpr int kV2T = {T};                 // warps per team (each owns a subset of the paths)
constexpr int kV2Teams = {teams};         // teams per CTA
constexpr int kV2Threads = kV2T * kV2Teams * 32;
constexpr int kV2Depth = {depth};         // ring stages (edges in flight) per team
constexpr int kV2StageW = {stage_w};      // bytes: one edge's weight row
constexpr int kV2StageX = {stage_x};      // bytes: one gathered source-feature row
constexpr int kV2StageBytes = {stage};
constexpr int kV2RingBytes = kV2Depth * kV2StageBytes;
constexpr int kV2YStride = 20;            // floats per edge of the harmonics batch (16-byte aligned rows)
constexpr int kV2SmemBytes = kV2Teams * kV2RingBytes + kV2Teams * 2 * kV2Depth * 8 + 128 + kV2Teams * 32 * kV2YStride * 4;

__device__ __forceinline__ void v2_issue(uint8_t* stage, uint64_t* bar, const float* wrow, const float* xrow) {{
    const uint32_t b = tc::smem_u32(bar);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(kV2StageW + kV2StageX) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(tc::smem_u32(stage)), "l"(wrow), "r"(kV2StageW), "r"(b) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(tc::smem_u32(stage + kV2StageW)), "l"(xrow), "r"(kV2StageX), "r"(b) : "memory");
}}

// barrier of the T warps of one team (hardware barrier 1 + team; every lane of every warp of the team calls it)
template <int T>
__device__ __forceinline__ void v2_team_sync(int team) {{
    if (T == 1) __syncwarp();
    else asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(T * 32) : "memory");
}}

// One lane per edge: harmonics of a batch of <= 32 consecutive edges into shared memory.
__device__ __forceinline__ void v2_batch_harmonics(const float* __restrict__ vec, int64_t e0, int64_t e_hi, float* ybuf, int lane) {{
    const int64_t ee = e0 + lane;
    if (ee < e_hi) {{
        const float vx = vec[ee * 3], vy = vec[ee * 3 + 1], vz = vec[ee * 3 + 2];
        const float inv = 1.0f / fmaxf(sqrtf(vx * vx + vy * vy + vz * vz), 1e-12f);
        float Y[kD2];
        e3b_sh_fwd<kShLmax>(vx * inv, vy * inv, vz * inv, Y);
#pragma unroll
        for (int j = 0; j < kD2; ++j) ybuf[lane * kV2YStride + j] = Y[j];
    }}
}}

// smallest n in [0, num_nodes] with rowptr[n] >= target
__device__ __forceinline__ int64_t v2_lower_bound(const int64_t* __restrict__ rowptr, int64_t num_nodes, int64_t target) {{
    int64_t lo = 0, hi = num_nodes;
    while (lo < hi) {{
        const int64_t mid = (lo + hi) >> 1;
        if (rowptr[mid] < target) lo = mid + 1; else hi = mid;
    }}
    return lo;
}}

// The warps of a team run one copy of the loop code and differ only in the two switch statements (per-path
// arithmetic, stores of their output slots): the hot code stays inside the SM's instruction cache.
__global__ void __launch_bounds__(kV2Threads, 1) conv_fwd_tma_kernel(const float* __restrict__ node_x, const float* __restrict__ vec,
        const int64_t* __restrict__ edge_src, const int64_t* __restrict__ rowptr, const float* __restrict__ w,
        float* __restrict__ out, int64_t num_nodes, int64_t num_src, int64_t num_edges, float scale, int* __restrict__ status) {{
    extern __shared__ __align__(128) uint8_t v2_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int team = warp / kV2T, tw = warp % kV2T;
    uint8_t* ring = v2_smem + team * kV2RingBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(v2_smem + kV2Teams * kV2RingBytes);
    uint64_t* full = bars + team * 2 * kV2Depth;
    uint64_t* empty = full + kV2Depth;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kV2Teams * 2 * kV2Depth);
    float* ybuf = reinterpret_cast<float*>(v2_smem + kV2Teams * kV2RingBytes + kV2Teams * 2 * kV2Depth * 8 + 128) + team * 32 * kV2YStride;
    if (threadIdx.x == 0) *abort_flag = 0;
    if (tw == 0 && lane == 0) {{
        for (int s = 0; s < kV2Depth; ++s) {{ tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], kV2T); }}
        tc::mbar_init_fence();
    }}
    __syncthreads();
    // contiguous destination range of this team, balanced by edge count
    const int64_t team_id = static_cast<int64_t>(blockIdx.x) * kV2Teams + team;
    const int64_t num_teams = static_cast<int64_t>(gridDim.x) * kV2Teams;
    const int64_t n_lo = team_id == 0 ? 0 : v2_lower_bound(rowptr, num_nodes, (num_edges * team_id) / num_teams);
    const int64_t n_hi = team_id + 1 == num_teams ? num_nodes : v2_lower_bound(rowptr, num_nodes, (num_edges * (team_id + 1)) / num_teams);
    if (n_lo >= n_hi) return;
    const bool leader = tw == 0 && lane == 0;
    int64_t e = rowptr[n_lo];
    const int64_t e_hi = rowptr[n_hi];
    int64_t issue = e;          // next edge to stage (leader lane only)
    int64_t src_pref = 0;
    bool ok = true;
    if (leader) {{
        for (int s = 0; s < kV2Depth && issue < e_hi; ++s, ++issue) {{
            int64_t sidx = edge_src[issue];
            if (sidx < 0 || sidx >= num_src) {{ atomicExch(status, 2); sidx = 0; }}
            v2_issue(ring + s * kV2StageBytes, &full[s], w + issue * kWn, node_x + sidx * kD1);
        }}
        if (issue < e_hi) src_pref = edge_src[issue];
    }}
{_indent(decl, 4)}
    uint32_t it = 0;
    int64_t seg_end = rowptr[n_lo + 1];
    for (int64_t n = n_lo; n < n_hi; ++n) {{
        const int64_t e_end = seg_end;
        if (n + 2 <= n_hi) seg_end = rowptr[n + 2];   // next row's end, fetched one row ahead
        for (; e < e_end; ++e, ++it) {{
            const int slot = static_cast<int>(it & 31u);
            if (slot == 0) {{
                // batch boundary: the harmonics are per-edge scalar work, evaluated one lane per edge
                __syncwarp();
                v2_team_sync<kV2T>(team);
                if (tw == 0) v2_batch_harmonics(vec, e, e_hi, ybuf, lane);
                __syncwarp();
                v2_team_sync<kV2T>(team);
            }}
            if (!ok) continue;      // a wait gave up: keep the loop (and the team barriers) going without work
            const int s = it % kV2Depth;
            const uint32_t ph = (it / kV2Depth) & 1u;
            ok = __all_sync(0xffffffffu, tc::mbar_wait(&full[s], ph, abort_flag));
            if (!ok) continue;
            const float* sw = reinterpret_cast<const float*>(ring + s * kV2StageBytes);
            const float* sx = reinterpret_cast<const float*>(ring + s * kV2StageBytes + kV2StageW);
            float Y[kD2];
#pragma unroll
            for (int j = 0; j < kD2; ++j) Y[j] = ybuf[slot * kV2YStride + j];
{switch([p[1] for p in parts], 12)}
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&empty[s]);
            if (leader && it > 0 && issue < e_hi) {{
                // refill the stage released one iteration ago (the other warps of the team had an edge of slack)
                const int sp = (it - 1) % kV2Depth;
                const uint32_t php = ((it - 1) / kV2Depth) & 1u;
                if (tc::mbar_wait(&empty[sp], php, abort_flag)) {{
                    int64_t sidx = src_pref;
                    if (sidx < 0 || sidx >= num_src) {{ atomicExch(status, 2); sidx = 0; }}
                    tc::fence_proxy_async_smem();
                    v2_issue(ring + sp * kV2StageBytes, &full[sp], w + issue * kWn, node_x + sidx * kD1);
                    ++issue;
                    if (issue < e_hi) src_pref = edge_src[issue];
                }}
            }}
        }}
        if (ok) {{
            float* orow = out + n * kDout;
{switch(stores, 12)}
        }}
    }}
    if (!ok) {{
        if (lane == 0) atomicExch(status, 3);
        // give copies that are still in flight time to land before this warp's shared memory can go away
        for (int q = 0; q < 2000; ++q) __nanosleep(500);
    }}
}}
"""
    launch = """
    if (in2_mode == 1 && perm == nullptr && g_conv_impl != 1 && num_edges > 0 &&
        reinterpret_cast<uintptr_t>(w) % 16 == 0 && reinterpret_cast<uintptr_t>(node_x) % 16 == 0) {
        cudaError_t err = cudaFuncSetAttribute(conv_fwd_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kV2SmemBytes);
        if (err != cudaSuccess) return e3b_layout_fail(-2, "conv_fwd: smem attribute: %s", cudaGetErrorString(err));
        const int64_t want = (num_nodes + kV2Teams - 1) / kV2Teams;
        const unsigned v2grid = static_cast<unsigned>(want < 148 ? want : 148);
        conv_fwd_tma_kernel<<<v2grid, kV2Threads, kV2SmemBytes, s>>>(node_x, x2, edge_src, rowptr, w, out, num_nodes, num_src,
                                                                     num_edges, scale, status);
        return e3b_layout_check("conv_fwd (bulk-copy pipeline)");
    }
"""
    return {"kernel": kernel, "launch": launch, "T": T, "teams": teams}
