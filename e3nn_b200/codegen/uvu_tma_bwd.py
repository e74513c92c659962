"""Generator of the bulk-copy pipelined gradient kernel of the fused convolution.

Same staging and work split as ``uvu_tma.py`` (one warp per edge, two channels per lane, packed
``FFMA2``, weight row and gathered source row brought in by ``cp.async.bulk``), computing for a
cotangent ``g`` given per destination row

    grad_w[e, p, u]  = sum_k g[dst, p, u, k] * s_k,           s_k = sum_i t_ik x[src, u, i]
    grad_Y[e, j]     = sum_{p,u,i,k} C_ijk x[src, u, i] w[e, p, u] g[dst, p, u, k]
    grad_vec[e]      = J_SH(vec[e])^T grad_Y[e]

Per path both gradients come from R_j = sum_ik C_ijk x_i g_k (packed pairs, no per-edge coupling
table): grad_w = sum_j Y_j R_j and grad_Y_j += w R_j.  A warp keeps the cotangent of its output slots
(constant over a destination segment) in registers, accumulates grad_Y as packed pairs and reduces the
<= 16 components over the 32 lanes by recursive halving (16 shuffles instead of 80) into a per-team
shared-memory batch of 32 edges.  The harmonics and their Jacobian are per-edge scalar work: at every
batch boundary the first warp of the team evaluates them one lane per edge (Y of the next 32 edges into
shared memory; grad_vec of the last 32 edges from the sum of the warps' partial grad_Y, in a fixed order,
so the result does not depend on scheduling).  All warps of a team run one copy of the loop code and differ
only in two switch statements: the hot code stays inside the SM's instruction cache (a first version with
one inlined loop per warp role ran at a third of the issue rate, stalled on instruction fetch).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np

from ..o3._wigner import wigner_3j_numpy
from . import uvu_tma

G_FLOATS_PER_WARP = 100     # cotangent registers (2 per output component) one warp may hold: measured on the
                            # 23-path l<=3 layout, teams of 2 fat warps (240 registers, 8 warps per SM) beat teams of
                            # 3 or 4 (9-12 warps) by 12-25 %: every warp repeats the reduction and the staging loads
SMEM_BUDGET = 200 * 1024


def _f(v: float) -> str:
    return f"{np.float32(v):.9e}f"


def eligible(layout) -> bool:
    return uvu_tma.eligible(layout) and layout.d2 <= 16


def split_slots(layout, per_warp: int = 0) -> List[List]:
    """Paths grouped by output slot into the fewest warps that hold ``per_warp`` cotangent registers each."""
    total = 2 * sum(layout.spec.irreps_out[io].ir.dim for io in layout.out_used)
    T = max(1, -(-total // (per_warp or G_FLOATS_PER_WARP)))
    if T == 1:
        return [list(layout.paths)]
    slots: Dict[int, List] = {}
    for p in layout.paths:
        slots.setdefault(p.io, []).append(p)
    items = sorted(slots.values(), key=lambda ps: -sum(uvu_tma._path_cost(p) for p in ps))
    groups: List[List] = [[] for _ in range(T)]
    load = [0] * T
    for ps in items:
        g = load.index(min(load))
        groups[g] += ps
        load[g] += sum(uvu_tma._path_cost(p) for p in ps)
    for g in groups:
        g.sort(key=lambda p: p.index)
    return [g for g in groups if g]


def body(layout, paths) -> Tuple[str, str]:
    """(cotangent loads for a destination row, per-edge body) for one warp of a team.

    Row loads expect ``grow`` (cotangent row) and ``scale``; the edge body expects ``sx``, ``sw`` (staged
    rows), ``Y`` and ``gwrow`` (this edge's weight-gradient row) and accumulates ``DY<j>`` pairs."""
    spec = layout.spec
    o1, oo = spec.irreps_in1.offsets(), spec.irreps_out.offsets()
    gload, out = [], []
    gname: Dict[Tuple[int, int], str] = {}
    for io in sorted({p.io for p in paths}):
        dim = spec.irreps_out[io].ir.dim
        for k in range(dim):
            gname[(io, k)] = f"G{len(gname)}"     # registers are shared by the roles: role-local numbering
            gload.append(f"{gname[(io, k)]} = make_float2(grow[{oo[io]} + lane * {dim} + {k}] * scale, "
                         f"grow[{oo[io]} + (lane + 32) * {dim} + {k}] * scale);")
    for i1 in sorted({p.i1 for p in paths}):
        d = spec.irreps_in1[i1].ir.dim
        for i in range(d):
            out.append(f"const float2 X{i1}_{i} = make_float2(sx[{o1[i1]} + lane * {d} + {i}], sx[{o1[i1]} + (lane + 32) * {d} + {i}]);")
    for p in paths:
        # R_j = sum_ik C_ijk x_i g_k is shared by both gradients: grad_w = sum_j Y_j R_j, grad_Y_j += w R_j
        c = wigner_3j_numpy(p.l1, p.l2, p.l3) * p.pw
        out.append(f"{{ // path {p.index}: l={p.l1} (x) l={p.l2} -> l={p.l3}")
        have = set()
        for i in range(2 * p.l1 + 1):
            for k in range(2 * p.l3 + 1):
                js = [(j, c[i, j, k]) for j in range(2 * p.l2 + 1) if c[i, j, k] != 0.0]
                if not js:
                    continue
                out.append(f"  {{ const float2 P = __fmul2_rn(X{p.i1}_{i}, {gname[(p.io, k)]});")
                for j, v in js:
                    cc = f"make_float2({_f(v)}, {_f(v)})"
                    if j in have:
                        out.append(f"    R{j} = __ffma2_rn({cc}, P, R{j});")
                    else:
                        out.append(f"    R{j} = __fmul2_rn({cc}, P);")
                        have.add(j)
                out.append("  }")
        out.append(f"  const float2 Wp = make_float2(sw[{p.woff} + lane], sw[{p.woff} + lane + 32]);")
        js = sorted(have)
        if js:
            expr = f"__fmul2_rn(YY{p.off2 + js[0]}, R{js[0]})"
            for j in js[1:]:
                expr = f"__ffma2_rn(YY{p.off2 + j}, R{j}, {expr})"
            out.append(f"  const float2 DW = {expr};")
        else:
            out.append("  const float2 DW = make_float2(0.0f, 0.0f);")
        out.append(f"  gwrow[{p.woff} + lane] = DW.x; gwrow[{p.woff} + lane + 32] = DW.y;")
        for j in js:
            out.append(f"  DY{p.off2 + j} = __ffma2_rn(Wp, R{j}, DY{p.off2 + j});")
        out.append("}")
        # declare the R accumulators at the head of the path block
        head = max(idx for idx, line in enumerate(out) if line.startswith("{ // path"))
        out.insert(head + 1, "  float2 " + ", ".join(f"R{j}" for j in range(2 * p.l2 + 1)) + ";")
    return "\n".join(gload), "\n".join(out)


def g_count(layout, paths) -> int:
    return sum(layout.spec.irreps_out[io].ir.dim for io in sorted({p.io for p in paths}))


def _indent(text: str, n: int) -> str:
    pad = " " * n
    return "\n".join(pad + line if line else line for line in text.split("\n"))


def emit(layout, depth: int = 4, max_warps: int = 0) -> Optional[Dict[str, str]]:
    """Backward kernel source + launch code; relies on v2_issue / v2_lower_bound of the forward kernel text."""
    if not eligible(layout):
        return None
    groups = split_slots(layout)
    T = len(groups)
    if max_warps == 0:
        # register budget: a warp holding more than 72 cotangent floats needs about 240 registers per thread
        per_warp = max(2 * g_count(layout, paths) for paths in groups)
        max_warps = 8 if per_warp > 72 else 12
    stage_w, stage_x = layout.wn * 4, layout.d1 * 4
    stage = (stage_w + stage_x + 127) // 128 * 128
    teams = max(1, min(SMEM_BUDGET // (depth * stage + 32 * 20 * 4 + T * 32 * 17 * 4), max_warps // T, 8))
    d2 = layout.d2
    dy_decl = "\n".join(f"float2 DY{j} = make_float2(0.0f, 0.0f); const float2 YY{j} = make_float2(Y[{j}], Y[{j}]);"
                        for j in range(d2))
    dy_fold = "\n".join(f"dy[{j}] = DY{j}.x + DY{j}.y;" for j in range(d2)) + "\n" + \
              "\n".join(f"dy[{j}] = 0.0f;" for j in range(d2, 16))
    bodies = [body(layout, paths) for paths in groups]
    n_g = max(g_count(layout, paths) for paths in groups)
    g_decl = "\n".join(f"float2 G{i} = make_float2(0.0f, 0.0f);" for i in range(n_g))

    def switch(parts: List[str], pad: int) -> str:
        if T == 1:
            return _indent(parts[0], pad)
        lines = ["switch (tw) {"]
        for tw, text in enumerate(parts):
            lines.append(f"case {tw}: {{")
            lines.append(_indent(text, 4))
            lines.append("} break;")
        lines.append("default: break;")
        lines.append("}")
        return _indent("\n".join(lines), pad)

    kernel = f"""
// ================================================================= bulk-copy pipelined gradient of the fused convolution
constexpr int kB2T = {T};
constexpr int kB2Teams = {teams};
constexpr int kB2Threads = kB2T * kB2Teams * 32;
constexpr int kB2Depth = {depth};
constexpr int kB2RingBytes = kB2Depth * kV2StageBytes;
constexpr int kB2YStride = kV2YStride;
constexpr int kB2DyStride = 17;                            // floats per edge of a warp's partial grad_Y (conflict-free columns)
constexpr int kB2BatchFloats = 32 * kB2YStride + kB2T * 32 * kB2DyStride;
constexpr int kB2SmemBytes = kB2Teams * kB2RingBytes + kB2Teams * 2 * kB2Depth * 8 + 128 + kB2Teams * kB2BatchFloats * 4;

// One lane per edge: sum the warps' partial grad_Y of a finished batch, apply the harmonics Jacobian, store.
__device__ __forceinline__ void b2_batch_finish(const float* __restrict__ vec, float* __restrict__ grad_vec, int64_t e0, int count,
                                                const float* dybuf, int lane) {{
    if (lane < count) {{
        const int64_t ee = e0 + lane;
        float gY[kD2];
#pragma unroll
        for (int j = 0; j < kD2; ++j) {{
            float acc = dybuf[lane * kB2DyStride + j];
#pragma unroll
            for (int t = 1; t < kB2T; ++t) acc += dybuf[(t * 32 + lane) * kB2DyStride + j];
            gY[j] = acc;
        }}
        float gx, gy, gz;
        e3b_sh_unit_bwd<kShLmax>(vec[ee * 3], vec[ee * 3 + 1], vec[ee * 3 + 2], gY, gx, gy, gz);
        grad_vec[ee * 3] = gx; grad_vec[ee * 3 + 1] = gy; grad_vec[ee * 3 + 2] = gz;
    }}
}}

// one step of the recursive-halving reduction: lanes with bit O set keep the upper half of the values
template <int O, int H>
__device__ __forceinline__ void b2_halve(float* dy, int lane) {{
    const bool up = (lane & O) != 0;
#pragma unroll
    for (int i = 0; i < H; ++i) {{
        const float send = up ? dy[i] : dy[i + H];
        const float keep = up ? dy[i + H] : dy[i];
        dy[i] = keep + __shfl_xor_sync(0xffffffffu, send, O);
    }}
}}

// The warps of a team differ only in the two switch statements (cotangent loads, per-path arithmetic of
// their output slots); staging, harmonics, reduction and stores are one copy of code for all of them, which
// keeps the kernel's hot code inside the SM's instruction cache.
__global__ void __launch_bounds__(kB2Threads, 1) conv_bwd_tma_kernel(const float* __restrict__ node_x, const float* __restrict__ vec,
        const int64_t* __restrict__ edge_src, const int64_t* __restrict__ rowptr, const float* __restrict__ w,
        const float* __restrict__ gout, float* __restrict__ grad_w, float* __restrict__ grad_vec, int64_t num_nodes,
        int64_t num_src, int64_t num_edges, float scale, int* __restrict__ status) {{
    extern __shared__ __align__(128) uint8_t v2_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int team = warp / kB2T, tw = warp % kB2T;
    uint8_t* ring = v2_smem + team * kB2RingBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(v2_smem + kB2Teams * kB2RingBytes);
    uint64_t* full = bars + team * 2 * kB2Depth;
    uint64_t* empty = full + kB2Depth;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kB2Teams * 2 * kB2Depth);
    float* ybuf = reinterpret_cast<float*>(v2_smem + kB2Teams * kB2RingBytes + kB2Teams * 2 * kB2Depth * 8 + 128) + team * kB2BatchFloats;
    float* dybuf = ybuf + 32 * kB2YStride;
    if (threadIdx.x == 0) *abort_flag = 0;
    if (tw == 0 && lane == 0) {{
        for (int s = 0; s < kB2Depth; ++s) {{ tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], kB2T); }}
        tc::mbar_init_fence();
    }}
    __syncthreads();
    const int64_t team_id = static_cast<int64_t>(blockIdx.x) * kB2Teams + team;
    const int64_t num_teams = static_cast<int64_t>(gridDim.x) * kB2Teams;
    const int64_t n_lo = team_id == 0 ? 0 : v2_lower_bound(rowptr, num_nodes, (num_edges * team_id) / num_teams);
    const int64_t n_hi = team_id + 1 == num_teams ? num_nodes : v2_lower_bound(rowptr, num_nodes, (num_edges * (team_id + 1)) / num_teams);
    if (n_lo >= n_hi) return;
    const bool leader = tw == 0 && lane == 0;
    int64_t e = rowptr[n_lo];
    const int64_t e_hi = rowptr[n_hi];
    int64_t issue = e;
    int64_t src_pref = 0;
    bool ok = true;
    if (leader) {{
        for (int s = 0; s < kB2Depth && issue < e_hi; ++s, ++issue) {{
            int64_t sidx = edge_src[issue];
            if (sidx < 0 || sidx >= num_src) {{ atomicExch(status, 2); sidx = 0; }}
            v2_issue(ring + s * kV2StageBytes, &full[s], w + issue * kWn, node_x + sidx * kD1);
        }}
        if (issue < e_hi) src_pref = edge_src[issue];
    }}
{_indent(g_decl, 4)}
    uint32_t it = 0;
    int64_t seg_end = rowptr[n_lo + 1];
    for (int64_t n = n_lo; n < n_hi; ++n) {{
        const int64_t e_end = seg_end;
        if (n + 2 <= n_hi) seg_end = rowptr[n + 2];
        if (e < e_end) {{
            const float* grow = gout + n * kDout;
{switch([b[0] for b in bodies], 12)}
        }}
        for (; e < e_end; ++e, ++it) {{
            const int slot = static_cast<int>(it & 31u);
            if (slot == 0) {{
                // batch boundary: harmonics and their Jacobian are per-edge scalar work, done one lane per edge
                __syncwarp();
                v2_team_sync<kB2T>(team);
                if (tw == 0) {{
                    if (it > 0) b2_batch_finish(vec, grad_vec, e - 32, 32, dybuf, lane);
                    v2_batch_harmonics(vec, e, e_hi, ybuf, lane);
                }}
                __syncwarp();
                v2_team_sync<kB2T>(team);
            }}
            if (!ok) continue;      // a wait gave up: keep the loop (and the team barriers) going without work
            const int s = it % kB2Depth;
            const uint32_t ph = (it / kB2Depth) & 1u;
            ok = __all_sync(0xffffffffu, tc::mbar_wait(&full[s], ph, abort_flag));
            if (!ok) continue;
            const float* sw = reinterpret_cast<const float*>(ring + s * kV2StageBytes);
            const float* sx = reinterpret_cast<const float*>(ring + s * kV2StageBytes + kV2StageW);
            float* gwrow = grad_w + e * kWn;
            float Y[kD2];
#pragma unroll
            for (int j = 0; j < kD2; ++j) Y[j] = ybuf[slot * kB2YStride + j];
{_indent(dy_decl, 12)}
{switch([b[1] for b in bodies], 12)}
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&empty[s]);
            if (leader && it > 0 && issue < e_hi) {{
                const int sp = (it - 1) % kB2Depth;
                const uint32_t php = ((it - 1) / kB2Depth) & 1u;
                if (tc::mbar_wait(&empty[sp], php, abort_flag)) {{
                    int64_t sidx = src_pref;
                    if (sidx < 0 || sidx >= num_src) {{ atomicExch(status, 2); sidx = 0; }}
                    tc::fence_proxy_async_smem();
                    v2_issue(ring + sp * kV2StageBytes, &full[sp], w + issue * kWn, node_x + sidx * kD1);
                    ++issue;
                    if (issue < e_hi) src_pref = edge_src[issue];
                }}
            }}
            // sum grad_Y over the 64 channels: fold the pairs, then recursive halving over the lanes
            float dy[16];
{_indent(dy_fold, 12)}
            b2_halve<16, 8>(dy, lane); b2_halve<8, 4>(dy, lane); b2_halve<4, 2>(dy, lane); b2_halve<2, 1>(dy, lane);
            dy[0] += __shfl_xor_sync(0xffffffffu, dy[0], 1);
            if ((lane & 1) == 0) dybuf[(tw * 32 + slot) * kB2DyStride + ((lane >> 1) & 15)] = dy[0];
        }}
    }}
    {{
        const int count = (it & 31u) != 0u ? static_cast<int>(it & 31u) : (it > 0 ? 32 : 0);
        __syncwarp();
        v2_team_sync<kB2T>(team);
        if (tw == 0 && ok) b2_batch_finish(vec, grad_vec, e - count, count, dybuf, lane);
    }}
    if (!ok) {{
        if (lane == 0) atomicExch(status, 3);
        for (int q = 0; q < 2000; ++q) __nanosleep(500);
    }}
}}
"""
    launch = """
    if (in2_mode == 1 && perm == nullptr && g_conv_impl != 1 &&
        reinterpret_cast<uintptr_t>(w) % 16 == 0 && reinterpret_cast<uintptr_t>(node_x) % 16 == 0) {
        cudaError_t err = cudaFuncSetAttribute(conv_bwd_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kB2SmemBytes);
        if (err != cudaSuccess) return e3b_layout_fail(-2, "conv_bwd: smem attribute: %s", cudaGetErrorString(err));
        const int64_t want = (num_nodes + kB2Teams - 1) / kB2Teams;
        const unsigned b2grid = static_cast<unsigned>(want < 148 ? want : 148);
        conv_bwd_tma_kernel<<<b2grid, kB2Threads, kB2SmemBytes, s>>>(node_x, x2, edge_src, rowptr, w, grad_out, grad_w, grad_x2,
                                                                     num_nodes, num_src, num_edges, scale, status);
        return e3b_layout_check("conv_bwd (bulk-copy pipeline)");
    }
"""
    return {"kernel": kernel, "launch": launch, "T": T, "teams": teams}
