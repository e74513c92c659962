"""Generator of the bulk-copy pipelined gradient kernel of the fused convolution.

Same staging and work split as ``uvu_tma.py`` (one warp per edge, two channels per lane, packed
``FFMA2``, weight row and gathered source row brought in by ``cp.async.bulk``), computing for a
cotangent ``g`` given per destination row

    grad_w[e, p, u]  = sum_k g[dst, p, u, k] * s_k,           s_k = sum_i t_ik x[src, u, i]
    grad_Y[e, j]     = sum_{p,u,i,k} C_ijk x[src, u, i] w[e, p, u] g[dst, p, u, k]
    grad_vec[e]      = J_SH(vec[e])^T grad_Y[e]

A warp keeps the cotangent of its output slots (constant over a destination segment) in registers,
accumulates grad_Y as packed pairs, reduces the <= 16 components over the 32 lanes by recursive halving
(16 shuffles instead of 80), and applies the spherical-harmonics Jacobian in the kernel.  When the
slots are split over T > 1 warps of a team every warp adds its partial edge-vector gradient with
three float atomics into a zeroed buffer (two addends commute; with three the last bits depend on
the order).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np

from ..o3._wigner import wigner_3j_numpy
from . import uvu_tma

G_FLOATS_PER_WARP = 72      # cotangent registers (2 per output component) one warp may hold
SMEM_BUDGET = 200 * 1024


def _f(v: float) -> str:
    return f"{np.float32(v):.9e}f"


def eligible(layout) -> bool:
    return uvu_tma.eligible(layout) and layout.d2 <= 16


def split_slots(layout) -> List[List]:
    total = 2 * sum(layout.spec.irreps_out[io].ir.dim for io in layout.out_used)
    T = max(1, -(-total // G_FLOATS_PER_WARP))
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
    for io in sorted({p.io for p in paths}):
        dim = spec.irreps_out[io].ir.dim
        for k in range(dim):
            gload.append(f"G{io}_{k} = make_float2(grow[{oo[io]} + lane * {dim} + {k}] * scale, "
                         f"grow[{oo[io]} + (lane + 32) * {dim} + {k}] * scale);")
    for i1 in sorted({p.i1 for p in paths}):
        d = spec.irreps_in1[i1].ir.dim
        for i in range(d):
            out.append(f"const float2 X{i1}_{i} = make_float2(sx[{o1[i1]} + lane * {d} + {i}], sx[{o1[i1]} + (lane + 32) * {d} + {i}]);")
    for p in paths:
        c = wigner_3j_numpy(p.l1, p.l2, p.l3) * p.pw
        out.append(f"{{ // path {p.index}: l={p.l1} (x) l={p.l2} -> l={p.l3}")
        names = {}
        for i in range(2 * p.l1 + 1):
            for k in range(2 * p.l3 + 1):
                terms = [(j, c[i, j, k]) for j in range(2 * p.l2 + 1) if c[i, j, k] != 0.0]
                if terms:
                    expr = " + ".join(f"{_f(v)} * Y[{p.off2 + j}]" for j, v in terms)
                    out.append(f"  const float t{i}_{k} = {expr}; const float2 T{i}_{k} = make_float2(t{i}_{k}, t{i}_{k});")
                    names[(i, k)] = f"T{i}_{k}"
        out.append(f"  const float2 Wp = make_float2(sw[{p.woff} + lane], sw[{p.woff} + lane + 32]);")
        # grad_w = sum_k g_k s_k
        dw = None
        for k in range(2 * p.l3 + 1):
            terms = [(names[(i, k)], f"X{p.i1}_{i}") for i in range(2 * p.l1 + 1) if (i, k) in names]
            if not terms:
                continue
            expr = f"__fmul2_rn({terms[0][0]}, {terms[0][1]})"
            for t, x in terms[1:]:
                expr = f"__ffma2_rn({t}, {x}, {expr})"
            if dw is None:
                out.append(f"  float2 DW = __fmul2_rn(G{p.io}_{k}, {expr});")
                dw = True
            else:
                out.append(f"  DW = __ffma2_rn(G{p.io}_{k}, {expr}, DW);")
        if dw is None:
            out.append("  const float2 DW = make_float2(0.0f, 0.0f);")
        out.append(f"  gwrow[{p.woff} + lane] = DW.x; gwrow[{p.woff} + lane + 32] = DW.y;")
        # grad_Y_j += C_ijk x_i (w g_k)
        for k in range(2 * p.l3 + 1):
            out.append(f"  const float2 WG{k} = __fmul2_rn(Wp, G{p.io}_{k});")
        for i in range(2 * p.l1 + 1):
            for k in range(2 * p.l3 + 1):
                js = [(j, c[i, j, k]) for j in range(2 * p.l2 + 1) if c[i, j, k] != 0.0]
                if not js:
                    continue
                out.append(f"  {{ const float2 Q = __fmul2_rn(X{p.i1}_{i}, WG{k});")
                for j, v in js:
                    out.append(f"    DY{p.off2 + j} = __ffma2_rn(make_float2({_f(v)}, {_f(v)}), Q, DY{p.off2 + j}); }}"
                               if (j, v) == js[-1] else
                               f"    DY{p.off2 + j} = __ffma2_rn(make_float2({_f(v)}, {_f(v)}), Q, DY{p.off2 + j});")
        out.append("}")
    return "\n".join(gload), "\n".join(out)


def g_decl(layout, paths) -> str:
    spec = layout.spec
    lines = []
    for io in sorted({p.io for p in paths}):
        for k in range(spec.irreps_out[io].ir.dim):
            lines.append(f"float2 G{io}_{k} = make_float2(0.0f, 0.0f);")
    return "\n".join(lines)


def _indent(text: str, n: int) -> str:
    pad = " " * n
    return "\n".join(pad + line if line else line for line in text.split("\n"))


def emit(layout, depth: int = 3) -> Optional[Dict[str, str]]:
    """Backward kernel source + launch code; relies on v2_issue / v2_lower_bound of the forward kernel text."""
    if not eligible(layout):
        return None
    groups = split_slots(layout)
    T = len(groups)
    stage_w, stage_x = layout.wn * 4, layout.d1 * 4
    stage = (stage_w + stage_x + 127) // 128 * 128
    teams = max(1, min(SMEM_BUDGET // (depth * stage), 12 // T, 8))
    d2 = layout.d2
    dy_decl = "\n".join(f"float2 DY{j} = make_float2(0.0f, 0.0f);" for j in range(d2))
    dy_fold = "\n".join(f"dy[{j}] = DY{j}.x + DY{j}.y;" for j in range(d2)) + "\n" + \
              "\n".join(f"dy[{j}] = 0.0f;" for j in range(d2, 16))
    funcs = []
    for tw, paths in enumerate(groups):
        gload, edge_body = body(layout, paths)
        leader = "true" if tw == 0 else "false"
        funcs.append(f"""
__device__ __forceinline__ void b2_team_warp_{tw}(const float* __restrict__ node_x, const float* __restrict__ vec,
        const int64_t* __restrict__ edge_src, const int64_t* __restrict__ rowptr, const float* __restrict__ w,
        const float* __restrict__ gout, float* __restrict__ grad_w, float* __restrict__ grad_vec, int64_t n_lo, int64_t n_hi,
        int64_t num_src, float scale, uint8_t* ring, uint64_t* full, uint64_t* empty, float* sdy,
        volatile int* abort_flag, int* status, int lane) {{
    constexpr bool kLeader = {leader};
    if (n_lo >= n_hi) return;
    int64_t e = rowptr[n_lo];
    const int64_t e_hi = rowptr[n_hi];
    int64_t issue = e;
    int64_t src_pref = 0;
    bool ok = true;
    if (kLeader && lane == 0) {{
        for (int s = 0; s < kB2Depth && issue < e_hi; ++s, ++issue) {{
            int64_t sidx = edge_src[issue];
            if (sidx < 0 || sidx >= num_src) {{ atomicExch(status, 2); sidx = 0; }}
            v2_issue(ring + s * kV2StageBytes, &full[s], w + issue * kWn, node_x + sidx * kD1);
        }}
        if (issue < e_hi) src_pref = edge_src[issue];
    }}
    float vx = 0.f, vy = 0.f, vz = 0.f;
    if (e < e_hi) {{ vx = vec[e * 3]; vy = vec[e * 3 + 1]; vz = vec[e * 3 + 2]; }}
{_indent(g_decl(layout, paths), 4)}
    uint32_t it = 0;
    int64_t seg_end = rowptr[n_lo + 1];
    for (int64_t n = n_lo; n < n_hi && ok; ++n) {{
        const int64_t e_end = seg_end;
        if (n + 2 <= n_hi) seg_end = rowptr[n + 2];
        if (e < e_end) {{
            const float* grow = gout + n * kDout;
{_indent(gload, 12)}
        }}
        for (; e < e_end; ++e, ++it) {{
            const int s = it % kB2Depth;
            const uint32_t ph = (it / kB2Depth) & 1u;
            float nvx = 0.f, nvy = 0.f, nvz = 0.f;
            if (e + 1 < e_hi) {{ nvx = vec[(e + 1) * 3]; nvy = vec[(e + 1) * 3 + 1]; nvz = vec[(e + 1) * 3 + 2]; }}
            if (!tc::mbar_wait(&full[s], ph, abort_flag)) {{ ok = false; break; }}
            const float* sw = reinterpret_cast<const float*>(ring + s * kV2StageBytes);
            const float* sx = reinterpret_cast<const float*>(ring + s * kV2StageBytes + kV2StageW);
            float* gwrow = grad_w + e * kWn;
            float Y[kD2];
            {{
                const float inv = 1.0f / fmaxf(sqrtf(vx * vx + vy * vy + vz * vz), 1e-12f);
                e3b_sh_fwd<kShLmax>(vx * inv, vy * inv, vz * inv, Y);
            }}
{_indent(dy_decl, 12)}
{_indent(edge_body, 12)}
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&empty[s]);
            if (kLeader && lane == 0 && it > 0 && issue < e_hi) {{
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
            __syncwarp();
            if ((lane & 1) == 0) sdy[(lane >> 1) & 15] = dy[0];
            __syncwarp();
            float gY[kD2];
#pragma unroll
            for (int j = 0; j < kD2; ++j) gY[j] = sdy[j];
            float gx, gy, gz;
            e3b_sh_unit_bwd<kShLmax>(vx, vy, vz, gY, gx, gy, gz);
            if (lane == 0) {{
                if (kB2T == 1) {{ grad_vec[e * 3] = gx; grad_vec[e * 3 + 1] = gy; grad_vec[e * 3 + 2] = gz; }}
                else {{ atomicAdd(grad_vec + e * 3, gx); atomicAdd(grad_vec + e * 3 + 1, gy); atomicAdd(grad_vec + e * 3 + 2, gz); }}
            }}
            vx = nvx; vy = nvy; vz = nvz;
        }}
    }}
    if (!ok) {{
        if (lane == 0) atomicExch(status, 3);
        for (int q = 0; q < 2000; ++q) __nanosleep(500);
    }}
}}
""")
    dispatch = "\n".join(
        f"    {'else ' if tw else ''}if (tw == {tw}) b2_team_warp_{tw}(node_x, vec, edge_src, rowptr, w, gout, grad_w, grad_vec, n_lo, n_hi, num_src, scale, ring, full, empty, sdy, abort_flag, status, lane);"
        for tw in range(T))
    kernel = f"""
// ================================================================= bulk-copy pipelined gradient of the fused convolution
constexpr int kB2T = {T};
constexpr int kB2Teams = {teams};
constexpr int kB2Threads = kB2T * kB2Teams * 32;
constexpr int kB2Depth = {depth};
constexpr int kB2RingBytes = kB2Depth * kV2StageBytes;
constexpr int kB2SmemBytes = kB2Teams * kB2RingBytes + kB2Teams * 2 * kB2Depth * 8 + 128 + kB2Teams * kB2T * 64;

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
{''.join(funcs)}
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
    float* sdy = reinterpret_cast<float*>(v2_smem + kB2Teams * kB2RingBytes + kB2Teams * 2 * kB2Depth * 8 + 128) + warp * 16;
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
{dispatch}
}}
"""
    launch = """
    if (in2_mode == 1 && perm == nullptr && g_conv_impl != 1 &&
        reinterpret_cast<uintptr_t>(w) % 16 == 0 && reinterpret_cast<uintptr_t>(node_x) % 16 == 0) {
        cudaError_t err = cudaFuncSetAttribute(conv_bwd_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kB2SmemBytes);
        if (err != cudaSuccess) return e3b_layout_fail(-2, "conv_bwd: smem attribute: %s", cudaGetErrorString(err));
        if (kB2T > 1) {
            err = cudaMemsetAsync(grad_x2, 0, sizeof(float) * 3 * static_cast<size_t>(num_edges), s);
            if (err != cudaSuccess) return e3b_layout_fail(-2, "conv_bwd: memset: %s", cudaGetErrorString(err));
        }
        const int64_t want = (num_nodes + kB2Teams - 1) / kB2Teams;
        const unsigned b2grid = static_cast<unsigned>(want < 148 ? want : 148);
        conv_bwd_tma_kernel<<<b2grid, kB2Threads, kB2SmemBytes, s>>>(node_x, x2, edge_src, rowptr, w, grad_out, grad_w, grad_x2,
                                                                     num_nodes, num_src, num_edges, scale, status);
        return e3b_layout_check("conv_bwd (bulk-copy pipeline)");
    }
"""
    return {"kernel": kernel, "launch": launch, "T": T, "teams": teams}
