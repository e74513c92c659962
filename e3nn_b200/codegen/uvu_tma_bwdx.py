"""Generator of the bulk-copy pipelined node-feature gradient of the fused convolution.

    grad_x[src(e), u, i] += sum_paths sum_jk C_ijk Y_e[j] w[e, p, u] g[dst(e), p, u, k]

Same teams, staging ring and batched harmonics as ``uvu_tma.py`` / ``uvu_tma_bwd.py`` (whose device helpers
it reuses), with only the weight row of an edge staged (the result does not depend on the source features).
A warp keeps the cotangent of its output slots for the current destination row in registers, forms per path
``WG_k = w g_k`` and accumulates ``dx_i += C_ijk (Y_j WG_k)`` as packed pairs, then adds its partial row to the
zeroed table: the warps of a team first store their partial rows in shared memory (two sets, alternating
edges), and after a team barrier their sum goes to the table as float atomics on whole 128-byte lines (measured: a
warp adding 32 contiguous floats per instruction runs at HBM speed, the strided per-channel form at a third of it).
Edges are sorted by destination, so the rows of a source are not contiguous and nothing cheaper than an atomic
can combine them.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

from ..o3._wigner import wigner_3j_numpy
from . import uvu_tma, uvu_tma_bwd
from .uvu_tma_bwd import _f, _indent

SMEM_BUDGET = 200 * 1024


def body(layout, paths) -> Tuple[str, str]:
    """(cotangent loads for a destination row, per-edge body) for one warp of a team.

    The edge body expects ``sw`` (staged weight row) and ``Y`` and accumulates ``DX<c>`` pairs, ``c`` the flat
    component index of the first operand (irrep after irrep)."""
    spec = layout.spec
    oo = spec.irreps_out.offsets()
    comp_base: Dict[int, int] = {}
    n = 0
    for i1 in layout.in1_used:
        comp_base[i1] = n
        n += spec.irreps_in1[i1].ir.dim
    gload, out = [], []
    gname: Dict[Tuple[int, int], str] = {}
    for io in sorted({p.io for p in paths}):
        dim = spec.irreps_out[io].ir.dim
        for k in range(dim):
            gname[(io, k)] = f"G{len(gname)}"
            gload.append(f"{gname[(io, k)]} = make_float2(grow[{oo[io]} + lane * {dim} + {k}] * scale, "
                         f"grow[{oo[io]} + (lane + 32) * {dim} + {k}] * scale);")
    for p in paths:
        c = wigner_3j_numpy(p.l1, p.l2, p.l3) * p.pw
        out.append(f"{{ // path {p.index}: l={p.l1} (x) l={p.l2} -> l={p.l3}")
        out.append(f"  const float2 Wp = make_float2(sw[{p.woff} + lane], sw[{p.woff} + lane + 32]);")
        for k in range(2 * p.l3 + 1):
            if not (c[:, :, k] != 0.0).any():
                continue
            out.append(f"  {{ const float2 WG = __fmul2_rn(Wp, {gname[(p.io, k)]});")
            for j in range(2 * p.l2 + 1):
                terms = [(i, c[i, j, k]) for i in range(2 * p.l1 + 1) if c[i, j, k] != 0.0]
                if not terms:
                    continue
                out.append(f"    {{ const float2 P = __fmul2_rn(WG, make_float2(Y[{p.off2 + j}], Y[{p.off2 + j}]));")
                for i, v in terms:
                    d = f"DX{comp_base[p.i1] + i}"
                    out.append(f"      {d} = __ffma2_rn(make_float2({_f(v)}, {_f(v)}), P, {d});")
                out.append("    }")
            out.append("  }")
        out.append("}")
    return "\n".join(gload), "\n".join(out)


# cotangent registers (2 per output component) one warp holds.  Measured on the 23-path lmax-3 layout, 1.7 M edges:
# 100 (2 warps per team, 8 warps, 202 registers) 5.8 ms; 66 (3 warps per team, 12 warps, 159 registers) 5.2 ms --
# the kernel waits on dependent FFMA2 chains and shared-memory loads, so the extra warps pay here, unlike in the
# weight-gradient kernel whose warps hold twice the state.
G_FLOATS_PER_WARP = 66


def emit(layout, depth: int = 4) -> Optional[Dict[str, str]]:
    """Kernel source + launch code; relies on the helpers of the forward and gradient kernels' text."""
    if not uvu_tma_bwd.eligible(layout):
        return None
    groups = uvu_tma_bwd.split_slots(layout, G_FLOATS_PER_WARP)
    T = len(groups)
    spec = layout.spec
    per_warp = max(2 * uvu_tma_bwd.g_count(layout, paths) for paths in groups)
    max_warps = 8 if per_warp > 72 else 12
    stage = (layout.wn * 4 + 127) // 128 * 128
    teams = max(1, min(SMEM_BUDGET // (depth * stage + 32 * 20 * 4 + 2 * T * 4 * ((layout.d1 + 31) // 32 * 32)), max_warps // T, 8))
    bodies = [body(layout, paths) for paths in groups]
    n_g = max(uvu_tma_bwd.g_count(layout, paths) for paths in groups)
    g_decl = "\n".join(f"float2 G{i} = make_float2(0.0f, 0.0f);" for i in range(n_g))
    comps = []      # (flat component, input offset, irrep dim, component within the irrep)
    o1 = spec.irreps_in1.offsets()
    for i1 in layout.in1_used:
        d = spec.irreps_in1[i1].ir.dim
        for i in range(d):
            comps.append((len(comps), o1[i1], d, i))
    dx_decl = "\n".join(f"float2 DX{c} = make_float2(0.0f, 0.0f);" for c, _, _, _ in comps)
    dx_add = "\n".join(
        f"xb[{off} + lane * {d} + {i}] = DX{c}.x; xb[{off} + (lane + 32) * {d} + {i}] = DX{c}.y;"
        for c, off, d, i in comps)

    def switch(parts, pad):
        if T == 1:
            return _indent(parts[0], pad)
        lines = ["switch (tw) {"]
        for tw, text in enumerate(parts):
            lines += [f"case {tw}: {{", _indent(text, 4), "} break;"]
        lines += ["default: break;", "}"]
        return _indent("\n".join(lines), pad)

    kernel = f"""
// ================================================================= bulk-copy pipelined node-feature gradient
constexpr int kX2T = {T};
constexpr int kX2Teams = {teams};
constexpr int kX2Threads = kX2T * kX2Teams * 32;
constexpr int kX2Depth = {depth};
constexpr int kX2StageBytes = {stage};       // one edge's weight row
constexpr int kX2RingBytes = kX2Depth * kX2StageBytes;
constexpr int kX2RowFloats = (kD1 + 31) / 32 * 32;   // one gradient row, padded to whole 128-byte lines
constexpr int kX2SmemBytes = kX2Teams * kX2RingBytes + kX2Teams * 2 * kX2Depth * 8 + 128 + kX2Teams * 32 * kV2YStride * 4 +
                             kX2Teams * 2 * kX2T * kX2RowFloats * 4;

__device__ __forceinline__ void x2_issue(uint8_t* stage, uint64_t* bar, const float* wrow) {{
    const uint32_t b = tc::smem_u32(bar);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(kV2StageW) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(tc::smem_u32(stage)), "l"(wrow), "r"(kV2StageW), "r"(b) : "memory");
}}

__global__ void __launch_bounds__(kX2Threads, 1) conv_bwd_x_tma_kernel(const float* __restrict__ vec,
        const int64_t* __restrict__ edge_src, const int64_t* __restrict__ rowptr, const float* __restrict__ w,
        const float* __restrict__ gout, float* __restrict__ grad_node_x, int64_t num_nodes, int64_t num_src,
        int64_t num_edges, float scale, int* __restrict__ status) {{
    extern __shared__ __align__(128) uint8_t v2_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int team = warp / kX2T, tw = warp % kX2T;
    uint8_t* ring = v2_smem + team * kX2RingBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(v2_smem + kX2Teams * kX2RingBytes);
    uint64_t* full = bars + team * 2 * kX2Depth;
    uint64_t* empty = full + kX2Depth;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kX2Teams * 2 * kX2Depth);
    float* ybuf = reinterpret_cast<float*>(v2_smem + kX2Teams * kX2RingBytes + kX2Teams * 2 * kX2Depth * 8 + 128) + team * 32 * kV2YStride;
    // two sets (alternating edges) of one row per warp: the warps of a team put their partial rows here first, so that
    // the table receives one row per edge in whole 128-byte lines instead of one strided float at a time per warp
    float* xrows = reinterpret_cast<float*>(v2_smem + kX2Teams * kX2RingBytes + kX2Teams * 2 * kX2Depth * 8 + 128) +
                   kX2Teams * 32 * kV2YStride + team * 2 * kX2T * kX2RowFloats;
    if (threadIdx.x == 0) *abort_flag = 0;
    if (tw == 0 && lane == 0) {{
        for (int s = 0; s < kX2Depth; ++s) {{ tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], kX2T); }}
        tc::mbar_init_fence();
    }}
    __syncthreads();
    const int64_t team_id = static_cast<int64_t>(blockIdx.x) * kX2Teams + team;
    const int64_t num_teams = static_cast<int64_t>(gridDim.x) * kX2Teams;
    const int64_t n_lo = team_id == 0 ? 0 : v2_lower_bound(rowptr, num_nodes, (num_edges * team_id) / num_teams);
    const int64_t n_hi = team_id + 1 == num_teams ? num_nodes : v2_lower_bound(rowptr, num_nodes, (num_edges * (team_id + 1)) / num_teams);
    if (n_lo >= n_hi) return;
    const bool leader = tw == 0 && lane == 0;
    int64_t e = rowptr[n_lo];
    const int64_t e_hi = rowptr[n_hi];
    int64_t issue = e;
    bool ok = true;
    if (leader) {{
        for (int s = 0; s < kX2Depth && issue < e_hi; ++s, ++issue) x2_issue(ring + s * kX2StageBytes, &full[s], w + issue * kWn);
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
                __syncwarp();
                v2_team_sync<kX2T>(team);
                if (tw == 0) v2_batch_harmonics(vec, e, e_hi, ybuf, lane);
                __syncwarp();
                v2_team_sync<kX2T>(team);
            }}
            if (!ok) {{ __syncwarp(); v2_team_sync<kX2T>(team); continue; }}   // keep the team barriers in step
            const int s = it % kX2Depth;
            const uint32_t ph = (it / kX2Depth) & 1u;
            int64_t sidx = edge_src[e];   // issued before the wait: its latency overlaps the wait for the staged row
            ok = __all_sync(0xffffffffu, tc::mbar_wait(&full[s], ph, abort_flag));
            if (!ok) {{ __syncwarp(); v2_team_sync<kX2T>(team); continue; }}
            const float* sw = reinterpret_cast<const float*>(ring + s * kX2StageBytes);
            float Y[kD2];
#pragma unroll
            for (int j = 0; j < kD2; ++j) Y[j] = ybuf[slot * kV2YStride + j];
{_indent(dx_decl, 12)}
{switch([b[1] for b in bodies], 12)}
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&empty[s]);
            if (leader && it > 0 && issue < e_hi) {{
                const int sp = (it - 1) % kX2Depth;
                const uint32_t php = ((it - 1) / kX2Depth) & 1u;
                if (tc::mbar_wait(&empty[sp], php, abort_flag)) {{
                    tc::fence_proxy_async_smem();
                    x2_issue(ring + sp * kX2StageBytes, &full[sp], w + issue * kWn);
                    ++issue;
                }}
            }}
            {{
                float* xb = xrows + ((it & 1u) * kX2T + tw) * kX2RowFloats;
{_indent(dx_add, 16)}
            }}
            __syncwarp();
            v2_team_sync<kX2T>(team);
            const bool in_range = sidx >= 0 && sidx < num_src;
            if (!in_range && lane == 0) atomicExch(status, 2);
            {{
                // flush: every warp takes its share of the columns, sums the warps' partial rows, adds to the table
                const float* xb = xrows + (it & 1u) * kX2T * kX2RowFloats;
                float* dxrow = grad_node_x + (in_range ? sidx : 0) * kD1;
#pragma unroll 4
                for (int i = tw * 32 + lane; i < kD1; i += kX2T * 32) {{
                    float v = xb[i];
#pragma unroll
                    for (int t = 1; t < kX2T; ++t) v += xb[t * kX2RowFloats + i];
                    if (in_range) atomicAdd(dxrow + i, v);
                }}
            }}
        }}
    }}
    if (!ok) {{
        if (lane == 0) atomicExch(status, 3);
        for (int q = 0; q < 2000; ++q) __nanosleep(500);
    }}
}}
"""
    launch = """
    if (in2_mode == 1 && perm == nullptr && g_conv_impl != 1 && reinterpret_cast<uintptr_t>(w) % 16 == 0) {
        err = cudaFuncSetAttribute(conv_bwd_x_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kX2SmemBytes);
        if (err != cudaSuccess) return e3b_layout_fail(-2, "conv_bwd_x: smem attribute: %s", cudaGetErrorString(err));
        const int64_t want = (num_nodes + kX2Teams - 1) / kX2Teams;
        const unsigned x2grid = static_cast<unsigned>(want < 148 ? want : 148);
        conv_bwd_x_tma_kernel<<<x2grid, kX2Threads, kX2SmemBytes, s>>>(x2, edge_src, rowptr, w, grad_out, grad_node_x, num_nodes,
                                                                        num_src, num_edges, scale, status);
        return e3b_layout_check("conv_bwd_x (bulk-copy pipeline)");
    }
"""
    return {"kernel": kernel, "launch": launch, "T": T, "teams": teams}
