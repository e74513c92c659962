"""CUDA source generator for fully-connected ('uvw') tensor products on the tcgen05 tensor cores.

For every output irrep ("group") the shared-weight contraction
(``e3nn/o3/_tensor_product/_codegen.py:148-165``) is the GEMM

    D_k[z, w] = sum_K A_k[z, K] * W[K, w],     k = 0..2l3,   K = (path, u)

whose left operand is produced on the fly from the two input rows,
``A_k[z,(p,u)] = pw_p * sum_{ij} C_ijk x1[z,u,i] x2[z,j]`` (one multiplicity in x2 per irrep).

Kernel structure (one CTA per SM, persistent, a CTA serves one group):
  * prologue: the group's weights are copied once into shared memory, rounded to tf32, in the
    K-major 128-byte-swizzled layout the MMA reads;
  * 8 producer warps evaluate A for 32 consecutive K (one chunk = 32 channels of one path) of a
    128-row tile with generated straight-line Clebsch-Gordan code and store it (tf32, swizzled)
    into a shared-memory stage, one 128x32 sub-tile per k;
  * one thread issues ``tcgen05.mma.kind::tf32`` (M=128, N=mul_out, K=8) four times per chunk and k,
    accumulating in tensor memory; ``tcgen05.commit`` releases the stage and, after the last chunk,
    publishes the accumulators;
  * 4 epilogue warps read the accumulators with ``tcgen05.ld`` and write the output rows, while the
    next tile is already being accumulated in the second TMEM buffer.
All waits are bounded (mbarrier try_wait with an iteration limit and a block-wide abort flag).

Eligibility: every live path 'uvw' with shared weights, in2 multiplicities 1, in1 multiplicities
multiples of 32, 16 <= mul_out <= 256 and mul_out % 16 == 0.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

from ..o3._spec import TPSpec
from ..o3._wigner import wigner_3j_numpy

SMEM_LIMIT = 227 * 1024
STAGE_TILE_BYTES = 128 * 128  # 128 rows x 32 tf32


def _f(v: float) -> str:
    return f"{np.float32(v):.9e}f"


@dataclass
class TcPath:
    index: int
    l1: int
    l2: int
    l3: int
    mul1: int
    off1: int
    off2: int
    woff: int
    pw: float


@dataclass
class TcGroup:
    i_out: int
    out_off: int
    n: int
    dim: int
    paths: List[TcPath]

    @property
    def k(self) -> int:
        return sum(p.mul1 for p in self.paths)

    @property
    def nchunk(self) -> int:
        return self.k // 32

    def chunks(self) -> List[Tuple[int, int]]:
        """(path position in self.paths, first channel) per chunk of 32 K."""
        out = []
        for pi, p in enumerate(self.paths):
            for u0 in range(0, p.mul1, 32):
                out.append((pi, u0))
        return out

    def nbuf(self) -> int:
        return 2 if 2 * self.dim * self.n <= 512 else 1

    def nstage(self, y_bytes: int = 8192) -> int:
        b = self.n * self.k * 4
        stage = self.dim * STAGE_TILE_BYTES
        n = (SMEM_LIMIT - 2048 - y_bytes - b) // stage
        return int(max(0, min(n, 6)))

    def smem_bytes(self, y_bytes: int = 8192) -> int:
        return self.n * self.k * 4 + self.nstage(y_bytes) * self.dim * STAGE_TILE_BYTES + y_bytes + 1024 + 1024


def plan_groups(spec: TPSpec) -> Optional[List[TcGroup]]:
    """Groups of an eligible spec, or None when the layout does not fit the tensor-core kernel."""
    if not spec.shared_weights:
        return None
    live = spec.live_instructions()
    if not live or any(ins.connection_mode != "uvw" for _, ins in live):
        return None
    o1, o2, oo = spec.irreps_in1.offsets(), spec.irreps_in2.offsets(), spec.irreps_out.offsets()
    woffs = spec.weight_offsets()
    groups: Dict[int, TcGroup] = {}
    for n, ins in live:
        (m1, ir1), (m2, ir2), (mo, iro) = spec.irreps_in1[ins.i_in1], spec.irreps_in2[ins.i_in2], spec.irreps_out[ins.i_out]
        if m2 != 1 or m1 % 32 != 0 or mo % 16 != 0 or not (16 <= mo <= 256):
            return None
        g = groups.setdefault(ins.i_out, TcGroup(ins.i_out, oo[ins.i_out], mo, iro.dim, []))
        g.paths.append(TcPath(n, ir1.l, ir2.l, iro.l, m1, o1[ins.i_in1], o2[ins.i_in2], woffs[n], float(ins.path_weight)))
    out = [groups[k] for k in sorted(groups)]
    for g in out:
        if g.dim * g.n > 512 or g.nstage() < 2 or 128 * spec.irreps_in2.dim * 4 > 8192:
            return None
    if spec.irreps_out.dim % 4 != 0 or any(g.out_off % 4 != 0 for g in out):
        return None
    return out


def _producer_path_code(p: TcPath, dim: int, d1_total: int, d2_total: int) -> str:
    """Body of one `case` of the producer switch: fills this warp's rows of every k sub-tile.

    In scope: xbase (-> x1[z0, u, 0] of this lane's channel), sy (this warp's rows of x2 in shared
    memory, [kRowsPerWarp][D2]), z0, Z, pw (producer warp index), lane, stage.  All global loads of the
    warp's rows are issued before the first use (one exposed latency per chunk); rows past Z read
    row Z-1 (valid memory) and their values are never used.
    """
    c = wigner_3j_numpy(p.l1, p.l2, p.l3) * p.pw
    d1, d2 = 2 * p.l1 + 1, 2 * p.l2 + 1
    lines = [f"float xi[kRowsPerWarp][{d1}];"]
    lines.append("#pragma unroll\nfor (int b = 0; b < kRowsPerWarp; ++b) {")
    lines.append("  const int r = pw * kRowsPerWarp + b;")
    lines.append("  const int64_t zr = (z0 + r < Z) ? r : (Z - 1 - z0);")
    lines.append(f"  const float* xr = xbase + zr * {d1_total};")
    lines.append(f"#pragma unroll\n  for (int i = 0; i < {d1}; ++i) xi[b][i] = xr[i];")
    lines.append("}")
    lines.append("#pragma unroll\nfor (int b = 0; b < kRowsPerWarp; ++b) {")
    lines.append("  const int r = pw * kRowsPerWarp + b;")
    lines.append("  const uint32_t off = tc::sw128_offset(r, lane);")
    lines.append(f"  float yj[{d2}];")
    lines.append(f"#pragma unroll\n  for (int j = 0; j < {d2}; ++j) yj[j] = sy[b * {d2_total} + {p.off2} + j];")
    for k in range(dim):
        terms = []
        for i in range(d1):
            inner = [(j, c[i, j, k]) for j in range(d2) if c[i, j, k] != 0.0]
            if not inner:
                continue
            t = " + ".join(f"{_f(v)} * yj[{j}]" for j, v in inner)
            terms.append(f"({t}) * xi[b][{i}]")
        expr = " + ".join(terms) if terms else "0.0f"
        lines.append(f"  *reinterpret_cast<float*>(stage + {k} * TILE_BYTES + off) = tc::to_tf32({expr});")
    lines.append("}")
    return "\n".join(lines)


def _chunk_cost(p: TcPath, dim: int) -> int:
    """Relative cost of producing one 32-channel chunk of a path: one exposed load latency plus
    loads, FMAs and stores per row."""
    c = wigner_3j_numpy(p.l1, p.l2, p.l3)
    return 40 + (2 * p.l1 + 1) + (2 * p.l2 + 1) + 2 * int((c != 0).sum()) + 2 * dim


def _indent(text: str, n: int) -> str:
    pad = " " * n
    return "\n".join(pad + line if line and not line.startswith("#pragma") else line for line in text.split("\n"))


def emit_module(spec: TPSpec) -> str:
    groups = plan_groups(spec)
    assert groups is not None, "layout not eligible for the tensor-core kernel"
    d1, d2, dout = spec.irreps_in1.dim, spec.irreps_in2.dim, spec.irreps_out.dim
    smem_max = max(g.smem_bytes() for g in groups)
    assert smem_max <= SMEM_LIMIT

    consts, funcs = [], []
    for gi, g in enumerate(groups):
        chunks = g.chunks()
        wbase = [g.paths[pi].woff + u0 * g.n for pi, u0 in chunks]
        xoff = [g.paths[pi].off1 + u0 * (2 * g.paths[pi].l1 + 1) for pi, u0 in chunks]
        cpath = [pi for pi, _ in chunks]
        cd1 = [2 * g.paths[pi].l1 + 1 for pi, _ in chunks]
        consts.append(
            f"__constant__ int kWBase{gi}[{len(chunks)}] = {{{', '.join(map(str, wbase))}}};\n"
            f"__constant__ int kXOff{gi}[{len(chunks)}] = {{{', '.join(map(str, xoff))}}};\n"
            f"__constant__ int kCPath{gi}[{len(chunks)}] = {{{', '.join(map(str, cpath))}}};\n"
            f"__constant__ int kCD1{gi}[{len(chunks)}] = {{{', '.join(map(str, cd1))}}};"
        )
        cases = []
        for pi, p in enumerate(g.paths):
            cases.append(
                f"case {pi}: {{  // path {p.index}: l={p.l1} (x) l={p.l2} -> l={p.l3}\n"
                f"    const float* xbase = x1 + z0 * {d1} + xoff + lane * {2 * p.l1 + 1};\n"
                f"{_indent(_producer_path_code(p, g.dim, d1, d2), 4)}\n"
                f"    break; }}"
            )
        switch = "\n".join(cases)
        funcs.append(f"""
// ---------------------------------------------------------------- group {gi}: {g.n}x l={g.paths[0].l3}, K = {g.k}
__device__ __forceinline__ void run_group_{gi}(const float* __restrict__ x1, const float* __restrict__ x2,
        const float* __restrict__ W, float* __restrict__ out, int64_t Z, int cta, int nctas, uint8_t* smem, int* status) {{
    constexpr int N = {g.n}, DIM = {g.dim}, K = {g.k}, NCHUNK = {g.nchunk}, NSTAGE = {g.nstage()}, NBUF = {g.nbuf()};
    constexpr int OUT_OFF = {g.out_off};
    constexpr uint32_t B_BYTES = N * K * 4, TILE_BYTES = 128 * 128, STAGE_BYTES = DIM * TILE_BYTES;
    constexpr uint32_t IDESC = tc::idesc_tf32_m128(N);
    uint8_t* sB = smem;
    uint8_t* sA = smem + B_BYTES;
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(sA + NSTAGE * STAGE_BYTES);
    uint64_t* bar_empty = bar_full + NSTAGE;
    uint64_t* bar_acc_full = bar_empty + NSTAGE;
    uint64_t* bar_acc_empty = bar_acc_full + NBUF;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_acc_empty + NBUF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* sY = reinterpret_cast<float*>(sA + NSTAGE * STAGE_BYTES + 1024);   // [128][D2]: x2 rows of the tile

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- prologue: weights -> shared memory (tf32, K-major, 128B swizzle), barriers, TMEM
    for (int idx = tid; idx < K * N; idx += kThreads) {{
        const int kk = idx / N, w = idx - kk * N;
        const int c = kk >> 5, kc = kk & 31;
        const float v = W[kWBase{gi}[c] + kc * N + w];
        *reinterpret_cast<float*>(sB + c * (N * 128) + tc::sw128_offset(w, kc)) = tc::to_tf32(v);
    }}
    if (tid == 0) {{
        *abort_flag = 0;
        for (int s = 0; s < NSTAGE; ++s) {{ tc::mbar_init(&bar_full[s], kProducerWarps); tc::mbar_init(&bar_empty[s], 1); }}
        for (int b = 0; b < NBUF; ++b) {{ tc::mbar_init(&bar_acc_full[b], 1); tc::mbar_init(&bar_acc_empty[b], kEpilogueWarps); }}
        tc::mbar_init_fence();
    }}
    if (warp == kMmaWarp) tc::tmem_alloc(tmem_slot, kTmemCols);
    tc::fence_proxy_async_smem();
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t tiles = (Z + 127) / 128;

    if (warp < kEpilogueWarps) {{
        // ================= epilogue: TMEM -> registers -> global
        int tile_i = 0;
        for (int64_t t = cta; t < tiles; t += nctas, ++tile_i) {{
            const int b = tile_i % NBUF;
            const uint32_t bph = (tile_i / NBUF) & 1;
            if (!tc::mbar_wait(&bar_acc_full[b], bph, abort_flag)) break;
            tc::tc_fence_after_sync();
            const int64_t z = t * 128 + warp * 32 + lane;
            float* orow = out + z * {dout} + OUT_OFF;
            const uint32_t tbase = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + b * (DIM * N);
            for (int w0 = 0; w0 < N; w0 += 8) {{
                uint32_t r[DIM][8];
#pragma unroll
                for (int k = 0; k < DIM; ++k) tc::tmem_ld8(tbase + k * N + w0, r[k]);
                tc::tmem_ld_wait();
                if (z < Z) {{
                    float v[8 * DIM];
#pragma unroll
                    for (int j = 0; j < 8; ++j)
#pragma unroll
                        for (int k = 0; k < DIM; ++k) v[j * DIM + k] = __uint_as_float(r[k][j]);
                    float4* dst = reinterpret_cast<float4*>(orow + w0 * DIM);
#pragma unroll
                    for (int q = 0; q < 2 * DIM; ++q) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                }}
            }}
            tc::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&bar_acc_empty[b]);
        }}
    }} else if (warp < kEpilogueWarps + kProducerWarps) {{
        // ================= producers: A chunks (CG contraction of the two input rows)
        const int pw = warp - kEpilogueWarps;
        uint32_t it = 0;
        bool ok = true;
        float* sy = sY + pw * kRowsPerWarp * {d2};
        for (int64_t t = cta; t < tiles && ok; t += nctas) {{
            const int64_t z0 = t * 128;
            __syncwarp();
            for (int idx = lane; idx < kRowsPerWarp * {d2}; idx += 32) {{   // this warp's rows of x2 -> shared memory
                const int r = pw * kRowsPerWarp + idx / {d2};
                const int64_t zr = (z0 + r < Z) ? r : (Z - 1 - z0);
                sy[idx] = x2[(z0 + zr) * {d2} + idx % {d2}];
            }}
            __syncwarp();
            for (int c = 0; c < NCHUNK; ++c, ++it) {{
                {{
                    // the x1 values of the chunk two ahead (of this tile, or of the CTA's next tile) are
                    // requested into L2 now: no registers are held, and the loads that follow find them closer
                    const bool same = c + 2 < NCHUNK;
                    const int cn = same ? c + 2 : (c + 2 - NCHUNK < NCHUNK ? c + 2 - NCHUNK : NCHUNK - 1);
                    const int64_t zn = same ? z0 : z0 + static_cast<int64_t>(nctas) * 128;
                    if (zn < Z) {{
                        const float* nb = x1 + kXOff{gi}[cn] + lane * kCD1{gi}[cn];
#pragma unroll
                        for (int b = 0; b < kRowsPerWarp; ++b) {{
                            int64_t z = zn + pw * kRowsPerWarp + b;
                            if (z >= Z) z = Z - 1;
                            asm volatile("prefetch.global.L2 [%0];" ::"l"(nb + z * {d1}));
                        }}
                    }}
                }}
                const int s = it % NSTAGE;
                const uint32_t ph = (it / NSTAGE) & 1;
                if (!tc::mbar_wait(&bar_empty[s], ph ^ 1u, abort_flag)) {{ ok = false; break; }}
                uint8_t* stage = sA + s * STAGE_BYTES;
                const int path = kCPath{gi}[c], xoff = kXOff{gi}[c];
                switch (path) {{
{_indent(switch, 16)}
                }}
                tc::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&bar_full[s]);
            }}
        }}
    }} else if (warp == kMmaWarp && lane == 0) {{
        // ================= MMA issue (single thread)
        uint32_t it = 0;
        int tile_i = 0;
        bool ok = true;
        for (int64_t t = cta; t < tiles && ok; t += nctas, ++tile_i) {{
            const int b = tile_i % NBUF;
            const uint32_t bph = (tile_i / NBUF) & 1;
            if (!tc::mbar_wait(&bar_acc_empty[b], bph ^ 1u, abort_flag)) break;
            tc::tc_fence_after_sync();
            for (int c = 0; c < NCHUNK; ++c, ++it) {{
                const int s = it % NSTAGE;
                const uint32_t ph = (it / NSTAGE) & 1;
                if (!tc::mbar_wait(&bar_full[s], ph, abort_flag)) {{ ok = false; break; }}
                tc::tc_fence_after_sync();
                // descriptors differ only in their address field (bytes >> 4): constant offsets on two values
                const uint64_t adesc = tc::smem_desc_k_sw128(tc::smem_u32(sA + s * STAGE_BYTES));
                const uint64_t bdesc = tc::smem_desc_k_sw128(tc::smem_u32(sB + c * (N * 128)));
                const uint32_t d0 = tmem_base + b * (DIM * N);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {{
#pragma unroll
                    for (int k = 0; k < DIM; ++k) {{
                        tc::mma_tf32(d0 + k * N, adesc + ((k * TILE_BYTES + ks * 32) >> 4), bdesc + ((ks * 32) >> 4), IDESC,
                                     (c > 0 || ks > 0) ? 1u : 0u);
                    }}
                }}
                tc::mma_commit(&bar_empty[s]);
            }}
            if (ok) tc::mma_commit(&bar_acc_full[b]);
        }}
    }}
    tc::tc_fence_before_sync();
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicExch(status, 3);
    if (warp == kMmaWarp) tc::tmem_dealloc(tmem_base, kTmemCols);
}}
""")

    ngroups = len(groups)
    dispatch = "\n".join(
        f"    {'else ' if gi else ''}if (blockIdx.x < cta_end{gi}) run_group_{gi}(x1, x2, W, out, Z, blockIdx.x - cta_begin{gi}, cta_end{gi} - cta_begin{gi}, smem, status);"
        for gi in range(ngroups)
    )
    bounds_decl = "\n".join(
        f"    const int cta_begin{gi} = {'0' if gi == 0 else f'cta_end{gi-1}'}, cta_end{gi} = cta_begin{gi} + split.n[{gi}];" for gi in range(ngroups)
    )
    work = [sum(_chunk_cost(g.paths[pi], g.dim) for pi, _ in g.chunks()) for g in groups]
    # the scalar-output group (one sub-tile per stage, 128 rows per tile) needs about 1.35 x the CTAs this model gives it
    work = [int(w * 1.35) if g.dim == 1 else w for w, g in zip(work, groups)]
    return f"""// Generated by e3nn_b200/codegen/uvw_tc.py -- do not edit.
// layout: {spec.irreps_in1} (x) {spec.irreps_in2} -> {spec.irreps_out}, {sum(len(g.paths) for g in groups)} 'uvw' paths, key {spec.key()}
#include <cuda_runtime.h>
#include <cstdint>
#include "layout_common.cuh"
#include "tc_common.cuh"

namespace {{

constexpr int kEpilogueWarps = 4;
constexpr int kProducerWarps = 16;
constexpr int kMmaWarp = kEpilogueWarps + kProducerWarps;
constexpr int kThreads = (kMmaWarp + 1) * 32;
constexpr int kTmemCols = 512;
constexpr int kRowsPerWarp = 128 / kProducerWarps;
constexpr int kGroups = {ngroups};
constexpr int kSmemBytes = {smem_max};

struct CtaSplit {{ int n[kGroups]; }};

{chr(10).join(consts)}
{''.join(funcs)}

__global__ void __launch_bounds__(kThreads, 1) uvw_tc_kernel(const float* __restrict__ x1, const float* __restrict__ x2,
        const float* __restrict__ W, float* __restrict__ out, int64_t Z, CtaSplit split, int* status) {{
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle atoms of the MMA operands
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
{bounds_decl}
{dispatch}
}}

}}  // namespace

extern "C" int e3b_layout_info(int32_t* dims) {{
    dims[0] = {d1}; dims[1] = {d2}; dims[2] = {dout}; dims[3] = {spec.weight_numel}; dims[4] = -1; dims[5] = kThreads;
    return 0;
}}
extern "C" const char* e3b_layout_key(void) {{ return "{spec.key()}"; }}
extern "C" const char* e3b_layout_last_error(void) {{ return e3b_layout_error_buffer(); }}

// Relative cost of one 128-row tile per group (left-operand production dominates): used to split the CTAs.
static const int kGroupWork[kGroups] = {{{', '.join(map(str, work))}}};

extern "C" int e3b_uvw_tc_fwd(const float* x1, const float* x2, const float* weight, float* out, int64_t Z,
                              int num_ctas, int32_t* status, void* stream) {{
    if (Z < 0) return e3b_layout_fail(-1, "uvw_tc_fwd: negative row count");
    if (Z == 0) return 0;
    if (!x1 || !x2 || !weight || !out || !status) return e3b_layout_fail(-1, "uvw_tc_fwd: null pointer");
    if (reinterpret_cast<uintptr_t>(out) % 16 != 0) return e3b_layout_fail(-1, "uvw_tc_fwd: out must be 16-byte aligned");
    if (num_ctas <= 0) num_ctas = 148;
    if (num_ctas < kGroups) num_ctas = kGroups;
    CtaSplit split;
    long total = 0;
    for (int g = 0; g < kGroups; ++g) total += kGroupWork[g];
    int used = 0;
    for (int g = 0; g < kGroups; ++g) {{
        int n = static_cast<int>((static_cast<long>(num_ctas) * kGroupWork[g]) / total);
        if (n < 1) n = 1;
        split.n[g] = n;
        used += n;
    }}
    for (int g = kGroups - 1; used < num_ctas; g = (g + kGroups - 1) % kGroups) {{ split.n[g]++; used++; }}
    while (used > num_ctas) {{
        int big = 0;
        for (int g = 1; g < kGroups; ++g) if (split.n[g] > split.n[big]) big = g;
        split.n[big]--; used--;
    }}
    cudaError_t err = cudaFuncSetAttribute(uvw_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (err != cudaSuccess) return e3b_layout_fail(-2, "uvw_tc_fwd: smem attribute: %s", cudaGetErrorString(err));
    uvw_tc_kernel<<<used, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(x1, x2, weight, out, Z, split, status);
    return e3b_layout_check("uvw_tc_fwd");
}}
"""
