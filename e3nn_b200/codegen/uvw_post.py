"""CUDA source generator for fully-connected ('uvw') tensor products on the tcgen05 tensor cores, with the
Clebsch-Gordan coupling applied AFTER the matrix product.

The shared-weight contraction of ``e3nn/o3/_tensor_product/_codegen.py:148-165``,

    out[z, w, k] = sum_p pw_p sum_{u} W_p[u, w] sum_{ij} C^p_ijk x1[z, u, i] x2[z, j],

is evaluated as

    V_{p,i}[z, w] = sum_u x1[z, u, i] W_p[u, w]                    (tensor cores: rows z, raw input values)
    out[z, w, k] += sum_i t_{p,ik}(z) V_{p,i}[z, w],   t_{p,ik}(z) = pw_p sum_j C^p_ijk x2[z, j]   (epilogue)

so the left operand of the matrix product is the input row itself (de-interleaved per component i): ``sum(mul1)``
values per row instead of the ``sum_p (2 l3 + 1) mul1`` values of a left operand that already carries the
coupling, and the coupling costs ``nnz(i, k)`` multiply-adds per accumulator value in the thread that owns row z,
where ``t(z)`` is private to the thread (no work is repeated across lanes).  Both orders have the same
matrix-product FLOPs.

Kernel structure (persistent, one CTA per SM, a CTA serves one *group* = an output irrep restricted to a slab of
S <= 64 of its channels):
  * prologue: the group's weight slices W_p[:, slab] -> shared memory, rounded to tf32, K-major 128-byte swizzle;
  * 4 producer warps de-interleave x1: one stage = the 128 x 32 tile ``x1[z0 + r, block(p), 32 kc + u, i]``
    (fixed path p, component i, 32 channels); the 2 l1 + 1 component tiles of a chunk are filled together from
    one contiguous run of each input row (16-byte loads in, 16-byte swizzled stores out); the same run of the
    CTA's next row tile is requested into L2 at the same time;
  * one thread issues ``tcgen05.mma.kind::tf32`` (M = 128, N = S, K = 8): per *job* (path) 2 l1 + 1 accumulators of
    S columns each in one of two tensor-memory regions; jobs alternate between the regions so that the epilogue of
    one job overlaps the matrix products of the next;
  * 8 epilogue warps (two per lane quarter, each owning half of the slab's channels) compute t(z) from the x2 row,
    read the accumulators with ``tcgen05.ld``, keep ``out[z, slab half, :]`` in registers across the jobs of the
    tile and write it once, as one contiguous run per thread.
Register budget: the kernel is compiled for 128 registers per thread (512 threads); the epilogue and producer
warpgroups raise their limit with ``setmaxnreg``, the issue warpgroup lowers its own.
Every mbarrier wait is bounded; a wait that gives up sets the block's abort flag and status 3.

Eligibility: every live path 'uvw' with shared weights, x2 multiplicities 1, x1 multiplicities multiples of 32,
output multiplicities multiples of 16, output rows and group offsets multiples of four floats.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np

from ..o3._spec import TPSpec
from ..o3._wigner import wigner_3j_numpy

SMEM_LIMIT = 227 * 1024
TILE_BYTES = 128 * 128          # 128 rows x 32 tf32
REGION_COLS = (320, 192)        # the two tensor-memory regions (columns)
MAX_ACC_REGS = 96               # accumulator registers of an epilogue thread: (S / 2) * (2 l3 + 1)


def _f(v: float) -> str:
    return f"{np.float32(v):.9e}f"


@dataclass
class Job:
    """One path of a group: 2 l1 + 1 accumulators of S columns."""
    index: int          # instruction index
    l1: int
    l2: int
    l3: int
    mul1: int
    off1: int           # x1 column of the path's input block
    off2: int           # x2 column of the path's second operand
    woff: int           # weight offset of W_p[0, 0]
    pw: float
    region: int = 0
    boff: int = 0       # byte offset of the path's weight tiles in the resident B area

    @property
    def d1(self) -> int:
        return 2 * self.l1 + 1

    @property
    def nchunk(self) -> int:
        return self.mul1 // 32


@dataclass
class Group:
    i_out: int
    l3: int
    nfull: int          # output multiplicity
    col0: int           # first channel of the slab
    s: int              # slab width
    out_off: int        # output column of channel col0, component 0
    jobs: List[Job] = field(default_factory=list)

    @property
    def d3(self) -> int:
        return 2 * self.l3 + 1

    def b_bytes(self) -> int:
        return sum(j.mul1 * self.s * 4 for j in self.jobs)

    def nstage(self) -> int:
        return int(max(0, min(8, (SMEM_LIMIT - 4096 - self.b_bytes()) // TILE_BYTES)))

    def smem_bytes(self) -> int:
        return self.b_bytes() + self.nstage() * TILE_BYTES + 1024 + 1024

    def tiles_per_row_tile(self) -> int:
        return sum(j.d1 * j.nchunk for j in self.jobs)

    def work(self) -> int:
        """Relative cost of one 128-row tile: producer instructions (tiles) plus epilogue multiply-adds."""
        fma = 0
        for j in self.jobs:
            c = wigner_3j_numpy(j.l1, j.l2, j.l3)
            nik = int((np.abs(c).sum(axis=1) != 0).sum())
            fma += nik * self.s
        return 100 * self.tiles_per_row_tile() + fma // 16


def _slab_width(n: int, d1max: int, d3: int) -> Optional[int]:
    for s in (64, 32, 16):
        if n % s == 0 and d1max * s <= max(REGION_COLS) and (s // 2) * d3 <= MAX_ACC_REGS:
            return s
    return None


def plan_groups(spec: TPSpec) -> Optional[List[Group]]:
    """Groups of an eligible spec, or None when the layout does not fit this kernel."""
    if not spec.shared_weights:
        return None
    live = spec.live_instructions()
    if not live or any(ins.connection_mode != "uvw" for _, ins in live):
        return None
    if spec.irreps_in2.dim > 32 or spec.irreps_out.dim % 4 != 0 or spec.irreps_in1.dim % 4 != 0:
        return None
    o1, o2, oo = spec.irreps_in1.offsets(), spec.irreps_in2.offsets(), spec.irreps_out.offsets()
    woffs = spec.weight_offsets()
    by_out: Dict[int, List[Job]] = {}
    for n, ins in live:
        (m1, ir1), (m2, ir2), (mo, iro) = spec.irreps_in1[ins.i_in1], spec.irreps_in2[ins.i_in2], spec.irreps_out[ins.i_out]
        if m2 != 1 or m1 % 32 != 0 or mo % 16 != 0 or o1[ins.i_in1] % 4 != 0:
            return None
        by_out.setdefault(ins.i_out, []).append(
            Job(n, ir1.l, ir2.l, iro.l, m1, o1[ins.i_in1], o2[ins.i_in2], woffs[n], float(ins.path_weight)))
    groups: List[Group] = []
    for i_out in sorted(by_out):
        jobs = by_out[i_out]
        mo, iro = spec.irreps_out[i_out]
        s = _slab_width(mo, max(j.d1 for j in jobs), iro.dim)
        if s is None:
            return None
        for col0 in range(0, mo, s):
            g = Group(i_out, iro.l, mo, col0, s, oo[i_out] + col0 * iro.dim)
            # big jobs to the wide region, the others to the narrow one, alternating as long as both kinds last
            wide = [j for j in jobs if j.d1 * s > REGION_COLS[1]]
            narrow = [j for j in jobs if j.d1 * s <= REGION_COLS[1]]
            if not wide:            # everything fits either region: split evenly
                wide, narrow = narrow[1::2], narrow[0::2]
            order: List[Tuple[Job, int]] = []
            while wide or narrow:
                if narrow:
                    order.append((narrow.pop(0), 1))
                if wide:
                    order.append((wide.pop(0), 0))
            boff = 0
            for j, region in order:
                g.jobs.append(Job(j.index, j.l1, j.l2, j.l3, j.mul1, j.off1, j.off2, j.woff, j.pw, region, boff))
                boff += j.mul1 * s * 4
            if any(j.d1 * s > REGION_COLS[j.region] for j in g.jobs):
                return None
            if g.out_off % 4 != 0 or ((s // 2) * iro.dim) % 4 != 0 or g.nstage() < max(j.d1 for j in g.jobs) + 1:
                return None
            groups.append(g)
    return groups


def _indent(text: str, n: int) -> str:
    pad = " " * n
    return "\n".join(pad + line if line and not line.startswith("#pragma") else line for line in text.split("\n"))


def _epilogue_job_code(g: Group, j: Job, d2_total: int) -> str:
    """Straight-line epilogue of one job for the thread that owns row z: t(z), accumulator reads, multiply-adds.
    In scope: x2r[] (the x2 row), acc[] (HALF * D3 floats), rbase (tensor-memory address of this thread's lane at
    the thread's first column of region 0), valid."""
    c = wigner_3j_numpy(j.l1, j.l2, j.l3) * j.pw
    d1, d2, d3 = j.d1, 2 * j.l2 + 1, g.d3
    half = g.s // 2
    lines = [f"// path {j.index}: l={j.l1} (x) l={j.l2} -> l={j.l3}, {j.mul1} channels, region {j.region}"]
    tnames: Dict[Tuple[int, int], str] = {}
    for i in range(d1):
        for k in range(d3):
            terms = [(jj, c[i, jj, k]) for jj in range(d2) if c[i, jj, k] != 0.0]
            if not terms:
                continue
            expr = " + ".join(f"{_f(v)} * x2r[{j.off2 + jj}]" for jj, v in terms)
            tnames[(i, k)] = f"t{i}_{k}"
            lines.append(f"const float t{i}_{k} = {expr};")
    region_col = 0 if j.region == 0 else REGION_COLS[0]
    step = 8
    lines.append("#pragma unroll")
    lines.append(f"for (int w0 = 0; w0 < {half}; w0 += {step}) {{")
    for i in range(d1):
        lines.append(f"    uint32_t v{i}[{step}];")
        lines.append(f"    tc::tmem_ld8(rbase + {region_col + i * g.s} + w0, v{i});")
    lines.append("    tc::tmem_ld_wait();")
    lines.append("#pragma unroll")
    lines.append(f"    for (int c = 0; c < {step}; ++c) {{")
    for k in range(d3):
        for i in range(d1):
            if (i, k) in tnames:
                lines.append(f"        acc[(w0 + c) * {d3} + {k}] = fmaf({tnames[(i, k)]}, __uint_as_float(v{i}[c]), acc[(w0 + c) * {d3} + {k}]);")
    lines.append("    }")
    lines.append("}")
    return "\n".join(lines)


def emit_module(spec: TPSpec) -> str:
    groups = plan_groups(spec)
    assert groups is not None, "layout not eligible for the tensor-core kernel"
    d1t, d2t, dout = spec.irreps_in1.dim, spec.irreps_in2.dim, spec.irreps_out.dim
    smem_max = max(g.smem_bytes() for g in groups)
    assert smem_max <= SMEM_LIMIT

    consts, funcs = [], []
    for gi, g in enumerate(groups):
        nj = len(g.jobs)
        arr = lambda name, vals: f"__constant__ int {name}{gi}[{nj}] = {{{', '.join(str(v) for v in vals)}}};"
        consts.append("\n".join([
            arr("kJWoff", [j.woff + g.col0 for j in g.jobs]),
            arr("kJMul1", [j.mul1 for j in g.jobs]),
            arr("kJBoff", [j.boff for j in g.jobs]),
            arr("kJXoff", [j.off1 for j in g.jobs]),
            arr("kJD1", [j.d1 for j in g.jobs]),
            arr("kJRegion", [j.region for j in g.jobs]),
        ]))
        half, d3 = g.s // 2, g.d3
        nacc = half * d3
        epi_jobs = []
        for ji, j in enumerate(g.jobs):
            epi_jobs.append(f"""{{
    const int r = {j.region};
    if (!tc::mbar_wait(&bar_reg_full[r], use{j.region} & 1u, abort_flag)) {{ ok = false; break; }}
    tc::tc_fence_after_sync();
{_indent(_epilogue_job_code(g, j, d2t), 4)}
    tc::tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(&bar_reg_empty[r]);
    ++use{j.region};
}}""")
        epi_code = "\n".join(epi_jobs)
        producer_cases = "\n".join(
            f"                    case {d}: ok = produce_group<{d}, NSTAGE>(src, z0, Z, sA, bar_full, bar_empty, it, abort_flag, pw, lane); break;"
            for d in sorted({j.d1 for j in g.jobs}))
        funcs.append(f"""
// ---------------------------------------------------------------- group {gi}: output irrep {g.i_out} (l = {g.l3}), channels [{g.col0}, {g.col0 + g.s}) of {g.nfull}
__device__ __forceinline__ void run_group_{gi}(const float* __restrict__ x1, const float* __restrict__ x2,
        const float* __restrict__ W, float* __restrict__ out, int64_t Z, int cta, int nctas, uint8_t* smem, int* status) {{
    constexpr int S = {g.s}, HALF = {half}, NJOB = {nj}, NSTAGE = {g.nstage()}, NFULL = {g.nfull};
    constexpr int OUT_OFF = {g.out_off};
    constexpr uint32_t B_BYTES = {g.b_bytes()}, TILE = {TILE_BYTES};
    constexpr uint32_t IDESC = tc::idesc_tf32_m128(S);
    uint8_t* sB = smem;
    uint8_t* sA = smem + B_BYTES;
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(sA + NSTAGE * TILE);
    uint64_t* bar_empty = bar_full + NSTAGE;
    uint64_t* bar_reg_full = bar_empty + NSTAGE;      // [2] accumulators of a job complete
    uint64_t* bar_reg_empty = bar_reg_full + 2;       // [2] the epilogue has read them
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_reg_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* tile_progress = abort_flag + 1;     // row tiles the producers have started

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- prologue: the weight slices of the group's paths -> shared memory (tf32, K-major, 128-byte swizzle)
    for (int j = 0; j < NJOB; ++j) {{
        const int total = kJMul1{gi}[j] * S;
        for (int idx = tid; idx < total; idx += kThreads) {{
            const int u = idx / S, w = idx - u * S;
            const float v = W[kJWoff{gi}[j] + u * NFULL + w];
            *reinterpret_cast<float*>(sB + kJBoff{gi}[j] + (u >> 5) * (S * 128) + tc::sw128_offset(w, u & 31)) = tc::to_tf32(v);
        }}
    }}
    if (tid == 0) {{
        *abort_flag = 0;
        *tile_progress = 0;
        for (int s = 0; s < NSTAGE; ++s) {{ tc::mbar_init(&bar_full[s], kProducerWarps); tc::mbar_init(&bar_empty[s], 1); }}
        for (int r = 0; r < 2; ++r) {{ tc::mbar_init(&bar_reg_full[r], 1); tc::mbar_init(&bar_reg_empty[r], kEpilogueWarps); }}
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
        // ================= epilogue: t(z) from the x2 row, accumulators -> registers, coupling, one store per row
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kEpilogueRegs));
        const int q = warp & 3, h = warp >> 2;          // lane quarter of tensor memory, half of the slab
        const uint32_t rbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + h * HALF;
        uint32_t use0 = 0u, use1 = 0u;          // jobs seen so far per tensor-memory region (barrier phase)
        bool ok = true;
        for (int64_t t = cta; t < tiles && ok; t += nctas) {{
            const int64_t z = t * 128 + q * 32 + lane;
            const bool valid = z < Z;
            float x2r[{d2t}];
#pragma unroll
            for (int j = 0; j < {d2t}; ++j) x2r[j] = valid ? x2[z * {d2t} + j] : 0.0f;
            float acc[{nacc}];
#pragma unroll
            for (int a = 0; a < {nacc}; ++a) acc[a] = 0.0f;
            do {{
{_indent(epi_code, 16)}
            }} while (false);
            if (ok && valid) {{
                float4* dst = reinterpret_cast<float4*>(out + z * {dout} + OUT_OFF + h * {nacc});
#pragma unroll
                for (int a = 0; a < {nacc // 4}; ++a) dst[a] = make_float4(acc[4 * a], acc[4 * a + 1], acc[4 * a + 2], acc[4 * a + 3]);
            }}
        }}
    }} else if (warp < kEpilogueWarps + kProducerWarps) {{
        // ================= producers: de-interleaved x1 tiles; the 2 l1 + 1 component tiles of 32 channels are
        // filled together from one contiguous run of the input row (16-byte loads, 16-byte swizzled stores)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kProducerRegs));
        const int pw = warp - kEpilogueWarps;
        uint32_t it = 0;
        int tile_count = 0;
        bool ok = true;
        for (int64_t t = cta; t < tiles && ok; t += nctas) {{
            const int64_t z0 = t * 128;
            if (pw == 0 && lane == 0) *tile_progress = ++tile_count;      // lets the prefetch warp run one row tile ahead
            for (int j = 0; j < NJOB && ok; ++j) {{
                const int d1 = kJD1{gi}[j], nchunk = kJMul1{gi}[j] >> 5;
                for (int kc = 0; kc < nchunk && ok; ++kc) {{
                    const float* src = x1 + kJXoff{gi}[j] + kc * 32 * d1;
                    switch (d1) {{
{producer_cases}
                    default: ok = false; break;
                    }}
                }}
            }}
        }}
    }} else {{
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kIssueRegs));
        if (warp == kMmaWarp && lane == 0) {{
            // ================= MMA issue (single thread)
            uint32_t it = 0;
            uint32_t use0 = 0u, use1 = 0u;
            bool ok = true;
            for (int64_t t = cta; t < tiles && ok; t += nctas) {{
                for (int j = 0; j < NJOB && ok; ++j) {{
                    const int r = kJRegion{gi}[j], d1 = kJD1{gi}[j], nchunk = kJMul1{gi}[j] >> 5;
                    const uint32_t use = r == 0 ? use0 : use1;
                    if (!tc::mbar_wait(&bar_reg_empty[r], (use & 1u) ^ 1u, abort_flag)) {{ ok = false; break; }}
                    tc::tc_fence_after_sync();
                    const uint32_t d0 = tmem_base + (r == 0 ? 0u : {REGION_COLS[0]}u);
                    const uint64_t bdesc0 = tc::smem_desc_k_sw128(tc::smem_u32(sB + kJBoff{gi}[j]));
                    for (int kc = 0; kc < nchunk && ok; ++kc) {{
                        const uint64_t bdesc = bdesc0 + static_cast<uint64_t>(kc) * ((S * 128) >> 4);
                        for (int i = 0; i < d1; ++i, ++it) {{
                            const int s = it % NSTAGE;
                            const uint32_t ph = (it / NSTAGE) & 1;
                            if (!tc::mbar_wait(&bar_full[s], ph, abort_flag)) {{ ok = false; break; }}
                            tc::tc_fence_after_sync();
                            const uint64_t adesc = tc::smem_desc_k_sw128(tc::smem_u32(sA + s * TILE));
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks)
                                tc::mma_tf32(d0 + i * S, adesc + ((ks * 32) >> 4), bdesc + ((ks * 32) >> 4), IDESC,
                                             (kc > 0 || ks > 0) ? 1u : 0u);
                            tc::mma_commit(&bar_empty[s]);
                        }}
                    }}
                    if (ok) tc::mma_commit(&bar_reg_full[r]);
                    if (r == 0) ++use0; else ++use1;
                }}
            }}
        }} else if (warp == kMmaWarp + 1) {{
            // ================= prefetch warp: the x1 and x2 rows of this CTA's NEXT row tile -> L2 while the producers
            // work on the current one (one bulk prefetch per row; a prefetch stalls only this otherwise idle warp)
            int k = 0;
            const bool x2_aligned = (reinterpret_cast<uintptr_t>(x2) & 15u) == 0;
            for (int64_t t = cta; t + nctas < tiles; t += nctas, ++k) {{
                uint32_t spins = 0;
                while (*tile_progress <= k && !*abort_flag && ++spins < 4000000u) __nanosleep(200);
                if (*abort_flag) break;
                const int64_t zn = (t + nctas) * 128;
#pragma unroll
                for (int rr = 0; rr < 4; ++rr) {{
                    int64_t z = zn + rr * 32 + lane;
                    if (z >= Z) z = Z - 1;
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(x1 + z * {d1t}), "r"({d1t * 4}) : "memory");
                }}
                // x2: 16 rows per request.  A bulk prefetch needs a 16-byte aligned address and a size that is a
                // multiple of 16 bytes: rows in multiples of 16 start on such a boundary whatever the row length
                // (16 rows x 4 bytes x length); the size is rounded down, rows past the end are not requested
                if (lane < 8 && x2_aligned) {{
                    const int64_t z = zn + lane * 16;
                    if (z < Z) {{
                        const int64_t rows = Z - z < 16 ? Z - z : 16;
                        const uint32_t n = static_cast<uint32_t>(rows * {d2t * 4}) & ~15u;
                        if (n > 0) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(x2 + z * {d2t}), "r"(n) : "memory");
                    }}
                }}
            }}
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
        for gi in range(ngroups))
    bounds_decl = "\n".join(
        f"    const int cta_begin{gi} = {'0' if gi == 0 else f'cta_end{gi-1}'}, cta_end{gi} = cta_begin{gi} + split.n[{gi}];" for gi in range(ngroups))
    work = [g.work() for g in groups]
    written = {g.i_out for g in groups}
    oo = spec.irreps_out.offsets()
    zero_ranges = [(oo[i], mul * ir.dim) for i, (mul, ir) in enumerate(spec.irreps_out) if i not in written and mul * ir.dim > 0]
    zero_fill = "\n".join(
        f"    {{ cudaError_t e = cudaMemset2DAsync(out + {off}, {dout} * sizeof(float), 0, {n} * sizeof(float), Z, s); "
        f"if (e != cudaSuccess) return e3b_layout_fail(-2, \"uvw_tc_fwd: zero fill: %s\", cudaGetErrorString(e)); }}"
        for off, n in zero_ranges)
    return f"""// Generated by e3nn_b200/codegen/uvw_post.py -- do not edit.
// layout: {spec.irreps_in1} (x) {spec.irreps_in2} -> {spec.irreps_out}, {len(spec.live_instructions())} 'uvw' paths, key {spec.key()}
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdlib>
#include "layout_common.cuh"
#include "tc_common.cuh"

namespace {{

constexpr int kEpilogueWarps = 8;        // warpgroups 0 and 1
constexpr int kProducerWarps = 4;        // warpgroup 2
constexpr int kMmaWarp = 12;             // first warp of warpgroup 3; the next warp prefetches, the other two only take part in barriers
constexpr int kThreads = 16 * 32;
constexpr int kEpilogueRegs = 160, kProducerRegs = 152, kIssueRegs = 40;   // 32 x (8 x 160 + 4 x 152 + 4 x 40) = 65536 = 512 x 128 registers
constexpr int kTmemCols = 512;
constexpr int kGroups = {ngroups};
constexpr int kSmemBytes = {smem_max};

struct CtaSplit {{ int n[kGroups]; }};

// One chunk: rows z0 .. z0 + 127 of 32 channels of an input block with D = 2 l1 + 1 components, i.e. 32 D
// contiguous floats per row, into D consecutive ring stages (stage i = component i as a 128 x 32 K-major tile).
// A thread owns (row, 4 channels) items: D 16-byte loads (element (channel e, component i) at float e D + i), then
// one 16-byte store per component.  The raw fp32 values are stored: the tensor core reads the top 19 bits of a
// tf32 operand (truncation; the weights are rounded to nearest in the prologue).  src: x1 + block offset + 32 kc D.
template <int D, int NSTAGE>
__device__ __forceinline__ bool produce_group(const float* __restrict__ src, int64_t z0, int64_t Z, uint8_t* sA,
        uint64_t* bar_full, uint64_t* bar_empty, uint32_t& it, volatile int* abort_flag, int pw, int lane) {{
    static_assert(D < NSTAGE, "the ring must hold one chunk");
    constexpr int ROW = {d1t};
    const int q4 = lane & 7, rsub = lane >> 3;        // 16-byte column piece, row within a group of four rows
    constexpr int H = D <= 5 ? 4 : 2;        // items per pass and thread (4 D registers each); 8 items per thread and chunk
    constexpr int NPASS = 8 / H;
#pragma unroll
    for (int pass = 0; pass < NPASS; ++pass) {{
        float f[H][4 * D];
#pragma unroll
        for (int h = 0; h < H; ++h) {{
            const int r = pw * 32 + (pass * H + h) * 4 + rsub;
            int64_t z = z0 + r;
            if (z >= Z) z = Z - 1;
            const float4* p = reinterpret_cast<const float4*>(src + z * ROW + q4 * 4 * D);
#pragma unroll
            for (int m = 0; m < D; ++m) {{
                const float4 v = __ldg(p + m);
                f[h][4 * m] = v.x; f[h][4 * m + 1] = v.y; f[h][4 * m + 2] = v.z; f[h][4 * m + 3] = v.w;
            }}
        }}
        if (pass == 0) {{
            // the ring stages are waited for after the first loads are in flight: the wait overlaps their latency
#pragma unroll
            for (int i = 0; i < D; ++i) {{
                const uint32_t n = it + i;
                if (!tc::mbar_wait(&bar_empty[n % NSTAGE], ((n / NSTAGE) & 1u) ^ 1u, abort_flag)) return false;
            }}
        }}
#pragma unroll
        for (int h = 0; h < H; ++h) {{
            const int r = pw * 32 + (pass * H + h) * 4 + rsub;
            const uint32_t off = (r >> 3) * 1024 + (r & 7) * 128 + ((q4 ^ (r & 7)) << 4);
#pragma unroll
            for (int i = 0; i < D; ++i)
                *reinterpret_cast<float4*>(sA + ((it + i) % NSTAGE) * {TILE_BYTES} + off) =
                    make_float4(f[h][i], f[h][D + i], f[h][2 * D + i], f[h][3 * D + i]);
        }}
    }}
    tc::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {{
#pragma unroll
        for (int i = 0; i < D; ++i) tc::mbar_arrive(&bar_full[(it + i) % NSTAGE]);
    }}
    it += D;
    return true;
}}

{chr(10).join(consts)}
{''.join(funcs)}

__global__ void __launch_bounds__(kThreads, 1) uvw_post_kernel(const float* __restrict__ x1, const float* __restrict__ x2,
        const float* __restrict__ W, float* __restrict__ out, int64_t Z, CtaSplit split, int* status) {{
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle atoms of the MMA operands
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
{bounds_decl}
{dispatch}
}}

}}  // namespace

extern "C" int e3b_layout_info(int32_t* dims) {{
    dims[0] = {d1t}; dims[1] = {d2t}; dims[2] = {dout}; dims[3] = {spec.weight_numel}; dims[4] = -1; dims[5] = kThreads;
    return 0;
}}
extern "C" const char* e3b_layout_key(void) {{ return "{spec.key()}"; }}
extern "C" const char* e3b_layout_last_error(void) {{ return e3b_layout_error_buffer(); }}

// Relative cost of one 128-row tile per group: used to split the CTAs.
static const int kGroupWork[kGroups] = {{{', '.join(map(str, work))}}};

extern "C" int e3b_uvw_tc_fwd(const float* x1, const float* x2, const float* weight, float* out, int64_t Z,
                              int num_ctas, int32_t* status, void* stream) {{
    if (Z < 0) return e3b_layout_fail(-1, "uvw_tc_fwd: negative row count");
    if (Z == 0) return 0;
    if (!x1 || !x2 || !weight || !out || !status) return e3b_layout_fail(-1, "uvw_tc_fwd: null pointer");
    if (reinterpret_cast<uintptr_t>(out) % 16 != 0 || reinterpret_cast<uintptr_t>(x1) % 16 != 0)
        return e3b_layout_fail(-1, "uvw_tc_fwd: x1 and out must be 16-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
{zero_fill}
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
    if (const char* env = std::getenv("E3B_UVW_CTA_SPLIT")) {{
        // tuning aid: comma-separated CTA counts per group, in group order (all must be given and positive)
        int vals[kGroups], n = 0;
        const char* p = env;
        while (n < kGroups && *p) {{
            char* end = nullptr;
            const long v = std::strtol(p, &end, 10);
            if (end == p || v < 1 || v > 1024) break;
            vals[n++] = static_cast<int>(v);
            p = (*end == ',') ? end + 1 : end;
        }}
        if (n == kGroups) {{ used = 0; for (int g = 0; g < kGroups; ++g) {{ split.n[g] = vals[g]; used += vals[g]; }} }}
    }}
    cudaError_t err = cudaFuncSetAttribute(uvw_post_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (err != cudaSuccess) return e3b_layout_fail(-2, "uvw_tc_fwd: smem attribute: %s", cudaGetErrorString(err));
    uvw_post_kernel<<<used, kThreads, kSmemBytes, s>>>(x1, x2, weight, out, Z, split, status);
    return e3b_layout_check("uvw_tc_fwd");
}}
"""
