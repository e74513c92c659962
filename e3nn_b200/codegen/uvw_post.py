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

Kernel structure (persistent, one CTA per SM, a CTA serves one *group* = one or more output irreps, or slabs of
their channels, whose accumulators fit the registers of the epilogue threads together):
  * prologue: for every input irrep ("block") of x1 the weight matrices of all paths that lead from it into the
    group lie side by side as ONE right operand of N <= 256 columns -> shared memory, rounded to tf32, K-major
    128-byte swizzle.  Paths that share an input block therefore share its left-operand tiles and its MMAs;
  * left-operand tiles, one ring stage = the 128 x 32 tile ``x1[z0 + r, block, 32 kc + u, i]`` (component i, 32
    channels).  Blocks of scalars need no de-interleaving: one thread issues a tensor-map TMA copy per stage.  For
    the other blocks 4 producer warps fill the 2 l1 + 1 component tiles of a chunk together from one contiguous
    run of each input row (16-byte streaming loads in, 16-byte swizzled stores out);
  * one thread issues ``tcgen05.mma.kind::tf32`` (M = 128, N = the block's columns, K = 8).  A *job* is what the
    epilogue receives as a whole: one component of a block when the block has a single 32-channel chunk (or a
    single component), else all components of the block (the producers deliver chunk by chunk, so all component
    accumulators are live).  Tensor memory is a ring of equal slots; the issuing thread runs ahead of the epilogue
    by as many jobs as there are free slots, which also releases the ring stages of later jobs early;
  * 8 epilogue warps (two per lane quarter, each owning half of every member's channels) compute t(z) from the x2
    row, read the accumulators with ``tcgen05.ld``, keep their part of ``out[z, :]`` in registers across the jobs
    of the tile and write it once through a per-warp staging tile, as 64-byte row segments with streaming stores.
Register budget: the kernel is compiled for 128 registers per thread (512 threads); the epilogue and producer
warpgroups raise their limit with ``setmaxnreg``, the issue warpgroup lowers its own.
Every mbarrier wait is bounded; a wait that gives up sets the block's abort flag and status 3.

Eligibility: every live path 'uvw' with shared weights, x2 multiplicities 1, x1 multiplicities multiples of 32,
output multiplicities multiples of 16, output rows, input rows and block offsets multiples of four floats.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np

from ..o3._spec import TPSpec
from ..o3._wigner import wigner_3j_numpy

SMEM_LIMIT = 227 * 1024
TILE_BYTES = 128 * 128          # 128 rows x 32 tf32
TMEM_COLS = 512
STAGING_BYTES = 8 * 2048        # output staging tile of 32 rows x 16 floats per epilogue warp
MAX_ACC_REGS = 96               # accumulator registers of an epilogue thread: sum over members of (width / 2) * (2 l3 + 1)
MAX_N = 256                     # columns of one MMA instruction (M = 128)


def _f(v: float) -> str:
    return f"{np.float32(v):.9e}f"


@dataclass
class Member:
    """An output irrep (or a slab of its channels) whose rows a group computes."""
    i_out: int
    l3: int
    nfull: int          # output multiplicity
    col0: int           # first channel of the slab
    width: int          # channels of the slab
    out_off: int        # output column of channel col0, component 0
    acc_off: int = 0    # first accumulator register of an epilogue thread

    @property
    def d3(self) -> int:
        return 2 * self.l3 + 1

    @property
    def half(self) -> int:
        return self.width // 2


@dataclass
class Path:
    index: int          # instruction index
    l2: int
    off2: int           # x2 column of the path's second operand
    woff: int           # weight offset of W_p[0, col0]
    pw: float
    member: int         # index into Group.members
    coloff: int = 0     # first accumulator column of the path within its block's N columns


@dataclass
class Block:
    """An input irrep of x1 with the paths that lead from it into the group's members.  All those paths share the
    left operand, so their weight matrices lie side by side as ONE right operand of ``ncols`` columns."""
    i_in1: int
    l1: int
    mul1: int
    off1: int           # x1 column of the block
    paths: List[Path] = field(default_factory=list)
    ncols: int = 0
    boff: int = 0       # byte offset of the block's weight tiles in the resident B area

    @property
    def d1(self) -> int:
        return 2 * self.l1 + 1

    @property
    def nchunk(self) -> int:
        return self.mul1 // 32

    @property
    def live(self) -> bool:
        """True: the 2 l1 + 1 component accumulators are live together (one job); False: one job per component.
        The producers emit the component tiles of a 32-channel chunk together, so components can only be separate
        jobs when a block has a single chunk (or a single component)."""
        return self.d1 > 1 and self.nchunk > 1


@dataclass
class Job:
    """A run of ring stages accumulated into a range of tensor-memory slots and handed to the epilogue as a whole."""
    block: int
    comps: List[int]    # components of the block whose accumulators the job holds (ncols columns each)
    nchunk: int
    slot0: int = 0      # first slot; the job's barriers are those of this slot
    nslot: int = 1
    use_idx: int = 0    # this job is the use_idx-th job of a tile whose first slot is slot0
    # completions of earlier jobs the issuing thread must have seen before it may overwrite the job's slots:
    # (barrier = first slot of that job, its use_idx, True when that job belongs to the previous row tile)
    waits: List[Tuple[int, int, bool]] = field(default_factory=list)

    def cols(self, blocks: List[Block]) -> int:
        return len(self.comps) * blocks[self.block].ncols


@dataclass
class Group:
    members: List[Member]
    blocks: List[Block] = field(default_factory=list)
    jobs: List[Job] = field(default_factory=list)
    slot_cols: int = 128        # tensor memory is handed out in slots of this many columns
    nslots: int = 4
    uses: List[int] = field(default_factory=list)   # per slot: jobs of a tile whose first slot it is

    def nacc(self) -> int:
        return sum(m.half * m.d3 for m in self.members)

    def b_bytes(self) -> int:
        return sum(b.mul1 * b.ncols * 4 for b in self.blocks)

    def nstage(self) -> int:
        return int(max(0, min(8, (SMEM_LIMIT - 2048 - STAGING_BYTES - self.b_bytes()) // TILE_BYTES)))

    def smem_bytes(self) -> int:
        return self.b_bytes() + self.nstage() * TILE_BYTES + STAGING_BYTES + 1024 + 1024

    def tiles_per_row_tile(self) -> int:
        return sum(b.d1 * b.nchunk for b in self.blocks)

    def fma_per_row(self) -> int:
        fma = 0
        for b in self.blocks:
            for p in b.paths:
                m = self.members[p.member]
                c = wigner_3j_numpy(b.l1, p.l2, m.l3)
                fma += int((np.abs(c).sum(axis=1) != 0).sum()) * m.width
        return fma

    def work(self) -> int:
        """Relative cost of one 128-row tile: producer instructions (tiles) plus epilogue multiply-adds."""
        return 100 * self.tiles_per_row_tile() + self.fma_per_row() // 16


def _plan_group(spec: TPSpec, members: List[Member]) -> Optional[Group]:
    """Blocks, jobs and tensor-memory slots of a group, or None when it does not fit."""
    live = spec.live_instructions()
    o1, o2 = spec.irreps_in1.offsets(), spec.irreps_in2.offsets()
    woffs = spec.weight_offsets()
    g = Group(members=[Member(m.i_out, m.l3, m.nfull, m.col0, m.width, m.out_off) for m in members])
    acc = 0
    for m in g.members:
        m.acc_off = acc
        acc += m.half * m.d3
        if m.out_off % 4 != 0 or (m.half * m.d3) % 4 != 0 or m.half % 8 != 0:
            return None
    if acc > MAX_ACC_REGS:
        return None
    by_block: Dict[int, Block] = {}
    for n, ins in live:
        for mi, m in enumerate(g.members):
            if ins.i_out != m.i_out:
                continue
            (m1, ir1), (_, ir2) = spec.irreps_in1[ins.i_in1], spec.irreps_in2[ins.i_in2]
            b = by_block.setdefault(ins.i_in1, Block(ins.i_in1, ir1.l, m1, o1[ins.i_in1]))
            b.paths.append(Path(n, ir2.l, o2[ins.i_in2], woffs[n] + m.col0, float(ins.path_weight), mi))
    if not by_block:
        return None
    boff = 0
    for i_in1 in sorted(by_block):
        b = by_block[i_in1]
        col = 0
        for p in b.paths:
            p.coloff = col
            col += g.members[p.member].width
        b.ncols, b.boff = col, boff
        boff += b.mul1 * b.ncols * 4
        if b.ncols > MAX_N or b.ncols % 16 != 0:
            return None
        g.blocks.append(b)
    jobs: List[Job] = []
    for bi, b in enumerate(g.blocks):
        if b.live or b.d1 == 1:
            jobs.append(Job(bi, list(range(b.d1)), b.nchunk))
        else:
            jobs.extend(Job(bi, [i], 1) for i in range(b.d1))
    # Tensor memory as a ring of equal slots: a single-component job takes one slot, a job that holds all components
    # of a block takes as many as it needs.  The issuing thread runs ahead of the epilogue by as many jobs as there
    # are free slots, so the ring stages of later jobs are consumed (and released to the producers) while the
    # epilogue is still busy with an earlier, larger job.
    single = [j.cols(g.blocks) for j in jobs if len(j.comps) == 1]
    w = -(-max(single) // 32) * 32 if single else 128
    nslots = min(8, TMEM_COLS // w)
    pos = 0
    uses = [0] * nslots
    for j in jobs:
        k = -(-j.cols(g.blocks) // w)
        if k > nslots:
            return None
        if pos + k > nslots:
            pos = 0
        j.slot0, j.nslot = pos, k
        j.use_idx = uses[pos]
        uses[pos] += 1
        pos += k
    g.slot_cols, g.nslots, g.uses = w, nslots, uses
    # who held a slot last, over two consecutive tiles (the schedule repeats per tile)
    occupant: List[Optional[Tuple[int, int]]] = [None] * nslots       # (job index, tile)
    seen = set()
    for tile in (0, 1):
        for ji, j in enumerate(jobs):
            waits = []
            for sl in range(j.slot0, j.slot0 + j.nslot):
                o = occupant[sl]
                if o is not None and o not in seen:
                    seen.add(o)
                    waits.append((jobs[o[0]].slot0, jobs[o[0]].use_idx, o[1] != tile))
                occupant[sl] = (ji, tile)
            if tile == 1:
                j.waits = waits     # on a CTA's first tile the entries of the previous tile are skipped at run time
    g.jobs = jobs
    if g.nstage() < max(b.d1 for b in g.blocks) + 1:
        return None
    return g


def plan_groups(spec: TPSpec) -> Optional[List[Group]]:
    """Groups of an eligible spec, or None when the layout does not fit this kernel."""
    if not spec.shared_weights:
        return None
    live = spec.live_instructions()
    if not live or any(ins.connection_mode != "uvw" for _, ins in live):
        return None
    if spec.irreps_in2.dim > 32 or spec.irreps_out.dim % 4 != 0 or spec.irreps_in1.dim % 4 != 0:
        return None
    o1, oo = spec.irreps_in1.offsets(), spec.irreps_out.offsets()
    for _, ins in live:
        (m1, _), (m2, _), (mo, _) = spec.irreps_in1[ins.i_in1], spec.irreps_in2[ins.i_in2], spec.irreps_out[ins.i_out]
        if m2 != 1 or m1 % 32 != 0 or mo % 16 != 0 or o1[ins.i_in1] % 4 != 0:
            return None
    groups: List[Group] = []
    for i_out in sorted({ins.i_out for _, ins in live}):
        mo, iro = spec.irreps_out[i_out]
        planned = None
        for s in (mo, mo // 2, mo // 4, mo // 8):
            if s < 16 or s % 16 != 0 or mo % s != 0:
                continue
            trial = [_plan_group(spec, [Member(i_out, iro.l, mo, col0, s, oo[i_out] + col0 * iro.dim)]) for col0 in range(0, mo, s)]
            if all(t is not None for t in trial):
                planned = trial
                break
        if planned is None:
            return None
        groups.extend(planned)
    # neighbouring groups whose accumulators fit one thread together share their left-operand tiles
    merged = True
    while merged:
        merged = False
        for a in range(len(groups) - 1):
            both = _plan_group(spec, groups[a].members + groups[a + 1].members)
            if both is not None:
                groups[a:a + 2] = [both]
                merged = True
                break
    return groups


def _indent(text: str, n: int) -> str:
    pad = " " * n
    return "\n".join(pad + line if line and not line.startswith("#pragma") else line for line in text.split("\n"))


def _epilogue_block_code(g: Group, gi: int, bi: int) -> Tuple[str, List[str]]:
    """Epilogue of all jobs of one input block as a loop over the block's components, for the thread that owns (row z,
    half h of every member's channels).  The body is the same for every component: t_k(z) = sum_j C[i, j, k] x2[z, j]
    with the coefficients of component i read from constant memory, then ``acc[w, k] += t_k V_i[w]`` for all k (the
    accumulator registers depend on (w, k) only).  Unrolling over the components instead (with the zero coefficients
    left out) is straight-line code of 800 - 2,000 instructions per row tile and thread, more than the instruction
    cache holds for the two epilogue warps of a scheduler.  Returns (code, constant tables).
    In scope: x2r[], acc[], lbase (tensor-memory address of this thread's lane, column 0), h, tcount, ok."""
    b = g.blocks[bi]
    jobs = [j for j in g.jobs if j.block == bi]
    consts: List[str] = []
    body = []
    for pi, p in enumerate(b.paths):
        m = g.members[p.member]
        c = wigner_3j_numpy(b.l1, p.l2, m.l3) * p.pw              # [d1, d2, d3]
        d2, d3 = 2 * p.l2 + 1, m.d3
        name = f"kC{gi}_{bi}_{pi}"
        consts.append(f"__constant__ float {name}[{b.d1 * d2 * d3}] = {{{', '.join(_f(v) for v in c.reshape(-1))}}};")
        step = 32 if m.half % 32 == 0 else (16 if m.half % 16 == 0 else 8)
        lines = [f"{{   // path {p.index}: l={b.l1} (x) l={p.l2} -> l={m.l3}", f"    float tk[{d3}];"]
        tk_lines = []
        for k in range(d3):
            expr = " + ".join(f"{name}[(i * {d2} + {jj}) * {d3} + {k}] * x2r[{p.off2 + jj}]" for jj in range(d2))
            tk_lines.append(f"        if (w0 == 0) tk[{k}] = {expr};")
        lines.append(f"    const uint32_t cb = jb + {p.coloff} + h * {m.half};")
        lines.append("#pragma unroll")
        lines.append(f"    for (int w0 = 0; w0 < {m.half}; w0 += {step}) {{")
        for part in range(step // 8):
            lines.append(f"        uint32_t v{part}[8];")
            lines.append(f"        tc::tmem_ld8(cb + w0 + {part * 8}, v{part});")
        lines.extend(tk_lines)      # the coefficients are formed while the first accumulator loads are in flight
        lines.append("        tc::tmem_ld_wait();")
        for part in range(step // 8):
            lines.append("#pragma unroll")
            lines.append("        for (int c = 0; c < 8; ++c) {")
            for k in range(d3):
                a = f"acc[{m.acc_off} + (w0 + {part * 8} + c) * {d3} + {k}]"
                lines.append(f"            {a} = fmaf(tk[{k}], __uint_as_float(v{part}[c]), {a});")
            lines.append("        }")
        lines.append("    }")
        lines.append("}")
        body.append("\n".join(lines))
    body_code = "\n".join(body)
    head = f"// block {b.i_in1} (l = {b.l1}, {b.mul1} channels)"
    if len(jobs) == 1:
        j = jobs[0]
        code = f"""{head}: one job, slots [{j.slot0}, {j.slot0 + j.nslot})
{{
    constexpr int r = {j.slot0};
    if (!tc::mbar_wait(&bar_reg_full[r], (tcount * {g.uses[j.slot0]}u + {j.use_idx}u) & 1u, abort_flag)) {{ ok = false; break; }}
    tc::tc_fence_after_sync();
#pragma unroll 1
    for (int i = 0; i < {b.d1}; ++i) {{
        const uint32_t jb = lbase + {j.slot0 * g.slot_cols} + i * {b.ncols};
{_indent(body_code, 8)}
    }}
    tc::tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(&bar_reg_empty[r]);
}}"""
    else:
        arr = lambda nm, vals: f"__constant__ int {nm}{gi}_{bi}[{len(vals)}] = {{{', '.join(str(v) for v in vals)}}};"
        consts.append(arr("kESlot", [j.slot0 for j in jobs]))
        consts.append(arr("kEUses", [g.uses[j.slot0] for j in jobs]))
        consts.append(arr("kEIdx", [j.use_idx for j in jobs]))
        code = f"""{head}: one job per component
#pragma unroll 1
for (int i = 0; i < {b.d1}; ++i) {{
    const int r = kESlot{gi}_{bi}[i];
    if (!tc::mbar_wait(&bar_reg_full[r], (tcount * kEUses{gi}_{bi}[i] + kEIdx{gi}_{bi}[i]) & 1u, abort_flag)) {{ ok = false; break; }}
    tc::tc_fence_after_sync();
    const uint32_t jb = lbase + r * {g.slot_cols};
{_indent(body_code, 4)}
    tc::tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(&bar_reg_empty[r]);
}}
if (!ok) break;"""
    return code, consts


def emit_module(spec: TPSpec) -> str:
    groups = plan_groups(spec)
    assert groups is not None, "layout not eligible for the tensor-core kernel"
    d1t, d2t, dout = spec.irreps_in1.dim, spec.irreps_in2.dim, spec.irreps_out.dim
    smem_max = max(g.smem_bytes() for g in groups)
    assert smem_max <= SMEM_LIMIT

    consts, funcs = [], []
    for gi, g in enumerate(groups):
        nb = len(g.blocks)
        paths = [(b, p) for b in g.blocks for p in b.paths]
        npth = len(paths)
        arr = lambda name, vals: f"__constant__ int {name}{gi}[{len(vals)}] = {{{', '.join(str(v) for v in vals)}}};"
        consts.append("\n".join([
            # per block (producers)
            arr("kBXoff", [b.off1 for b in g.blocks]),
            arr("kBD1", [b.d1 for b in g.blocks]),
            arr("kBNchunk", [b.nchunk for b in g.blocks]),
            # per path (weight prologue)
            arr("kPWoff", [p.woff for b, p in paths]),
            arr("kPMul1", [b.mul1 for b, p in paths]),
            arr("kPBoff", [b.boff for b, p in paths]),
            arr("kPNcols", [b.ncols for b, p in paths]),
            arr("kPColoff", [p.coloff for b, p in paths]),
            arr("kPWidth", [g.members[p.member].width for b, p in paths]),
            arr("kPNfull", [g.members[p.member].nfull for b, p in paths]),
        ]))
        nacc = g.nacc()
        blocks_code = []
        for bi in range(len(g.blocks)):
            code, tables = _epilogue_block_code(g, gi, bi)
            blocks_code.append(code)
            consts.append("\n".join(tables))
        epi_code = "\n".join(blocks_code)
        mma_jobs = []
        for ji, j in enumerate(g.jobs):
            b = g.blocks[j.block]
            waits = []
            for bar, idx, prev in j.waits:
                if prev:
                    waits.append(f"    if (tcount > 0u && !tc::mbar_wait(&bar_reg_empty[{bar}], ((tcount - 1u) * {g.uses[bar]}u + {idx}u) & 1u, abort_flag)) {{ ok = false; break; }}")
                else:
                    waits.append(f"    if (!tc::mbar_wait(&bar_reg_empty[{bar}], (tcount * {g.uses[bar]}u + {idx}u) & 1u, abort_flag)) {{ ok = false; break; }}")
            wait_code = "\n".join(waits)
            mma_jobs.append(f"""{{   // job {ji}: block {b.i_in1}, components {j.comps}, slots [{j.slot0}, {j.slot0 + j.nslot})
{wait_code}
    tc::tc_fence_after_sync();
    constexpr int ncomp = {len(j.comps)}, nchunk = {j.nchunk}, ncols = {b.ncols};
    const uint32_t d0 = tmem_base + {j.slot0 * g.slot_cols}u;
    constexpr uint32_t idesc = tc::idesc_tf32_m128({b.ncols}u);
    const uint64_t bdesc0 = tc::smem_desc_k_sw128(tc::smem_u32(sB + {b.boff}));
    for (int kc = 0; kc < nchunk && ok; ++kc) {{
        const uint64_t bdesc = bdesc0 + static_cast<uint64_t>(kc) * ((ncols * 128) >> 4);
        for (int c = 0; c < ncomp; ++c, ++it) {{
            const int s = it % NSTAGE;
            const uint32_t ph = (it / NSTAGE) & 1;
            if (!tc::mbar_wait(&bar_full[s], ph, abort_flag)) {{ ok = false; break; }}
            tc::tc_fence_after_sync();
            const uint64_t adesc = tc::smem_desc_k_sw128(tc::smem_u32(sA + s * TILE));
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
                tc::mma_tf32(d0 + c * ncols, adesc + ((ks * 32) >> 4), bdesc + ((ks * 32) >> 4), idesc, (kc > 0 || ks > 0) ? 1u : 0u);
            tc::mma_commit(&bar_empty[s]);
        }}
    }}
    if (!ok) break;
    tc::mma_commit(&bar_reg_full[{j.slot0}]);
}}""")
        mma_code = "\n".join(mma_jobs)
        # The thread that owns row z holds a contiguous run of each member's output row.  Stored directly, one
        # instruction would touch 32 rows; the runs go through a per-warp staging tile of 32 rows x 16 floats instead
        # (16-byte pieces, XOR-swizzled so that neither side has bank conflicts) and leave as 64-byte row segments,
        # eight rows per instruction.
        stores = []
        for m in g.members:
            n = m.half * m.d3
            for c0 in range(0, n, 16):
                wd = min(16, n - c0)
                P = wd // 4
                lines = [f"                {{   // member irrep {m.i_out}: floats [{c0}, {c0 + wd}) of the thread's run of {n}"]
                for pc in range(P):
                    a = m.acc_off + c0 + 4 * pc
                    lines.append(f"                    *reinterpret_cast<float4*>(stg + lane * 16 + (({pc} ^ ((lane >> 1) & 3)) << 2)) = "
                                 f"make_float4(acc[{a}], acc[{a + 1}], acc[{a + 2}], acc[{a + 3}]);")
                lines.append("                    __syncwarp();")
                lines.append("#pragma unroll")
                lines.append(f"                    for (int it = 0; it < {P}; ++it) {{")
                lines.append(f"                        const int idx = it * 32 + lane, rr = idx / {P}, pc = idx - rr * {P};")
                lines.append("                        const float4 v = *reinterpret_cast<const float4*>(stg + rr * 16 + ((pc ^ ((rr >> 1) & 3)) << 2));")
                lines.append(f"                        if (zw + rr < Z) __stcs(reinterpret_cast<float4*>(out + (zw + rr) * {dout} + {m.out_off + c0} + h * {n} + pc * 4), v);")
                lines.append("                    }")
                lines.append("                    __syncwarp();")
                lines.append("                }")
                stores.append("\n".join(lines))
        store_code = "\n".join(stores)
        producer_cases = "\n".join(
            f"                    case {d}: ok = produce_group<{d}, NSTAGE>(src, z0, Z, sA, bar_full, bar_empty, it, abort_flag, pw, lane); break;"
            for d in sorted({b.d1 for b in g.blocks}) if d > 1)
        if any(b.d1 == 1 for b in g.blocks):
            # a block of scalars needs no de-interleaving: its 128 x 32 tile is one tensor-map copy (128-byte swizzle,
            # rows past the end read as zero) issued by one thread, which also makes the arrivals of all producer warps
            producer_cases += f"""
                    case 1:
                        if (pw == 0) {{
                            if (lane == 0) {{
                                const int s = it % NSTAGE;
                                if (tc::mbar_wait(&bar_empty[s], ((it / NSTAGE) & 1u) ^ 1u, abort_flag))
                                    tma_tile_to_stage(sA + s * TILE, tmap_x1, kBXoff{gi}[b] + kc * 32, static_cast<int32_t>(z0), &bar_full[s]);
                                else
                                    ok = false;
                            }}
                            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                        }}
                        ++it;
                        break;"""
        desc = ", ".join(f"irrep {m.i_out} (l = {m.l3}) channels [{m.col0}, {m.col0 + m.width}) of {m.nfull}" for m in g.members)
        funcs.append(f"""
// ---------------------------------------------------------------- group {gi}: {desc}
__device__ __forceinline__ void run_group_{gi}(const float* __restrict__ x1, const float* __restrict__ x2,
        const float* __restrict__ W, float* __restrict__ out, int64_t Z, int cta, int nctas, uint8_t* smem, int* status,
        const CUtensorMap* tmap_x1) {{
    constexpr int NBLOCK = {nb}, NPATH = {npth}, NSTAGE = {g.nstage()};
    constexpr uint32_t B_BYTES = {g.b_bytes()}, TILE = {TILE_BYTES};
    constexpr int NSLOT = {g.nslots};                      // tensor memory in slots of {g.slot_cols} columns
    uint8_t* sB = smem;
    uint8_t* sA = smem + B_BYTES;
    uint8_t* sStage = sA + NSTAGE * TILE;             // output staging: 2 KB per epilogue warp
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(sStage + kEpilogueWarps * 2048);
    uint64_t* bar_empty = bar_full + NSTAGE;
    uint64_t* bar_reg_full = bar_empty + NSTAGE;      // [NSLOT] accumulators of the job whose first slot this is are complete
    uint64_t* bar_reg_empty = bar_reg_full + NSLOT;   // [NSLOT] the epilogue has read them
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_reg_empty + NSLOT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* tile_progress = abort_flag + 1;     // row tiles the producers have started

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- prologue: the weight matrices of the paths that leave one input block lie side by side as the block's
    // right operand -> shared memory (tf32, K-major, 128-byte swizzle; row = accumulator column)
    for (int p = 0; p < NPATH; ++p) {{
        const int width = kPWidth{gi}[p], total = kPMul1{gi}[p] * width;
        for (int idx = tid; idx < total; idx += kThreads) {{
            const int u = idx / width, w = idx - u * width;
            const float v = W[kPWoff{gi}[p] + u * kPNfull{gi}[p] + w];
            *reinterpret_cast<float*>(sB + kPBoff{gi}[p] + (u >> 5) * (kPNcols{gi}[p] * 128) + tc::sw128_offset(kPColoff{gi}[p] + w, u & 31)) = tc::to_tf32(v);
        }}
    }}
    if (tid == 0) {{
        *abort_flag = 0;
        *tile_progress = 0;
        for (int s = 0; s < NSTAGE; ++s) {{ tc::mbar_init(&bar_full[s], kProducerWarps); tc::mbar_init(&bar_empty[s], 1); }}
        for (int r = 0; r < NSLOT; ++r) {{ tc::mbar_init(&bar_reg_full[r], 1); tc::mbar_init(&bar_reg_empty[r], kEpilogueWarps); }}
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
        const int q = warp & 3, h = warp >> 2;          // lane quarter of tensor memory, half of every member's channels
        const uint32_t lbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        float* stg = reinterpret_cast<float*>(sStage + warp * 2048);
        uint32_t tcount = 0u;                   // row tiles of this CTA so far (barrier phases follow from it)
        bool ok = true;
        float x2r[{d2t}];
        {{
            const int64_t z = cta * 128 + q * 32 + lane;
#pragma unroll
            for (int j = 0; j < {d2t}; ++j) x2r[j] = (cta < tiles && z < Z) ? x2[z * {d2t} + j] : 0.0f;
        }}
        for (int64_t t = cta; t < tiles && ok; t += nctas, ++tcount) {{
            float acc[{nacc}];
#pragma unroll
            for (int a = 0; a < {nacc}; ++a) acc[a] = 0.0f;
            do {{
{_indent(epi_code, 16)}
            }} while (false);
            {{
                // the x2 row of this CTA's next row tile is requested before the store phase, which hides its latency
                const int64_t zn = (t + nctas) * 128 + q * 32 + lane;
#pragma unroll
                for (int j = 0; j < {d2t}; ++j) x2r[j] = (t + nctas < tiles && zn < Z) ? x2[zn * {d2t} + j] : 0.0f;
            }}
            if (ok) {{
                const int64_t zw = t * 128 + q * 32;        // first row of this warp
{store_code}
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
            for (int b = 0; b < NBLOCK && ok; ++b) {{
                const int d1 = kBD1{gi}[b], nchunk = kBNchunk{gi}[b];
                for (int kc = 0; kc < nchunk && ok; ++kc) {{
                    const float* src = x1 + kBXoff{gi}[b] + kc * 32 * d1;
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
            // ================= MMA issue (single thread): a job's stages arrive chunk by chunk, within a chunk
            // component by component; component c of the job accumulates into columns [c N, (c + 1) N) of its slots
            uint32_t it = 0;
            uint32_t tcount = 0u;
            bool ok = true;
            for (int64_t t = cta; t < tiles && ok; t += nctas, ++tcount) {{
                do {{
{_indent(mma_code, 20)}
                }} while (false);
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
        f"    {'else ' if gi else ''}if (blockIdx.x < cta_end{gi}) run_group_{gi}(x1, x2, W, out, Z, blockIdx.x - cta_begin{gi}, cta_end{gi} - cta_begin{gi}, smem, status, &tmap_x1);"
        for gi in range(ngroups))
    bounds_decl = "\n".join(
        f"    const int cta_begin{gi} = {'0' if gi == 0 else f'cta_end{gi-1}'}, cta_end{gi} = cta_begin{gi} + split.n[{gi}];" for gi in range(ngroups))
    work = [g.work() for g in groups]
    written = {m.i_out for g in groups for m in g.members}
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
constexpr int kEpilogueRegs = 152, kProducerRegs = 152, kIssueRegs = 56;   // 32 x (8 x 152 + 4 x 152 + 4 x 56) = 65536 = 512 x 128 registers
constexpr int kTmemCols = 512;
constexpr int kGroups = {ngroups};
constexpr int kSmemBytes = {smem_max};

struct CtaSplit {{ int n[kGroups]; }};

// One chunk: rows z0 .. z0 + 127 of 32 channels of an input block with D = 2 l1 + 1 components, i.e. 32 D
// contiguous floats per row, into D consecutive ring stages (stage i = component i as a 128 x 32 K-major tile).
// A thread owns (row, 4 channels) items: D 16-byte loads (element (channel e, component i) at float e D + i), then
// one 16-byte store per component.  The raw fp32 values are stored: the tensor core reads the top 19 bits of a
// tf32 operand (truncation; the weights are rounded to nearest in the prologue).  src: x1 + block offset + 32 kc D.
// One 128 x 32 tile of the tensor map -> a ring stage; the issuing thread arrives for every producer warp, the
// copy completes the phase through its byte count.  x: first column (a multiple of four floats), y: first row.
__device__ __forceinline__ void tma_tile_to_stage(void* dst, const CUtensorMap* map, int32_t x, int32_t y, uint64_t* bar) {{
    const uint32_t b = tc::smem_u32(bar);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"({TILE_BYTES}) : "memory");
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(kProducerWarps - 1) : "memory");
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {{%2, %3}}], [%4];"
                 ::"r"(tc::smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(b)
                 : "memory");
}}

template <int D, int NSTAGE>
__device__ __forceinline__ bool produce_group(const float* __restrict__ src, int64_t z0, int64_t Z, uint8_t* sA,
        uint64_t* bar_full, uint64_t* bar_empty, uint32_t& it, volatile int* abort_flag, int pw, int lane) {{
    static_assert(D < NSTAGE, "the ring must hold one chunk");
    constexpr int ROW = {d1t};
    const int q4 = lane & 7, rsub = lane >> 3;        // 16-byte column piece, row within a group of four rows
    constexpr int H = D <= 3 ? 8 : (D <= 5 ? 4 : 2);        // items per pass and thread (4 D registers each); 8 items per thread and chunk
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
                const float4 v = __ldcs(p + m);      // streaming: a row tile is read once per group
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
        const float* __restrict__ W, float* __restrict__ out, int64_t Z, CtaSplit split, int* status,
        const __grid_constant__ CUtensorMap tmap_x1) {{
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
    CUtensorMap tmap_x1;
    if (Z > 0x7fffffffLL) return e3b_layout_fail(-1, "uvw_tc_fwd: more than 2^31 - 1 rows");
    const int enc = tc::encode_tensor_map_2d(&tmap_x1, x1, {d1t}, Z, 32, 128);
    if (enc != 0) return e3b_layout_fail(-2, "uvw_tc_fwd: cuTensorMapEncodeTiled failed (%d)", enc);
    cudaError_t err = cudaFuncSetAttribute(uvw_post_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (err != cudaSuccess) return e3b_layout_fail(-2, "uvw_tc_fwd: smem attribute: %s", cudaGetErrorString(err));
    uvw_post_kernel<<<used, kThreads, kSmemBytes, s>>>(x1, x2, weight, out, Z, split, status, tmap_x1);
    return e3b_layout_check("uvw_tc_fwd");
}}
"""
