// Blackwell (sm_100a) primitives used by the tensor-core kernels: mbarriers with bounded
// waits, tcgen05 MMA / TMEM access, shared-memory matrix descriptors.  Inline PTX only.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "gate_act.cuh"

namespace tc {

using e3b::gate_act;    // activation codes of the Gate epilogue (csrc/gate_act.cuh)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One poll.  (A suspend-time hint on the try_wait, which parks the warp in hardware for up to that long, was measured:
// no effect on the kernels whose waiting warps share a scheduler with busy ones, and 4 - 12 % slower on the dense
// contractions, whose producers wake up later; the plain form stays.)
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls (or as soon as another thread of the block has
// raised *abort), raises *abort itself and returns false.  No wait in these kernels is unbounded.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort, uint32_t limit = 200000u) {
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 63u) {
            if (*abort) return false;
            __nanosleep(64);
        }
    }
    *abort = 1;
    return false;
}

// generic-proxy writes to shared memory -> visible to the async proxy (tcgen05.mma operand reads)
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 16-byte read-only global load that keeps its place among the other volatile statements (the software
// pipelines of the producers rely on the order in which loads are issued)
__device__ __forceinline__ float4 ld_nc_f4(const float4* p) {
    float4 v;
    asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

// ---------------------------------------------------------------- tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 lanes x 8 consecutive 32-bit columns: thread i of the warp receives lane (base_lane + i)
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
// 32 lanes x 4 consecutive 32-bit columns
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------- MMA
// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes packed in
// 8-row atoms of 1024 bytes (the atom base must be 1024-byte aligned).
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);      // start address
    d |= static_cast<uint64_t>(1) << 16;                        // leading byte offset (unused for this layout)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                // stride byte offset: next 8-row atom
    d |= static_cast<uint64_t>(1) << 46;                        // descriptor version (sm_100)
    d |= static_cast<uint64_t>(2) << 61;                        // SWIZZLE_128B
    return d;
}

// Instruction descriptor for kind::tf32, fp32 accumulate, both operands K-major, M = 128.
__host__ __device__ constexpr uint32_t idesc_tf32_m128(uint32_t n) {
    return (1u << 4)          // D format: F32
           | (2u << 7)        // A format: TF32
           | (2u << 10)       // B format: TF32
           | ((n >> 3) << 17) // N / 8
           | ((128u >> 4) << 24);  // M / 16
}

// D[tmem] (+)= A[smem] * B[smem]^T, one thread issues.
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// All MMAs of one 32-wide K chunk (4 k-steps of 8): operand pieces a_i * b_j with i + j < P, smallest
// magnitudes first; even / odd k-steps go to different partial accumulators when NACC == 2.
// adesc / bdesc: descriptors of piece 0 at k-step 0; other pieces / k-steps are constant address offsets.
// ACCW: columns between the partial accumulators of a buffer.
template <int P, int N, int NACC, uint32_t A_TILE, uint32_t B_HALF, int ACCW = N>
__device__ __forceinline__ void issue_chunk(uint32_t d_base, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool not_first_chunk) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
        const uint32_t d_tmem = d_base + (NACC == 2 ? (ks & 1) * ACCW : 0);
        uint32_t acc = (not_first_chunk || ks >= NACC) ? 1u : 0u;
#pragma unroll
        for (int deg = P - 1; deg >= 0; --deg) {
#pragma unroll
            for (int i = 0; i <= deg; ++i) {
                const int j = deg - i;
                mma_tf32(d_tmem, adesc + ((i * A_TILE + ks * 32) >> 4), bdesc + ((j * B_HALF + ks * 32) >> 4), idesc, acc);
                acc = 1u;
            }
        }
    }
}

// Two-piece split with two MMAs per k-step instead of three (N <= 128): the hi and lo pieces of B lie next to
// each other in the stage, so  a_hi x [b_hi | b_lo]  is ONE instruction of width 2N whose result columns
// [0, N) hold hi*hi and [N, 2N) hold hi*lo;  a_lo x b_hi  (width N) is added to the first half and the epilogue
// sums the halves.  Per k-step the tensor core reads A twice and B 1.5 times instead of three times each.
template <int N, int NACC, uint32_t A_TILE, uint32_t B_HALF>
__device__ __forceinline__ void issue_chunk_wide(uint32_t d_base, uint64_t adesc, uint64_t bdesc, uint32_t idesc_n,
                                                 uint32_t idesc_2n, bool not_first_chunk) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
        const uint32_t d_tmem = d_base + (NACC == 2 ? (ks & 1) * 2 * N : 0);
        const uint32_t acc = (not_first_chunk || ks >= NACC) ? 1u : 0u;
        mma_tf32(d_tmem, adesc + ((ks * 32) >> 4), bdesc + ((ks * 32) >> 4), idesc_2n, acc);
        mma_tf32(d_tmem, adesc + ((A_TILE + ks * 32) >> 4), bdesc + ((ks * 32) >> 4), idesc_n, 1u);
    }
}

// mbarrier arrive once every MMA issued so far by this thread has completed
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Round to the nearest tf32 (10 explicit mantissa bits) with two full-rate integer operations
// (round half away from zero in magnitude) instead of cvt.rna.tf32.f32, which issues on the
// low-throughput conversion pipe.  NaN stays NaN, values within 2^-11 of FLT_MAX round to infinity.
__device__ __forceinline__ float to_tf32(float x) {
    return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
}

// lo pieces of four raw fp32 values whose hi pieces are the values themselves (the tensor core reads only
// sign, exponent and the top 10 mantissa bits of a tf32 operand): lo = x - trunc(x), rounded to tf32
__device__ __forceinline__ float4 lo_piece4(float4 v) {
    return make_float4(to_tf32(v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u)),
                       to_tf32(v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u)),
                       to_tf32(v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u)),
                       to_tf32(v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u)));
}

// ---------------------------------------------------------------- tensor-map TMA (2-D tiles)
// One box of the tensor map -> shared memory (no multicast, this CTA only); completion as `bytes` on `bar`.
// x (innermost coordinate, in elements) times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int32_t x, int32_t y, uint64_t* bar,
                                            uint32_t bytes) {
    const uint32_t b = smem_u32(bar);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(b)
                 : "memory");
}

// Host: row-major fp32 matrix [rows, cols] (row stride = cols) as a 2-D tensor map with boxes of
// box_rows x box_cols, 128-byte swizzle, zero fill outside the matrix.  Returns 0 or a driver error code
// (-1: the driver entry point is not available).  The driver is reached through the runtime's entry-point
// query, so nothing links against libcuda.
inline int encode_tensor_map_2d(CUtensorMap* map, const float* base, int64_t cols, int64_t rows, uint32_t box_cols,
                                uint32_t box_rows) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || !p)
            return -1;
        fn = reinterpret_cast<EncodeFn>(p);
    }
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(cols) * sizeof(float)};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estride[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), gdim, gstride, box, estride,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return static_cast<int>(r);
}

// byte offset of element (row, col) in a K-major SWIZZLE_128B tile of 32 fp32 columns
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t col) {
    return (row >> 3) * 1024u + (row & 7u) * 128u + ((((col >> 2) ^ (row & 7u)) & 7u) << 4) + ((col & 3u) << 2);
}

}  // namespace tc
