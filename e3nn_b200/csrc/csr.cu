// Destination-sorted CSR of an edge list: stable LSD radix sort of (dst, edge id) + row pointers.
//
// Integer, HBM-bound work.  Keys are the destination ids (range-checked, < 2^31), values the
// edge ids; 8-bit digits, ceil(bits(num_nodes-1)/8) passes.  A pass is three launches:
//   1. per-block digit histogram            -> hist[digit][block]
//   2. exclusive scan over hist (one block) -> global base of every (digit, block)
//   3. stable scatter: inside a block the keys are ranked round by round (round-major order,
//      lane order inside a round via __match_any_sync), so equal keys keep their input order.
// Row pointers come from a histogram of dst and a single-block exclusive scan.
// The result is bit-identical to argsort(dst, stable=True) / cumsum(bincount(dst)).
#include "common.cuh"
#include "scan.cuh"

#include <mutex>

namespace e3b {

constexpr int kSortThreads = 256;
constexpr int kSortItems = 8;                          // keys per thread per block
constexpr int kSortChunk = kSortThreads * kSortItems;  // 2048 keys per block
constexpr int kRadix = 256;

struct CsrScratch {
    uint32_t* keys[2];
    uint32_t* vals[2];
    uint32_t* hist;    // [kRadix * nblocks]
    int32_t* counts;   // [num_nodes]
    int64_t nblocks;
};

__host__ inline int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

__host__ int64_t csr_layout(int64_t E, int64_t N, char* base, CsrScratch* out) {
    const int64_t nblocks = ceil_div(E > 0 ? E : 1, kSortChunk);
    int64_t off = 0;
    auto take = [&](int64_t bytes) {
        char* p = base ? base + off : nullptr;
        off += align256(bytes);
        return p;
    };
    char* k0 = take(E * 4); char* k1 = take(E * 4);
    char* v0 = take(E * 4); char* v1 = take(E * 4);
    char* h = take(kRadix * nblocks * 4);
    char* c = take(N * 4);
    if (out) {
        out->keys[0] = reinterpret_cast<uint32_t*>(k0); out->keys[1] = reinterpret_cast<uint32_t*>(k1);
        out->vals[0] = reinterpret_cast<uint32_t*>(v0); out->vals[1] = reinterpret_cast<uint32_t*>(v1);
        out->hist = reinterpret_cast<uint32_t*>(h);
        out->counts = reinterpret_cast<int32_t*>(c);
        out->nblocks = nblocks;
    }
    return off;
}

// dst (int64) -> 32-bit keys + identity values; counts[dst]++ ; out-of-range -> status.
__global__ void csr_prepare_kernel(const int64_t* __restrict__ dst, int64_t E, int64_t N, uint32_t* __restrict__ keys,
                                   uint32_t* __restrict__ vals, int32_t* __restrict__ counts, int32_t* status) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < E; e += stride) {
        const int64_t d = dst[e];
        if (d < 0 || d >= N) {
            atomicExch(status, 1);
            keys[e] = 0; vals[e] = static_cast<uint32_t>(e);
            continue;
        }
        keys[e] = static_cast<uint32_t>(d);
        vals[e] = static_cast<uint32_t>(e);
        atomicAdd(&counts[d], 1);
    }
}


__global__ void __launch_bounds__(kSortThreads) radix_hist_kernel(const uint32_t* __restrict__ keys, int64_t E, int shift,
                                                                  uint32_t* __restrict__ hist, int64_t nblocks) {
    __shared__ uint32_t h[kRadix];
    h[threadIdx.x] = 0;
    __syncthreads();
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kSortChunk;
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {
        const int64_t i = base + r * kSortThreads + threadIdx.x;
        if (i < E) atomicAdd(&h[(keys[i] >> shift) & 0xffu], 1u);
    }
    __syncthreads();
    hist[static_cast<int64_t>(threadIdx.x) * nblocks + blockIdx.x] = h[threadIdx.x];
}

// Exclusive scan of hist[kRadix * nblocks] in place (digit-major), one block of 1024 threads.
__global__ void __launch_bounds__(1024) radix_scan_kernel(uint32_t* __restrict__ hist, int64_t total) {
    __shared__ uint32_t warp_sums[32];
    __shared__ uint32_t carry;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    if (t == 0) carry = 0;
    __syncthreads();
    for (int64_t base = 0; base < total; base += 1024) {
        const int64_t i = base + t;
        const uint32_t v = i < total ? hist[i] : 0u;
        uint32_t incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            uint32_t w = warp_sums[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t up = __shfl_up_sync(0xffffffffu, w, o);
                if (lane >= o) w += up;
            }
            warp_sums[lane] = w;
        }
        __syncthreads();
        const uint32_t before = carry + (warp > 0 ? warp_sums[warp - 1] : 0u) + (incl - v);
        if (i < total) hist[i] = before;
        __syncthreads();
        if (t == 1023) carry = before + v;
        __syncthreads();
    }
}

// Stable scatter of one 8-bit digit.  LAST: write int64 edge ids to perm instead of the ping-pong buffers.
template <bool LAST>
__global__ void __launch_bounds__(kSortThreads) radix_scatter_kernel(const uint32_t* __restrict__ keys_in,
                                                                     const uint32_t* __restrict__ vals_in, int64_t E,
                                                                     int shift, const uint32_t* __restrict__ hist,
                                                                     int64_t nblocks, uint32_t* __restrict__ keys_out,
                                                                     uint32_t* __restrict__ vals_out,
                                                                     int64_t* __restrict__ perm) {
    constexpr int kWarps = kSortThreads / 32;
    __shared__ uint32_t base[kRadix];               // next free global slot of every digit for this block
    __shared__ uint16_t warp_cnt[kWarps][kRadix];   // per-round, per-warp digit counts
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    base[t] = hist[static_cast<int64_t>(t) * nblocks + blockIdx.x];
    const int64_t chunk0 = static_cast<int64_t>(blockIdx.x) * kSortChunk;

    for (int r = 0; r < kSortItems; ++r) {
        for (int w = 0; w < kWarps; ++w) warp_cnt[w][t] = 0;
        __syncthreads();
        const int64_t i = chunk0 + r * kSortThreads + t;
        const bool live = i < E;
        uint32_t key = 0, val = 0, digit = 0;
        if (live) { key = keys_in[i]; val = vals_in[i]; digit = (key >> shift) & 0xffu; }
        // lanes of this warp holding the same digit (dead lanes get a digit no live lane uses)
        const uint32_t same = __match_any_sync(0xffffffffu, live ? digit : 0xffffffffu);
        const uint32_t rank_in_warp = __popc(same & ((1u << lane) - 1u));
        if (live && rank_in_warp == 0) warp_cnt[warp][digit] = static_cast<uint16_t>(__popc(same));
        __syncthreads();
        if (live) {
            uint32_t before = 0;
            for (int w = 0; w < warp; ++w) before += warp_cnt[w][digit];
            const uint32_t pos = base[digit] + before + rank_in_warp;
            if (LAST) {
                perm[pos] = static_cast<int64_t>(val);
            } else {
                keys_out[pos] = key;
                vals_out[pos] = val;
            }
        }
        __syncthreads();
        uint32_t total = 0;
        for (int w = 0; w < kWarps; ++w) total += warp_cnt[w][t];
        base[t] += total;
        __syncthreads();
    }
}

__global__ void csr_identity_perm_kernel(int64_t* perm, int64_t E) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < E; e += stride) perm[e] = e;
}

}  // namespace e3b

extern "C" int64_t e3b_csr_scratch_bytes(int64_t num_edges, int64_t num_nodes) {
    if (num_edges < 0 || num_nodes < 0) return 0;
    return e3b::csr_layout(num_edges, num_nodes, nullptr, nullptr);
}

extern "C" int e3b_csr_from_dst(const int64_t* dst, int64_t num_edges, int64_t num_nodes, int64_t* perm,
                                int64_t* rowptr, void* scratch, int64_t scratch_bytes, int32_t* status, void* stream) {
    using namespace e3b;
    const int64_t E = num_edges, N = num_nodes;
    if (E < 0 || N < 0) return fail(E3B_ERR_ARG, "csr: negative size");
    if (E >= (1LL << 31) || N >= (1LL << 31)) return fail(E3B_ERR_ARG, "csr: sizes must be below 2^31");
    if (!rowptr || !status || (E > 0 && (!dst || !perm))) return fail(E3B_ERR_ARG, "csr: null pointer");
    if (E > 0 && N == 0) return fail(E3B_ERR_ARG, "csr: edges but no nodes");
    const int64_t need = csr_layout(E, N, nullptr, nullptr);
    if (!scratch || scratch_bytes < need) return fail(E3B_ERR_ARG, "csr: scratch of %lld bytes needed, %lld given", (long long)need, (long long)scratch_bytes);
    if (reinterpret_cast<uintptr_t>(scratch) % 256 != 0) return fail(E3B_ERR_ARG, "csr: scratch must be 256-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CsrScratch sc;
    csr_layout(E, N, static_cast<char*>(scratch), &sc);

    E3B_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int32_t), s));
    if (N > 0) E3B_CUDA_TRY(cudaMemsetAsync(sc.counts, 0, static_cast<size_t>(N) * 4, s));
    const int grid = static_cast<int>(std::min<int64_t>(ceil_div(std::max<int64_t>(E, 1), 256), kNumSMs * 8));
    if (E > 0) csr_prepare_kernel<<<grid, 256, 0, s>>>(dst, E, N, sc.keys[0], sc.vals[0], sc.counts, status);
    exclusive_scan_i32_kernel<<<1, 1024, 0, s>>>(sc.counts, N, rowptr);
    if (E == 0) return check_launch("e3b_csr_from_dst");

    int bits = 0;
    while (bits < 31 && ((N - 1) >> bits) != 0) ++bits;
    const int passes = (bits + 7) / 8;
    if (passes == 0) {  // a single node: every edge already in place
        csr_identity_perm_kernel<<<grid, 256, 0, s>>>(perm, E);
        return check_launch("e3b_csr_from_dst");
    }
    const unsigned nb = static_cast<unsigned>(sc.nblocks);
    int cur = 0;
    for (int p = 0; p < passes; ++p) {
        const int shift = 8 * p;
        radix_hist_kernel<<<nb, kSortThreads, 0, s>>>(sc.keys[cur], E, shift, sc.hist, sc.nblocks);
        radix_scan_kernel<<<1, 1024, 0, s>>>(sc.hist, static_cast<int64_t>(kRadix) * sc.nblocks);
        if (p == passes - 1)
            radix_scatter_kernel<true><<<nb, kSortThreads, 0, s>>>(sc.keys[cur], sc.vals[cur], E, shift, sc.hist,
                                                                    sc.nblocks, nullptr, nullptr, perm);
        else
            radix_scatter_kernel<false><<<nb, kSortThreads, 0, s>>>(sc.keys[cur], sc.vals[cur], E, shift, sc.hist,
                                                                     sc.nblocks, sc.keys[cur ^ 1], sc.vals[cur ^ 1], nullptr);
        cur ^= 1;
    }
    return check_launch("e3b_csr_from_dst");
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant: the scratch lives in this library's own device image.
//
// Some callers cannot hand over scratch memory because they cannot allocate any: code that
// runs inside a memory pool it does not own (an inference server's pre-sized arena), a plug-in
// invoked from a real-time loop where cudaMalloc's implicit device synchronisation is not
// acceptable, or a host language binding that has no device allocator of its own.  For them the
// work area is a fixed array in global memory that every GPU loading this library carries
// until the process exits (about 4.4 MiB).  The price is a hard size limit and a shared buffer.
namespace e3b {

constexpr int64_t kStaticCsrMaxEdges = 1 << 18;   // 262,144
constexpr int64_t kStaticCsrMaxNodes = 1 << 16;   // 65,536
// = csr_layout(kStaticCsrMaxEdges, kStaticCsrMaxNodes): 4 key/value buffers, digit histograms, row counts
constexpr int64_t kStaticCsrBytes = 4 * (kStaticCsrMaxEdges * 4) + kRadix * (kStaticCsrMaxEdges / kSortChunk) * 4
                                    + kStaticCsrMaxNodes * 4;

static __device__ __align__(256) unsigned char g_csr_static_scratch[kStaticCsrBytes];

constexpr int kMaxDevices = 64;
static void* g_csr_static_ptr[kMaxDevices] = {nullptr};
static std::mutex g_csr_static_mutex;

// Device address of the array on the current device.  In host code the array's name is only a
// handle for the runtime, never a device pointer: the address has to be asked for, once per
// device, while that device is current.
static int csr_static_address(void** out) {
    int dev = -1;
    E3B_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(E3B_ERR_UNSUPPORTED, "csr_static: device index %d not supported", dev);
    std::lock_guard<std::mutex> lock(g_csr_static_mutex);
    if (g_csr_static_ptr[dev] == nullptr) {
        void* p = nullptr;
        E3B_CUDA_TRY(cudaGetSymbolAddress(&p, g_csr_static_scratch));
        if (p == nullptr) return fail(E3B_ERR_CUDA, "csr_static: null symbol address");
        g_csr_static_ptr[dev] = p;
    }
    *out = g_csr_static_ptr[dev];
    return E3B_OK;
}

}  // namespace e3b

extern "C" int64_t e3b_csr_static_max_edges(void) { return e3b::kStaticCsrMaxEdges; }
extern "C" int64_t e3b_csr_static_max_nodes(void) { return e3b::kStaticCsrMaxNodes; }

extern "C" int e3b_csr_from_dst_static(const int64_t* dst, int64_t num_edges, int64_t num_nodes, int64_t* perm,
                                       int64_t* rowptr, int32_t* status, void* stream) {
    using namespace e3b;
    if (num_edges < 0 || num_nodes < 0) return fail(E3B_ERR_ARG, "csr_static: negative size");
    if (num_edges > kStaticCsrMaxEdges || num_nodes > kStaticCsrMaxNodes)
        return fail(E3B_ERR_ARG,
                    "csr_static: %lld edges / %lld nodes exceed the built-in work area (at most %lld edges and %lld nodes); "
                    "use e3b_csr_from_dst with caller-provided scratch",
                    (long long)num_edges, (long long)num_nodes, (long long)kStaticCsrMaxEdges, (long long)kStaticCsrMaxNodes);
    void* scratch = nullptr;
    const int rc = csr_static_address(&scratch);
    if (rc != E3B_OK) return rc;
    // Everything that must start from zero (row counts, status word) is cleared by the call below on
    // the caller's stream; the rest of the work area is fully overwritten before it is read.
    return e3b_csr_from_dst(dst, num_edges, num_nodes, perm, rowptr, scratch, kStaticCsrBytes, status, stream);
}
