// Single-block exclusive scan shared by the CSR builder and the neighbour-list builder.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace e3b {

// Exclusive scan of counts[N] into rowptr[N+1] (int64) by one block of 1024 threads.
static __global__ void __launch_bounds__(1024) exclusive_scan_i32_kernel(const int32_t* __restrict__ counts, int64_t N,
                                                          int64_t* __restrict__ rowptr) {
    __shared__ int64_t warp_sums[32];
    __shared__ int64_t carry;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    if (t == 0) carry = 0;
    __syncthreads();
    for (int64_t base = 0; base < N; base += 1024) {
        const int64_t i = base + t;
        int64_t v = i < N ? counts[i] : 0;
        int64_t incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int64_t up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int64_t w = warp_sums[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int64_t up = __shfl_up_sync(0xffffffffu, w, o);
                if (lane >= o) w += up;
            }
            warp_sums[lane] = w;  // inclusive over warps
        }
        __syncthreads();
        const int64_t before = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + (incl - v);
        if (i < N) rowptr[i] = before;
        __syncthreads();
        if (t == 1023) carry = before + v;
        __syncthreads();
    }
    if (t == 0) rowptr[N] = carry;
}

}  // namespace e3b
