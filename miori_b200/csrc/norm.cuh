// Row arithmetic shared by the stand-alone norm kernels and the GEMV epilogue that applies
// post_norm_add (shaders/ops.metal:605-631) to the rows it has just produced: the same 256 threads
// in the same order, so both give the same bits.
#pragma once
#include "common.cuh"

namespace miori_b200 {
namespace neighbors {

constexpr int NORM_THREADS = 256;

// Meeting point of the NORM_THREADS threads that work on a row.  BAR == 0: they are the whole CTA;
// otherwise the CTA's first NORM_THREADS threads, on named barrier BAR.
template <int BAR>
__device__ __forceinline__ void norm_sync() {
    if constexpr (BAR == 0) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(NORM_THREADS) : "memory");
}

// Element i of a row another CTA of this launch may have written (L2 is the point of coherence).
template <bool FRESH>
__device__ __forceinline__ float norm_load(const float* row, uint32_t i) {
    if constexpr (FRESH) return __ldcg(row + i);
    else return row[i];
}

// Sum of squares of a row, in a fixed order: every thread adds its strided elements, warps reduce
// by shuffles, every thread then adds the eight warp sums.  Called by threads 0 .. NORM_THREADS-1.
template <int BAR, bool FRESH>
__device__ __forceinline__ float row_sum_squares(const float* row, uint32_t n, float* part) {
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += NORM_THREADS) {
        const float v = norm_load<FRESH>(row, i);
        ss = __fmaf_rn(v, v, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if ((threadIdx.x & 31u) == 0) part[threadIdx.x >> 5] = ss;
    norm_sync<BAR>();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < NORM_THREADS / 32; ++i) tot += part[i];
    return tot;
}

// out = x + src * rsqrt(mean(src^2) + eps) * w for one row of n elements; out may be src.
template <int BAR, bool FRESH>
__device__ __forceinline__ void post_norm_add_row(const float* x, const float* src, const uint16_t* w, float* out,
                                                  uint32_t n, float eps, float* part) {
    const float inv = rsqrtf(row_sum_squares<BAR, FRESH>(src, n, part) / (float)n + eps);
    for (uint32_t i = threadIdx.x; i < n; i += NORM_THREADS)
        out[i] = x[i] + norm_load<FRESH>(src, i) * inv * bf16_bits_to_float(w[i]);
}

}  // namespace neighbors
}  // namespace miori_b200
