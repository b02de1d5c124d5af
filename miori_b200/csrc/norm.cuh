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

// The same for rows of at most NORM_THREADS * PER elements, with every load of the row issued before
// the first use -- one trip to memory instead of two dependent ones.  Same sums in the same order,
// same expression: the same bits.
template <int BAR, bool FRESH, int PER>
__device__ __forceinline__ void post_norm_add_row_regs(const float* x, const float* src, const uint16_t* w,
                                                       float* out, uint32_t n, float eps, float* part) {
    float v[PER], r[PER];
    uint16_t g[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const uint32_t i = threadIdx.x + (uint32_t)j * NORM_THREADS;
        v[j] = 0.0f, r[j] = 0.0f, g[j] = 0;
        if (i < n) {
            v[j] = norm_load<FRESH>(src, i);
            r[j] = x[i];
            g[j] = w[i];
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < PER; ++j)
        if (threadIdx.x + (uint32_t)j * NORM_THREADS < n) ss = __fmaf_rn(v[j], v[j], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if ((threadIdx.x & 31u) == 0) part[threadIdx.x >> 5] = ss;
    norm_sync<BAR>();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < NORM_THREADS / 32; ++i) tot += part[i];
    const float inv = rsqrtf(tot / (float)n + eps);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const uint32_t i = threadIdx.x + (uint32_t)j * NORM_THREADS;
        if (i < n) out[i] = r[j] + v[j] * inv * bf16_bits_to_float(g[j]);
    }
}

}  // namespace neighbors
}  // namespace miori_b200
