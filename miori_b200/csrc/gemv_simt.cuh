// fp32-dequant GEMV, SIMT: the shape-agnostic path (any N, any K % group == 0).
//
// One warp owns one output row at a time and walks it in 16-byte chunks (32 four-bit or
// 16 eight-bit codes), one chunk per lane per iteration, exactly the work split of the
// reference kernels (shaders/ops.metal:16-24, shaders/batch.metal:157-163): lane g
// strides the chunks by 32 and accumulates acc = fma(code*scale+bias, x, acc) in k order,
// then the lanes are summed with shuffles.  Up to MT activation rows share one pass over
// the weight row (the reference's gemv4_b does four).  x is staged once per CTA in shared
// memory as bf16 with a 16-byte-unit XOR swizzle so that the lanes' strided 64-byte reads
// do not collide on banks.
#pragma once
#include "common.cuh"

namespace miori_b200 {

// Physical 16-byte unit of logical unit u inside a staged x row.
__device__ __forceinline__ uint32_t simt_swz(uint32_t u) { return u ^ ((u >> 3) & 3u); }

template <int BITS, int MT, bool OUT_BF16>
__global__ void __launch_bounds__(256)
gemv_simt_kernel(const uint4* __restrict__ q, const uint16_t* __restrict__ s,
                 const uint16_t* __restrict__ b, const uint16_t* __restrict__ x,
                 void* __restrict__ y, uint32_t N, uint32_t K, uint32_t M, uint32_t gshift) {
    constexpr int WPC = 128 / BITS;   // weights per 16-byte chunk
    constexpr int UPC = WPC / 8;      // 16-byte units of bf16 x per chunk
    extern __shared__ uint4 xs[];     // [MT][K/8] units, swizzled
    const uint32_t units = K >> 3;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t chunks = K / WPC;
    const uint32_t ng = K >> gshift;

    pdl_launch_dependents();
    pdl_wait_prior();  // x may be produced by the preceding kernel

    for (uint32_t i = threadIdx.x; i < (uint32_t)MT * units; i += blockDim.x) {
        const uint32_t m = i / units, u = i - m * units;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (m < M) v = __ldg(reinterpret_cast<const uint4*>(x) + (size_t)m * units + u);
        xs[m * units + simt_swz(u)] = v;
    }
    __syncthreads();

    const uint32_t warps_per_grid = gridDim.x * (blockDim.x >> 5);
    for (uint32_t row = blockIdx.x * (blockDim.x >> 5) + warp; row < N; row += warps_per_grid) {
        const uint4* qrow = q + (size_t)row * chunks;
        const uint16_t* srow = s + (size_t)row * ng;
        const uint16_t* brow = b + (size_t)row * ng;
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = 0.0f;

        for (uint32_t c = lane; c < chunks; c += 32u) {
            const uint4 w = __ldg(qrow + c);
            const uint32_t g = (c * WPC) >> gshift;
            const float sc = bf16_bits_to_float(__ldg(srow + g));
            const float bi = bf16_bits_to_float(__ldg(brow + g));
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
            // dequantize the chunk once: float(code) via the 2^23 mantissa trick (exact)
            float wv[WPC];
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
                for (int j = 0; j < 32 / BITS; ++j) {
                    const uint32_t code = (ww[wi] >> (BITS * j)) & ((1u << BITS) - 1u);
                    const float qf = __uint_as_float(0x4B000000u | code) - 8388608.0f;
                    wv[wi * (32 / BITS) + j] = __fmaf_rn(qf, sc, bi);
                }
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
#pragma unroll
                for (int u = 0; u < UPC; ++u) {
                    const uint4 xv = xs[m * units + simt_swz(c * UPC + u)];
                    const uint32_t xr[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        acc[m] = __fmaf_rn(wv[u * 8 + 2 * p], bf16lo(xr[p]), acc[m]);
                        acc[m] = __fmaf_rn(wv[u * 8 + 2 * p + 1], bf16hi(xr[p]), acc[m]);
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = acc[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            if (lane == 0 && (uint32_t)m < M) {
                if (OUT_BF16)
                    reinterpret_cast<uint16_t*>(y)[(size_t)m * N + row] =
                        (uint16_t)float_to_bf16_bits(v);
                else
                    reinterpret_cast<float*>(y)[(size_t)m * N + row] = v;
            }
        }
    }
}

// Enqueue the SIMT GEMV for rows [0,M) of x, M <= 4 per pass; wider M runs as several
// passes over the weights (each pass is self-contained, so rows never depend on M).
template <int BITS>
int launch_gemv_simt(const void* q, const void* s, const void* b, const void* x, void* y,
                     uint32_t N, uint32_t K, uint32_t M, uint32_t group, uint32_t flags,
                     cudaStream_t stream) {
    const uint32_t gshift = group == 32 ? 5u : 6u;
    const bool out_bf16 = (flags & MIORI_OUT_BF16) != 0;
    const bool pdl = (flags & MIORI_LAUNCH_PDL) != 0;
    const size_t esz = out_bf16 ? 2 : 4;
    for (uint32_t m0 = 0; m0 < M; m0 += 4) {
        const uint32_t mt = (M - m0) >= 4 ? 4 : (M - m0);
        const uint16_t* xp = reinterpret_cast<const uint16_t*>(x) + (size_t)m0 * K;
        void* yp = reinterpret_cast<char*>(y) + (size_t)m0 * N * esz;
        const int mtc = mt == 1 ? 1 : (mt == 2 ? 2 : 4);
        const size_t smem = (size_t)mtc * K * 2;
        const uint32_t rows_per_cta = 8;
        uint32_t grid = (N + rows_per_cta - 1) / rows_per_cta;
        const uint32_t cap = (uint32_t)sm_count() * 8u;
        if (grid > cap) grid = cap;
        cudaError_t e = cudaSuccess;
#define MIORI_SIMT_CASE(MTV, OB)                                                              \
    do {                                                                                      \
        auto kern = gemv_simt_kernel<BITS, MTV, OB>;                                          \
        if (smem > 48 * 1024) {                                                               \
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                     (int)smem);                                              \
            if (e != cudaSuccess) break;                                                      \
        }                                                                                     \
        e = launch(kern, dim3(grid), dim3(256), smem, stream, pdl,                            \
                   reinterpret_cast<const uint4*>(q), reinterpret_cast<const uint16_t*>(s),   \
                   reinterpret_cast<const uint16_t*>(b), xp, yp, N, K, mt, gshift);           \
    } while (0)
        if (mtc == 1) { if (out_bf16) MIORI_SIMT_CASE(1, true); else MIORI_SIMT_CASE(1, false); }
        else if (mtc == 2) { if (out_bf16) MIORI_SIMT_CASE(2, true); else MIORI_SIMT_CASE(2, false); }
        else { if (out_bf16) MIORI_SIMT_CASE(4, true); else MIORI_SIMT_CASE(4, false); }
#undef MIORI_SIMT_CASE
        if (e != cudaSuccess) return cuda_fail(e, "gemv_simt launch");
    }
    return MIORI_OK;
}

}  // namespace miori_b200
