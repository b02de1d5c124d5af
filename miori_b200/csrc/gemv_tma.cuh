// Weight-streaming GEMV with the weights staged through shared memory by TMA.
//
// One CTA per SM (two for long streams) owns every gridDim-th 16-row tile.  Each slab -- 16 rows x 1 KiB of
// packed codes plus the rows' scales and biases, three cp.async.bulk.tensor requests -- goes
// into a ring of shared-memory stages; completion is counted in bytes on a "full" mbarrier
// per stage and consumers hand stages back through an "empty" mbarrier.  The ring is filled
// BEFORE the kernel waits for its predecessor (programmatic dependent launch): weights are
// immutable, so a CTA that starts as its predecessor's CTA exits has its first slabs in flight
// while the grids hand over.  After the wait the CTA stages x (see gemv_mma.cuh for the arithmetic
// and the k permutation).
//
// The 16 warps work in four independent groups of four; a group owns whole tiles, each of
// its warps multiplies 4 of the 16 steps of a slab out of shared memory, and the four
// partial sums per output are combined through shared memory behind a group-private named
// barrier by a fixed shuffle tree (so a row's value does not depend on M).  There is no
// CTA-wide barrier in the main loop.  A 17th warp is the TMA producer: one of its threads
// refills a stage as soon as its group hands it back.  Out-of-range rows and columns are
// zero-filled by TMA, which makes every code, scale and bias there contribute exactly 0.
//
// Optional neighbours of the projection, each a template parameter so that the plain instantiation
// is compiled as if they did not exist: NORMED (RMSNorm of fp32 activations inside the staging pass),
// GATED (SiLU x up behind the fused gate + up rows), POSTNORM (post-norm and residual add by the CTA
// that finishes last), ARGMAX (greedy pick of a sharded head).
#pragma once
#include "common.cuh"
#include "gemv_mma.cuh"
#include "norm.cuh"
#include "peers.cuh"
#include "tma_host.cuh"

#include <algorithm>

namespace miori_b200 {
namespace gemvtma {

constexpr int GROUPS = 4;                  // independent groups of 4 warps
constexpr int WARPS = 4 * GROUPS;           // compute warps
constexpr int THREADS = (WARPS + 1) * 32;  // plus one producer warp
constexpr int MAX_STAGES = 12;
constexpr int ROW_BYTES = 1024;            // packed bytes of one row in one slab
constexpr int Q_BYTES = 16 * ROW_BYTES;
constexpr int SB_BYTES = 16 * 128;         // scales (or biases) of 16 rows, up to 64 groups each
constexpr int STAGE_BYTES = Q_BYTES + 2 * SB_BYTES;  // 20480
// staged x in 16-byte units: the 4 chunks of a step sit at unit offsets 0,4,10,14 of an
// 18-unit step and rows have an odd pitch, so the 8 lanes of a quarter warp (2 rows x 4
// chunks) read 8 distinct bank groups with plain immediate offsets
constexpr int STEP_UNITS = 18;
constexpr int SLAB_X_BYTES = 16 * STEP_UNITS * 16;                 // staged x per k-slab and row
constexpr int ZERO_BYTES = 3 * 4 * STEP_UNITS * 16 + 4 * 16 + 64;  // zeros read by masked lanes

template <int MP>
struct Red {
    static constexpr int WS = 16 * MP + 1;           // padded stride of one warp's partials
    static constexpr int GROUP_FLOATS = 2 * 4 * WS;  // double-buffered, 4 warps
};

// Shared-memory loads by 32-bit shared address (one instruction each, no generic addressing).
// volatile: the data arrives through TMA, so the loads must stay behind the mbarrier wait.
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float ldsf32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}

__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
// two floats -> packed fp16 pair (lo, hi), round to nearest even
__device__ __forceinline__ uint32_t f16x2_bits(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// a float rounded to fp16 and back: the value the tensor core will see
__device__ __forceinline__ float through_f16(float v) {
    float r;
    asm("{\n\t.reg .b16 h;\n\tcvt.rn.f16.f32 h, %1;\n\tcvt.f32.f16 %0, h;\n\t}" : "=f"(r) : "f"(v));
    return r;
}

__device__ __forceinline__ void named_barrier(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint32_t x_unit(uint32_t step, uint32_t t, uint32_t wd) {
    return step * STEP_UNITS + 4u * t + 2u * (t >> 1) + wd;
}

// Stage x for the MMA B operand: permuted to the k order of the A fragments (8-bit codes: as
// fp16 scaled by `mul`), laid out by x_unit(); for EXACT also the fp32 sum of x over every chunk
// (PAIR: over every pair of chunks, i.e. every 64-weight group).
// `ld8(m, u)` returns the eight bf16 activations 8u .. 8u+7 of row m (4-bit codes; the plain
// loader reads x, the norm-fused one normalises fp32 activations on the fly).
template <int BITS, bool EXACT, int MP, bool PAIR, class LD>
__device__ __forceinline__ void stage_x_padded(const uint16_t* __restrict__ x, uint4* xs,
                                               float* xsum, uint32_t M, uint32_t K,
                                               uint32_t steps_p, uint32_t pitch, uint32_t cpr,
                                               const float* mul_rows, LD ld8) {
    constexpr int CW = 128 / BITS, KU = BITS == 4 ? 8 : 4;
    const uint32_t upr = steps_p * 16u;  // logical units per row
    for (uint32_t i = threadIdx.x; i < (uint32_t)MP * upr; i += THREADS) {
        const uint32_t m = i / upr, u = i - m * upr;
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        if (m < M && u * KU < K) {
            if (BITS == 4) {
                const uint4 v = ld8(m, u);
                o.x = __byte_perm(v.x, v.z, 0x5410);  // (x0,x4)
                o.y = __byte_perm(v.x, v.z, 0x7632);  // (x1,x5)
                o.z = __byte_perm(v.y, v.w, 0x5410);  // (x2,x6)
                o.w = __byte_perm(v.y, v.w, 0x7632);  // (x3,x7)
            } else {
                // 8-bit codes go to the tensor core as fp16 (1024 + code), so x goes as fp16 too,
                // scaled by the row's power of two that keeps its largest value below 2^15; the
                // unit holds (x0,x2) and (x1,x3), the k order of the byte pairs the unpack makes
                const uint2 v = __ldg(reinterpret_cast<const uint2*>(x + (size_t)m * K) + u);
                const float mul = mul_rows[m];
                o.x = f16x2_bits(bf16lo(v.x) * mul, bf16lo(v.y) * mul);
                o.y = f16x2_bits(bf16hi(v.x) * mul, bf16hi(v.y) * mul);
            }
        }
        xs[(size_t)m * pitch + x_unit(u >> 4, (u >> 2) & 3u, u & 3u)] = o;
    }
    if (EXACT) {
        const uint32_t chunks = K / CW;
        for (uint32_t i = threadIdx.x; i < (uint32_t)MP * cpr; i += THREADS) {
            const uint32_t m = i / cpr, c = i - m * cpr;
            float sum = 0.0f;
            if (m < M && c < chunks) {
                const float mul = BITS == 8 ? mul_rows[m] : 1.0f;
                // PAIR: both chunks of a 64-weight group carry the sum over the whole group
                const uint32_t c0 = PAIR ? (c & ~1u) : c;
                const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)m * K + (size_t)c0 * CW);
#pragma unroll
                for (int j = 0; j < (PAIR ? 2 : 1) * CW / 8; ++j) {
                    const uint4 v = BITS == 4 ? ld8(m, c0 * (CW / 8) + j) : __ldg(xp + j);
                    if (BITS == 4) {
                        sum += bf16lo(v.x); sum += bf16hi(v.x); sum += bf16lo(v.y); sum += bf16hi(v.y);
                        sum += bf16lo(v.z); sum += bf16hi(v.z); sum += bf16lo(v.w); sum += bf16hi(v.w);
                    } else {  // the sum of exactly the fp16 values staged above
                        sum += through_f16(bf16lo(v.x) * mul); sum += through_f16(bf16hi(v.x) * mul);
                        sum += through_f16(bf16lo(v.y) * mul); sum += through_f16(bf16hi(v.y) * mul);
                        sum += through_f16(bf16lo(v.z) * mul); sum += through_f16(bf16hi(v.z) * mul);
                        sum += through_f16(bf16lo(v.w) * mul); sum += through_f16(bf16hi(v.w) * mul);
                    }
                }
            }
            xsum[i] = sum;
        }
    }
}

// The same staging in one pass: a thread loads a unit, stores it permuted, and the 4 (PAIR: 8)
// lanes that hold a chunk (a 64-weight group) add up its fp32 sum with shuffles, so x is read once
// and there is one load latency instead of two.  Two units per thread and trip, both loads issued
// before either is used, so that a long row (K = 8192: four units per thread) costs two load
// latencies, not four.  Whole warps iterate (THREADS and the units per row are multiples of 32
// resp. 16, so lane groups never straddle a chunk).
template <int BITS, bool EXACT, int MP, bool PAIR, class LD>
__device__ __forceinline__ void stage_x_onepass(uint4* xs, float* xsum, uint32_t M, uint32_t K,
                                                uint32_t steps_p, uint32_t pitch, uint32_t cpr, LD ld8) {
    static_assert(BITS == 4, "one-pass staging exists for 4-bit codes only (8-bit x is staged as scaled fp16)");
    static_assert(MP <= 4, "row index by comparison");
    constexpr int KU = 8;
    const uint32_t upr = steps_p * 16u;  // logical units per row
    const uint32_t total = (uint32_t)MP * upr, lane = threadIdx.x & 31u;
    for (uint32_t i0 = threadIdx.x - lane; i0 < total; i0 += 2u * THREADS) {
        uint32_t i[2], m[2], u[2];
        bool live[2];
        uint4 v[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            i[h] = i0 + lane + (uint32_t)h * THREADS;
            m[h] = (i[h] >= upr ? 1u : 0u) + (MP > 2 ? (i[h] >= 2u * upr ? 1u : 0u) + (i[h] >= 3u * upr ? 1u : 0u) : 0u);
            u[h] = i[h] - m[h] * upr;
            live[h] = i[h] < total && m[h] < M && u[h] * KU < K;
            v[h] = make_uint4(0u, 0u, 0u, 0u);
            if (live[h]) v[h] = ld8(m[h], u[h]);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (i0 + (uint32_t)h * THREADS >= total) break;  // warp-uniform
            uint4 o;
            o.x = __byte_perm(v[h].x, v[h].z, 0x5410);  // (x0,x4)
            o.y = __byte_perm(v[h].x, v[h].z, 0x7632);  // (x1,x5)
            o.z = __byte_perm(v[h].y, v[h].w, 0x5410);  // (x2,x6)
            o.w = __byte_perm(v[h].y, v[h].w, 0x7632);  // (x3,x7)
            if (i[h] < total) xs[(size_t)m[h] * pitch + x_unit(u[h] >> 4, (u[h] >> 2) & 3u, u[h] & 3u)] = o;
            if (EXACT) {
                float sum = ((bf16lo(v[h].x) + bf16hi(v[h].x)) + (bf16lo(v[h].y) + bf16hi(v[h].y))) +
                            ((bf16lo(v[h].z) + bf16hi(v[h].z)) + (bf16lo(v[h].w) + bf16hi(v[h].w)));
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
                if (PAIR) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
                if (i[h] < total && (u[h] & 3u) == 0u) xsum[m[h] * cpr + (u[h] >> 2)] = sum;
            }
        }
    }
}

// One-pass staging for more than four staged rows, for rows short enough that every thread handles one or two
// units (K <= 2048): a thread loads a unit, stores it permuted, and the 4 (PAIR: 8) lanes that hold
// a chunk (a 64-weight group) add up its fp32 sum with shuffles, so x is read once and there is
// one load latency instead of two.  Whole warps iterate (THREADS and the units per row are
// multiples of 32 resp. 16, so lane groups never straddle a chunk).  For long rows the two-pass
// version above is faster: its loads are independent across iterations.
template <int BITS, bool EXACT, int MP, bool PAIR, class LD>
__device__ __forceinline__ void stage_x_onepass_wide(uint4* xs, float* xsum, uint32_t M, uint32_t K,
                                                uint32_t steps_p, uint32_t pitch, uint32_t cpr, LD ld8) {
    static_assert(BITS == 4, "one-pass staging exists for 4-bit codes only (8-bit x is staged as scaled fp16)");
    constexpr int KU = 8;
    const uint32_t upr = steps_p * 16u;  // logical units per row
    const uint32_t total = (uint32_t)MP * upr, lane = threadIdx.x & 31u;
    for (uint32_t i0 = threadIdx.x - lane; i0 < total; i0 += THREADS) {
        const uint32_t i = i0 + lane;
        const uint32_t m = i / upr, u = i - m * upr;
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        float sum = 0.0f;
        if (i < total && m < M && u * KU < K) {
            const uint4 v = ld8(m, u);
            o.x = __byte_perm(v.x, v.z, 0x5410);  // (x0,x4)
            o.y = __byte_perm(v.x, v.z, 0x7632);  // (x1,x5)
            o.z = __byte_perm(v.y, v.w, 0x5410);  // (x2,x6)
            o.w = __byte_perm(v.y, v.w, 0x7632);  // (x3,x7)
            if (EXACT)
                sum = ((bf16lo(v.x) + bf16hi(v.x)) + (bf16lo(v.y) + bf16hi(v.y))) +
                      ((bf16lo(v.z) + bf16hi(v.z)) + (bf16lo(v.w) + bf16hi(v.w)));
        }
        if (i < total) xs[(size_t)m * pitch + x_unit(u >> 4, (u >> 2) & 3u, u & 3u)] = o;
        if (EXACT) {
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
            if (PAIR) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
            if (i < total && (u & 3u) == 0u) xsum[m * cpr + (u >> 2)] = sum;
        }
    }
}

// Staging with the RMSNorm in it (shaders/ops.metal:86-115), rows of K <= 2048: x is fp32.  Thread
// i < K/4 loads piece i (four activations) of every row together with its four norm weights -- one
// trip to L2 for everything, which matters because every CTA of the grid asks for the same lines at
// the same moment -- the warps add up the rows' squares (shuffles, 16 warp sums per row through
// shared memory, every thread adds them in order), and each thread normalises its piece with the
// stand-alone kernel's arithmetic, x * inv * gamma rounded to bf16.  Lane pairs then form the
// eight-activation units of the plain staging (permuted store, and for EXACT the fp32 sum over
// every chunk resp. chunk pair, added up in the plain staging's order).
template <bool EXACT, int MP, bool PAIR>
__device__ __forceinline__ void stage_x_normed(const float* __restrict__ x, const uint16_t* __restrict__ gamma,
                                               float eps, uint4* xs, float* xsum, uint32_t M, uint32_t K,
                                               uint32_t pitch, uint32_t cpr, float* part) {
    static_assert(MP <= 4, "rows of the norm prologue");
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t qpr = K >> 2;  // pieces per row, at most 512
    const bool mine = tid < qpr;
    float4 v[MP];
    uint2 gq = make_uint2(0u, 0u);
    if (mine) gq = __ldg(reinterpret_cast<const uint2*>(gamma) + tid);
#pragma unroll
    for (int m = 0; m < MP; ++m) {
        v[m] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (mine && (uint32_t)m < M) v[m] = __ldg(reinterpret_cast<const float4*>(x) + (size_t)m * qpr + tid);
    }
    // units past K and rows past M read as zeros
    for (uint32_t i = tid; i < (uint32_t)MP * pitch; i += THREADS) xs[i] = make_uint4(0u, 0u, 0u, 0u);
    if (EXACT)
        for (uint32_t i = tid; i < (uint32_t)MP * cpr; i += THREADS) xsum[i] = 0.0f;
    if (warp < 16u) {
#pragma unroll
        for (int m = 0; m < MP; ++m) {
            float ss = __fmaf_rn(v[m].w, v[m].w, __fmaf_rn(v[m].z, v[m].z, __fmaf_rn(v[m].y, v[m].y, v[m].x * v[m].x)));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
            if (lane == 0) part[m * 16 + warp] = ss;
        }
    }
    __syncthreads();
    if (warp >= 16u) return;
#pragma unroll
    for (int m = 0; m < MP; ++m) {
        if ((uint32_t)m >= M) break;  // CTA-uniform
        float tot = 0.0f;
#pragma unroll
        for (int w = 0; w < 16; ++w) tot += part[m * 16 + w];
        const float inv = rsqrtf(tot / (float)K + eps);
        const uint32_t lo = float_to_bf16_bits(v[m].x * inv * bf16lo(gq.x)) |
                            (float_to_bf16_bits(v[m].y * inv * bf16hi(gq.x)) << 16);
        const uint32_t hi = float_to_bf16_bits(v[m].z * inv * bf16lo(gq.y)) |
                            (float_to_bf16_bits(v[m].w * inv * bf16hi(gq.y)) << 16);
        // the even lane of a pair collects the unit: activations 8u .. 8u+7, u = tid / 2
        const uint32_t olo = __shfl_down_sync(0xFFFFFFFFu, lo, 1), ohi = __shfl_down_sync(0xFFFFFFFFu, hi, 1);
        const uint32_t u = tid >> 1;
        if (mine && (tid & 1u) == 0u) {
            uint4 o;
            o.x = __byte_perm(lo, olo, 0x5410);  // (x0,x4)
            o.y = __byte_perm(lo, olo, 0x7632);  // (x1,x5)
            o.z = __byte_perm(hi, ohi, 0x5410);  // (x2,x6)
            o.w = __byte_perm(hi, ohi, 0x7632);  // (x3,x7)
            xs[(size_t)m * pitch + x_unit(u >> 4, (u >> 2) & 3u, u & 3u)] = o;
        }
        if (EXACT) {
            float sum = (bf16lo(lo) + bf16hi(lo)) + (bf16lo(hi) + bf16hi(hi));
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);  // the unit
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);  // the chunk of 32
            if (PAIR) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 8);
            if (mine && (tid & 7u) == 0u) xsum[m * cpr + (tid >> 3)] = sum;
        }
    }
}

// ROOMY: compiled for one CTA per SM (up to 120 registers instead of 56).  Problems of at most
// two tiles per SM run 4-18 % faster that way (no spills, freer scheduling); long streams prefer
// two CTAs per SM.
// PAIR (4-bit, group 64, EXACT, NT = 1): the two 32-weight chunks of a scale group sit in
// neighbouring lanes, so the MMA columns are (chunk pair, activation row) instead of (chunk,
// row) and one column set serves four activation rows.  Used for M = 3, 4 at group 64; the sums
// of a group's two chunks then meet inside the tensor core instead of after the scale, so a row
// agrees with its M <= 2 value to fp32 rounding, not bit for bit.
#ifdef MIORI_TMA_TRACE
// Profiling build only: %globaltimer marks of the first and the last CTA of the first 256 launches.
__device__ unsigned long long g_tma_marks[256 * 2 * 8];
__device__ unsigned int g_tma_launch[4];
__device__ unsigned long long g_tma_pmarks[256 * 2 * 4];  // the producer thread's marks
__device__ __forceinline__ unsigned long long gtimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TMA_MARK(i)                                                                              \
    do {                                                                                         \
        if (trace_slot < 256u) g_tma_marks[(trace_slot * 2 + trace_which) * 8 + (i)] = gtimer(); \
    } while (0)
#else
#define TMA_MARK(i) do { } while (0)
#endif

// What the post-norm epilogue needs besides the GEMV's own arguments (null residual: off).
struct PostNorm {
    const float* residual = nullptr;   // x of post_norm_add, fp32 [M][N]
    const uint16_t* gamma = nullptr;   // bf16 [N]
    unsigned int* arrivals = nullptr;  // one zeroed word; the kernel leaves it zero
    float eps = 0.0f;
};

// What the norm prologue needs (null gamma: off): x then points at fp32 activations.
struct PreNorm {
    const uint16_t* gamma = nullptr;  // bf16 [K]
    float eps = 0.0f;
};

// ARGMAX (with SHARDED, one activation row): the head of a greedy decode step.  The rows go to this
// rank's y only -- no packets -- and every thread tracks the best (value, index) of what it stores;
// the candidates meet in a 64-bit atomic maximum, and the CTA that finishes last exchanges this
// rank's best with the peers (peers.cuh: peer_argmax_exchange), so the kernel ends with the winning
// token on every rank and nothing else has crossed NVLink.
template <int BITS, bool EXACT, int NT, bool OUT_BF16, bool SHARDED, bool ROOMY, bool PAIR, bool ARGMAX = false,
          bool GATED = false, bool POSTNORM = false, bool NORMED = false>
__global__ void __launch_bounds__(THREADS, (NT == 1 && !ROOMY) ? 2 : 1)
gemv_tma_kernel(const __grid_constant__ CUtensorMap tmap_q,
                const __grid_constant__ CUtensorMap tmap_s,
                const __grid_constant__ CUtensorMap tmap_b, const uint8_t* __restrict__ qlin,
                const uint16_t* __restrict__ slin, const uint16_t* __restrict__ blin,
                const uint16_t* __restrict__ x, void* __restrict__ y, uint32_t N, uint32_t K,
                uint32_t M, uint32_t gshift, uint32_t ngrp, uint32_t nsg, uint32_t kpar,
                const PeerArgs pa, uint32_t n_total, uint32_t row0, size_t y_off,
                unsigned long long* __restrict__ best, const PostNorm pn, const PreNorm pre) {
    static_assert(!ARGMAX || SHARDED, "the arg-max epilogue lives in the sharded instantiation");
    // POSTNORM: y = residual + v * rsqrt(mean(v^2) + eps) * gamma over each whole output row v of
    // the GEMV (shaders/ops.metal:605-631).  Every CTA stores its part of v into y; the CTA that
    // arrives last then runs the stand-alone kernel's row pass over y in place.
    static_assert(!POSTNORM || (!OUT_BF16 && !SHARDED && !GATED), "the post-norm epilogue: fp32 out, one GPU");
    // NORMED: x points at fp32 activations; the staging pass stages bf16(x * rsqrt(mean(x^2) + eps) *
    // gamma) (shaders/ops.metal:86-115), each CTA computing the rows' sums of squares for itself.
    static_assert(!NORMED || (BITS == 4 && EXACT && !SHARDED && !POSTNORM), "the norm prologue: 4-bit, up to four rows, one GPU");
    // GATED: the weight rows are a gate half [0, N/2) and an up half [N/2, N) (the fused w1/w3
    // projection); a tile is eight rows of each, so that after the tile's reduction one thread
    // pair holds gate and up of the same output, and y is bf16 [M][N/2] of silu(gate) * up.
    static_assert(!GATED || (BITS == 4 && OUT_BF16 && !SHARDED), "the gated epilogue: 4-bit, bf16 out, one GPU");
    using namespace gemvmma;
    const uint32_t nstage = ngrp * nsg;  // every active group owns a private ring of nsg stages
    constexpr int CW = 128 / BITS;          // codes per 16-byte chunk
    constexpr int SK = 4 * CW;              // k per step
    constexpr int KC = 16 * SK;             // k per slab: 16 steps, 4 per warp of a group
    static_assert(!PAIR || (EXACT && NT == 1 && BITS == 4), "PAIR is an EXACT 4-bit single-set mode");
    constexpr int MP = EXACT ? (PAIR ? 4 : 2 * NT) : 8 * NT;
    constexpr float OFF = BITS == 4 ? 128.0f : 1024.0f;  // what the unpack adds to every code
    constexpr uint32_t MASK = 0x000F000Fu, MAGIC = 0x43004300u;  // bf16 128.0 in both halves

    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t grp = warp >> 2, wg = warp & 3u;
    const uint32_t tiles = (N + 15u) >> 4;
    const uint32_t kslabs = (K + KC - 1) / KC;
    const uint32_t steps_p = kslabs * 16u;                 // padded steps along K
    const uint32_t pitch = steps_p * STEP_UNITS + 1u;      // staged x row pitch (units, odd)
    const uint32_t cpr = steps_p * 4u;                     // chunks per padded row
    const uint32_t gps = KC >> gshift;                     // groups per slab row
    // Linear mode (K fits one slab): the 16 rows of a tile are contiguous in memory, so a slab
    // is three plain bulk copies and rows keep their global pitch in shared memory.  Otherwise
    // rows are gathered by 2-D tiled TMA at a fixed 1 KiB / gps pitch.
    const bool linear = qlin != nullptr;
    const uint32_t chunks = K / CW, ng = K >> gshift;
    const bool ktail = linear && chunks < 64u;  // K shorter than one slab of 64 chunks
    const uint32_t qpitch = linear ? K * BITS / 8 : (uint32_t)ROW_BYTES;
    const uint32_t spitch = linear ? ng : gps;

    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bars[MAX_STAGES];
    __shared__ __align__(8) uint64_t empty_bars[MAX_STAGES];
    __shared__ volatile uint32_t abort_flag;
    __shared__ uint32_t x_maxbits[4];  // 8-bit codes: largest |x| bit pattern of each staged row
    __shared__ float x_mul[4];         // 8-bit codes: per-row power-of-two scale of the fp16 staging
    __shared__ float x_rescale[4];     // ... and its inverse, applied at the store
    uint8_t* ring = smem_raw;                                            // [nstage][STAGE_BYTES]
    uint4* xs = reinterpret_cast<uint4*>(ring + (size_t)nstage * STAGE_BYTES);  // [MP][pitch]
    uint4* zeros = xs + (size_t)MP * pitch;                              // ZERO_BYTES of zeros
    float* xsum = reinterpret_cast<float*>(zeros + ZERO_BYTES / 16);     // [MP][cpr] (EXACT)
    float* red = xsum + (EXACT ? (size_t)MP * cpr : 0);                  // [GROUPS] group areas
    float* kred = red + (size_t)GROUPS * Red<MP>::GROUP_FLOATS;          // [2][GROUPS][16*MP]

    pdl_launch_dependents();
#ifdef MIORI_TMA_TRACE
    const unsigned int trace_which = blockIdx.x == 0 ? 0u : 1u;
    unsigned int trace_slot = 0xffffffffu;
    if (threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1))
        trace_slot = atomicAdd(&g_tma_launch[trace_which], 1u);
    TMA_MARK(0);
#endif

    // This CTA's tiles.  Slabs are enumerated in sets of ngrp tiles (one
    // per active group), k-slab major inside a set, so that consecutive slabs belong to
    // different groups.  Group gi's k-th slab lives in stage gi*nsg + k % nsg: a stage is only
    // ever waited on by one group, in order, so barrier parities are never ambiguous.
    // tiles are dealt round-robin (tile = blockIdx.x + j*gridDim.x): at any moment the CTAs
    // stream one contiguous window of the weight matrix, which HBM serves best
    // When a CTA has fewer tiles than groups and K spans several slabs, kpar groups share a
    // tile: each takes every kpar-th k-slab (a "virtual tile") and their partial outputs are
    // summed in a fixed order at the end.  kslabs is a multiple of kpar.
    const uint32_t kshift = kpar >> 1;  // kpar is 1, 2 or 4: log2 without a division
    const uint32_t ntiles = ((tiles - blockIdx.x + gridDim.x - 1) / gridDim.x) << kshift;  // virtual
    const uint32_t kslabs_v = kslabs >> kshift;
    const uint32_t total = ntiles * kslabs_v;
        const uint32_t stage_tx = Q_BYTES + 2u * 16u * gps * 2u;  // bytes tiled TMA delivers per slab

    // producer side (lane 0 of the producer warp only)
    uint32_t issued = 0;
    // Producer cursor, advanced incrementally (no divisions on the issue path): the next slab
    // to issue is k-slab p_ks of the p_gi-th tile of the set starting at tile index p_set0;
    // p_kmod = k % nsg and p_use = k / nsg for the owning group's slab counter k.
    uint32_t p_set0 = 0, p_ks = 0, p_gi = 0, p_kmod = 0, p_use = 0;
    // issue every slab whose stage is free, without blocking
    auto try_refill = [&](uint32_t upto) {
        while (issued < upto) {
            const uint32_t stage = p_gi * nsg + p_kmod;
            if (p_use != 0u) {
                if (!mbar_try(smem_addr(&empty_bars[stage]), (p_use - 1u) & 1u)) break;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            const uint32_t bar = smem_addr(&full_bars[stage]);
            const uint32_t dst = smem_addr(ring + (size_t)stage * STAGE_BYTES);
            const uint32_t vt = p_set0 + p_gi;
            const uint32_t row = (blockIdx.x + (vt >> kshift) * gridDim.x) * 16u;
            const uint32_t ks = (vt & (kpar - 1u)) + (p_ks << kshift);
            if (GATED && linear) {  // N is a multiple of 16: eight whole rows of each half
                const uint32_t r8 = row >> 1, up8 = (N >> 1) + r8;
                mbar_expect_tx(bar, 16u * (qpitch + 4u * spitch));
                bulk_g2s(dst, qlin + (size_t)r8 * qpitch, 8u * qpitch, bar);
                bulk_g2s(dst + 8u * qpitch, qlin + (size_t)up8 * qpitch, 8u * qpitch, bar);
                bulk_g2s(dst + Q_BYTES, slin + (size_t)r8 * spitch, 16u * spitch, bar);
                bulk_g2s(dst + Q_BYTES + 16u * spitch, slin + (size_t)up8 * spitch, 16u * spitch, bar);
                bulk_g2s(dst + Q_BYTES + SB_BYTES, blin + (size_t)r8 * spitch, 16u * spitch, bar);
                bulk_g2s(dst + Q_BYTES + SB_BYTES + 16u * spitch, blin + (size_t)up8 * spitch, 16u * spitch, bar);
            } else if (GATED) {  // the tensor maps' boxes are eight rows high
                const int r8 = (int)(row >> 1), up8 = (int)((N >> 1) + (row >> 1));
                mbar_expect_tx(bar, stage_tx);
                tma_load_2d(dst, &tmap_q, (int)(ks * (ROW_BYTES / 4)), r8, bar);
                tma_load_2d(dst + 8u * ROW_BYTES, &tmap_q, (int)(ks * (ROW_BYTES / 4)), up8, bar);
                tma_load_2d(dst + Q_BYTES, &tmap_s, (int)(ks * gps), r8, bar);
                tma_load_2d(dst + Q_BYTES + 16u * gps, &tmap_s, (int)(ks * gps), up8, bar);
                tma_load_2d(dst + Q_BYTES + SB_BYTES, &tmap_b, (int)(ks * gps), r8, bar);
                tma_load_2d(dst + Q_BYTES + SB_BYTES + 16u * gps, &tmap_b, (int)(ks * gps), up8, bar);
            } else if (linear) {
                const uint32_t nrows = min(16u, N - row);  // rows past N keep stale (unused) data
                mbar_expect_tx(bar, nrows * (qpitch + 4u * spitch));
                bulk_g2s(dst, qlin + (size_t)row * qpitch, nrows * qpitch, bar);
                bulk_g2s(dst + Q_BYTES, slin + (size_t)row * spitch, nrows * spitch * 2u, bar);
                bulk_g2s(dst + Q_BYTES + SB_BYTES, blin + (size_t)row * spitch, nrows * spitch * 2u, bar);
            } else {
                mbar_expect_tx(bar, stage_tx);
                tma_load_2d(dst, &tmap_q, (int)(ks * (ROW_BYTES / 4)), (int)row, bar);
                tma_load_2d(dst + Q_BYTES, &tmap_s, (int)(ks * gps), (int)row, bar);
                tma_load_2d(dst + Q_BYTES + SB_BYTES, &tmap_b, (int)(ks * gps), (int)row, bar);
            }
            ++issued;
            // advance the cursor: next group of the set, then next k-slab, then next set
            const uint32_t nt = min(ngrp, ntiles - p_set0);
            if (++p_gi == nt) {
                p_gi = 0;
                if (++p_kmod == nsg) { p_kmod = 0; ++p_use; }
                if (++p_ks == kslabs_v) { p_ks = 0; p_set0 += ngrp; }
            }
        }
    };

    const bool producer = threadIdx.x == WARPS * 32;
    if (producer) {
#ifdef MIORI_TMA_TRACE
        unsigned int pslot = 0xffffffffu;
        if (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1) pslot = atomicAdd(&g_tma_launch[2 + trace_which], 1u);
#define TMA_PMARK(i) do { if (pslot < 256u) g_tma_pmarks[(pslot * 2 + trace_which) * 4 + (i)] = gtimer(); } while (0)
        TMA_PMARK(0);
#else
#define TMA_PMARK(i) do { } while (0)
#endif
        abort_flag = 0u;
        x_maxbits[0] = x_maxbits[1] = x_maxbits[2] = x_maxbits[3] = 0u;
        for (uint32_t i = 0; i < nstage; ++i) {
            mbar_init(smem_addr(&full_bars[i]), 1);
            mbar_init(smem_addr(&empty_bars[i]), 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        TMA_PMARK(1);
        try_refill(total);  // fills the rings: up to nstage slabs in flight before the wait
        TMA_PMARK(2);
#ifdef MIORI_TMA_TRACE
        for (int spin = 0; spin < 100000 && !mbar_try(smem_addr(&full_bars[0]), 0u); ++spin) { }
        TMA_PMARK(3);
#endif
    }

    pdl_wait_prior();  // x (and y) belong to the predecessor until here
    TMA_MARK(1);

    // N-sharded launch (pa.world > 1): this rank's rows [row0, row0 + N) of an n_total-row output
    // go into its own y (at user offset y_off of its arena) and, as {value, launch number}
    // packets, into every peer's inbox; before the CTA exits it collects its share of the peers'
    // rows (peers.cuh).  The launch number is re-read from the control block at the point of
    // use, so the single-GPU path carries no extra registers through the loop; SHARDED is a
    // template parameter rather than a run-time test because the single-GPU instantiation then
    // compiles exactly as if the peer path did not exist (a run-time branch cost 3-16 %).
    const uint32_t world = SHARDED ? pa.world : 0u;
    unsigned long long my_best = 0ull;  // ARGMAX: key of the best element this thread has stored
    // one output element: y[m][row0 + row]
    auto store_out = [&](uint32_t m, uint32_t row, float v) {
        if (BITS == 8) v *= x_rescale[m];
        const size_t idx = (size_t)m * n_total + row0 + row;
        const uint32_t bits = OUT_BF16 ? float_to_bf16_bits(v) : __float_as_uint(v);
        if (OUT_BF16) reinterpret_cast<uint16_t*>(y)[idx] = (uint16_t)bits;
        else reinterpret_cast<uint32_t*>(y)[idx] = bits;
        if constexpr (ARGMAX) {  // compare what was stored (the rounded value when the output is bf16)
            if (v == v) {
                const unsigned long long key = peer_best_key(OUT_BF16 ? bits << 16 : bits, row0 + row);
                my_best = key > my_best ? key : my_best;
            }
        } else if constexpr (SHARDED) {
            if (world > 1u) {
                const uint32_t e = peer_epoch(pa);
                const size_t elem = y_off / (OUT_BF16 ? 2u : 4u) + idx;
                for (uint32_t p = 0; p < world; ++p)
                    if (p != pa.rank) peer_send(peer_slot(pa, peer_arena(pa, p), e, elem), bits, e);
            }
        }
    };

    // GATED: y[m][row] = bf16(silu(gate) * up) of the N/2-column output, with the arithmetic of the
    // stand-alone activation kernel (shaders/ops.metal:129-139)
    auto store_gated = [&](uint32_t m, uint32_t row, float gate, float up) {
        const float sg = gate / (1.0f + expf(-gate));
        reinterpret_cast<uint16_t*>(y)[(size_t)m * (N >> 1) + row] = (uint16_t)float_to_bf16_bits(sg * up);
    };
    (void)store_gated;

    // one-pass staging where it measured faster: one slab of K, and either the roomy
    // instantiation or at most two staged rows
    if constexpr (BITS == 8) {
        // per-row power-of-two scale for the fp16 staging: the row's largest |x| lands in
        // [2^14, 2^15); the outputs are multiplied back at the store.  Per row, so that a row's
        // result does not depend on its neighbours in the batch.
        static_assert(MP <= 4, "8-bit rows staged per launch");
        __syncthreads();  // x_maxbits was cleared before the wait
        const uint32_t upr8 = K / 8u;  // 16-byte pieces per row
        const uint4* x4 = reinterpret_cast<const uint4*>(x);
        for (uint32_t m = 0; m < M; ++m) {
            uint32_t mx = 0;
            for (uint32_t i = threadIdx.x; i < upr8; i += THREADS) {
                const uint4 v = __ldg(x4 + (size_t)m * upr8 + i);
                const uint32_t a = v.x & 0x7FFF7FFFu, b = v.y & 0x7FFF7FFFu, c = v.z & 0x7FFF7FFFu,
                               d = v.w & 0x7FFF7FFFu;
                mx = max(max(max(mx, a & 0xFFFFu), max(a >> 16, b & 0xFFFFu)),
                         max(max(b >> 16, c & 0xFFFFu), max(max(c >> 16, d & 0xFFFFu), d >> 16)));
            }
            mx = __reduce_max_sync(0xFFFFFFFFu, mx);
            if (lane == 0 && mx) atomicMax(&x_maxbits[m], mx);
        }
        __syncthreads();
        if (threadIdx.x < 4u) {
            const uint32_t top = x_maxbits[threadIdx.x];
            int sh = top ? (int)((top >> 7) & 0xFFu) - 141 : 0;  // bf16 exponent field - 127 - 14
            sh = max(-100, min(110, sh));
            x_mul[threadIdx.x] = __uint_as_float((uint32_t)(127 - sh) << 23);
            x_rescale[threadIdx.x] = __uint_as_float((uint32_t)(127 + sh) << 23);
        }
        __syncthreads();
    }
    __shared__ float nm_part[NORMED ? 4 * (WARPS + 1) : 1];
    __shared__ float nm_inv[4];
    if constexpr (NORMED) {
        if (K <= 2048u)
            stage_x_normed<EXACT, MP, PAIR>(reinterpret_cast<const float*>(x), pre.gamma, pre.eps, xs, xsum, M, K,
                                            pitch, cpr, nm_part);
    }
    if (NORMED && K > 2048u) {
        // longer rows: sums of squares of the (at most four) rows first -- all loads in flight together,
        // warps reduce by shuffles, one thread per row adds the warp sums in order -- then the plain
        // staging passes with a loader that normalises
        static_assert(!NORMED || MP <= 4, "rows of the norm prologue");
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const uint32_t qpr = K >> 2;  // float4 pieces per row (K is a multiple of 32)
        float ss[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (uint32_t i = threadIdx.x; i < qpr; i += THREADS) {
#pragma unroll
            for (uint32_t m = 0; m < 4u; ++m) {
                if (m < M) {
                    const float4 v = __ldg(x4 + (size_t)m * qpr + i);
                    ss[m] = __fmaf_rn(v.w, v.w, __fmaf_rn(v.z, v.z, __fmaf_rn(v.y, v.y, __fmaf_rn(v.x, v.x, ss[m]))));
                }
            }
        }
#pragma unroll
        for (uint32_t m = 0; m < 4u; ++m) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss[m] += __shfl_xor_sync(0xFFFFFFFFu, ss[m], o);
            if (lane == 0) nm_part[m * (WARPS + 1) + warp] = ss[m];
        }
        __syncthreads();
        if (threadIdx.x < 4u) {
            float tot = 0.0f;
            for (uint32_t w = 0; w <= (uint32_t)WARPS; ++w) tot += nm_part[threadIdx.x * (WARPS + 1) + w];
            nm_inv[threadIdx.x] = rsqrtf(tot / (float)K + pre.eps);
        }
        __syncthreads();
    }
    // the eight bf16 activations 8u .. 8u+7 of row m
    auto ld8 = [&](uint32_t m, uint32_t u) -> uint4 {
        if constexpr (NORMED) {
            const float4* xr = reinterpret_cast<const float4*>(x) + (size_t)m * (K >> 2) + 2u * u;
            const float4 a = __ldg(xr), c = __ldg(xr + 1);
            const uint4 gm = __ldg(reinterpret_cast<const uint4*>(pre.gamma) + u);
            const float inv = nm_inv[m];
            // the stand-alone norm kernel's arithmetic: x * inv * gamma, rounded to bf16
            auto two = [&](float lo, float hi, uint32_t g2) {
                return float_to_bf16_bits(lo * inv * bf16lo(g2)) | (float_to_bf16_bits(hi * inv * bf16hi(g2)) << 16);
            };
            return make_uint4(two(a.x, a.y, gm.x), two(a.z, a.w, gm.y), two(c.x, c.y, gm.z), two(c.z, c.w, gm.w));
        } else {
            return __ldg(reinterpret_cast<const uint4*>(x + (size_t)m * K) + u);
        }
    };
    bool staged = false;
    if constexpr (NORMED) staged = K <= 2048u;  // staged above, norm included
    if constexpr (BITS == 4) {
        if (staged) {
        } else if constexpr (MP <= 4) {
            if (ROOMY || MP <= 2) {
                stage_x_onepass<BITS, EXACT, MP, PAIR>(xs, xsum, M, K, steps_p, pitch, cpr, ld8);
                staged = true;
            }
        } else if ((ROOMY || MP <= 2) && kslabs == 1u) {
            stage_x_onepass_wide<BITS, EXACT, MP, PAIR>(xs, xsum, M, K, steps_p, pitch, cpr, ld8);
            staged = true;
        }
    }
    if (!staged) stage_x_padded<BITS, EXACT, MP, PAIR>(x, xs, xsum, M, K, steps_p, pitch, cpr, x_mul, ld8);
    for (uint32_t i = threadIdx.x; i < ZERO_BYTES / 16; i += THREADS)
        zeros[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    TMA_MARK(2);

    // per-lane constants, all as 32-bit shared addresses / byte offsets
    const uint32_t n = lane >> 2;
    const uint32_t lc0 = wg * 4u + t;                               // first chunk of this lane in a slab
    const uint32_t ring_a = smem_addr(ring);
    const uint32_t q_lane = g * qpitch + lc0 * 16u;                 // + i4*256 per step, + 8*qpitch for row g+8
    const uint32_t sb_lane = Q_BYTES + (g * spitch + ((lc0 * CW) >> gshift)) * 2u;
    const uint32_t sb_step = ((16u * CW) >> gshift) * 2u;           // groups advance per step (bytes)
    const uint32_t sb_row8 = 8u * spitch * 2u;
    uint32_t xb[NT];        // B-fragment base of this lane: k-slab 0, step wg
    uint32_t xadv[NT];      // advance per k-slab (0 for masked lanes, which read zeros)
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const uint32_t m = PAIR ? (n & 3u) : EXACT ? (2u * j + (n & 1u)) : (8u * j + n);
        const bool active = PAIR ? ((n >> 2) == (t >> 1)) : EXACT ? ((n >> 1) == t) : true;
        xb[j] = active ? smem_addr(xs + (size_t)m * pitch + x_unit(wg, t, 0)) : smem_addr(zeros);
        xadv[j] = active ? (uint32_t)SLAB_X_BYTES * kpar : 0u;  // groups sharing a tile stride kpar slabs
    }
    const uint32_t xs_adv = 256u * kpar;                            // chunk sums per k-slab stride (bytes)
    const uint32_t xs_row = cpr * 4u;
    // chunk (ks*16 + i4*4 + wg)*4 + t of row 0 (PAIR: of the lane's first row, 0 or 2)
    uint32_t xsp = smem_addr(xsum) + lc0 * 4u + (PAIR ? (t & 1u) * 2u * xs_row : 0u);
    float* gred = red + (size_t)grp * Red<MP>::GROUP_FLOATS;

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

    // `ok` turns false for good once a wait expires; the warp then skips waits and math but
    // still takes part in every group barrier so that no other warp is left waiting.
    bool ok = true;
    uint32_t tile_it = 0;
    uint32_t c_kmod = 0, c_par = 0;  // this group's slab counter k: k % nsg and (k / nsg) & 1
    if (producer) {
        // keep the rings fed until every slab has been issued (bounded: gives up with the CTA)
        const long long t0 = clock64();
        while (issued < total && !abort_flag) {
            try_refill(total);
            if (clock64() - t0 > 4 * WAIT_LIMIT_CYCLES) {
                abort_flag = 1u;
                device_error(0x6E14u, blockIdx.x, issued);
            }
        }
    }
    for (uint32_t set0 = 0; warp < WARPS && set0 < ntiles; set0 += ngrp) {
        const uint32_t nt = min(ngrp, ntiles - set0);
        if (grp >= nt) break;
        const uint32_t vt = set0 + grp;
        const uint32_t kp = vt & (kpar - 1u);
        const uint32_t tile = blockIdx.x + (vt >> kshift) * gridDim.x;
        // start at this group's first k-slab of the row
        if (kpar > 1u) {
#pragma unroll
            for (int j = 0; j < NT; ++j) xb[j] += kp * (xadv[j] >> kshift);
            xsp += kp * 256u;
        }
        for (uint32_t ks = 0; ks < kslabs_v; ++ks) {
            const uint32_t stage = grp * nsg + c_kmod, parity = c_par;
            if (++c_kmod == nsg) { c_kmod = 0; c_par ^= 1u; }
#ifdef MIORI_TMA_TRACE
            if (tile_it == 0 && ks == 0) TMA_MARK(7);
#endif
            if (ok) {
                ok = mbar_wait(smem_addr(&full_bars[stage]), parity, &abort_flag, 0x10);
                ok = __all_sync(0xFFFFFFFFu, ok);
            }
#ifdef MIORI_TMA_TRACE
            if (tile_it == 0 && ks == 0) TMA_MARK(4);
#endif
            if (ok) {
                const uint32_t st = ring_a + stage * (uint32_t)STAGE_BYTES;
                uint32_t qa = st + q_lane, sa = st + sb_lane, lc = lc0;
                uint32_t xa[NT];
#pragma unroll
                for (int j = 0; j < NT; ++j) xa[j] = xb[j];
                uint32_t xsa = xsp;
#pragma unroll 1
                for (uint32_t i4 = 0; i4 < 4u; ++i4) {
                    const uint4 q0 = lds128(qa);
                    const uint4 q1 = lds128(qa + 8u * qpitch);
                    uint32_t s0 = lds16(sa), b0 = lds16(sa + SB_BYTES);
                    uint32_t s1 = lds16(sa + sb_row8), b1 = lds16(sa + sb_row8 + SB_BYTES);
                    // past the end of K (linear mode with a short K only; tiled TMA zero-fills):
                    // a zero scale and bias against zero-staged x contribute exactly 0
                    if (ktail && lc >= chunks) s0 = b0 = s1 = b1 = 0u;
                    const uint32_t w0[4] = {q0.x, q0.y, q0.z, q0.w};
                    const uint32_t w1[4] = {q1.x, q1.y, q1.z, q1.w};
                    // two independent accumulation chains (even / odd words), each started by
                    // an MMA with a zero accumulator input
                    float d0[NT][4], d1[NT][4];
                    uint32_t s2a = 0, b2a = 0, s2b = 0, b2b = 0;
                    if (!EXACT) {
                        s2a = s0 | (s0 << 16); b2a = b0 | (b0 << 16);
                        s2b = s1 | (s1 << 16); b2b = b1 | (b1 << 16);
                    }
                    if constexpr (BITS == 8) {
                        // bytes (b0,b2) and (b1,b3) of a word become two fp16 pairs 1024 + code:
                        // two masks and one shift per word, one MMA per word
                        constexpr uint32_t BMASK = 0x00FF00FFu, HMAGIC = 0x64006400u;
#pragma unroll
                        for (int wd = 0; wd < 4; ++wd) {
                            const uint32_t a0 = lop3_and_or(w0[wd], BMASK, HMAGIC);
                            const uint32_t a1 = lop3_and_or(w0[wd] >> 8, BMASK, HMAGIC);
                            const uint32_t c0 = lop3_and_or(w1[wd], BMASK, HMAGIC);
                            const uint32_t c1 = lop3_and_or(w1[wd] >> 8, BMASK, HMAGIC);
#pragma unroll
                            for (int j = 0; j < NT; ++j) {
                                const uint2 xu = lds64(xa[j] + wd * 16);
                                if (wd == 0) mma_f16_z(d0[j], a0, c0, a1, c1, xu.x, xu.y);
                                else if (wd == 1) mma_f16_z(d1[j], a0, c0, a1, c1, xu.x, xu.y);
                                else if (wd == 2) mma_f16(d0[j], a0, c0, a1, c1, xu.x, xu.y);
                                else mma_f16(d1[j], a0, c0, a1, c1, xu.x, xu.y);
                            }
                        }
                    } else {
#pragma unroll
                    for (int wd = 0; wd < 4; ++wd) {
                        uint32_t a[4], c[4];  // pairs (n0,n4),(n1,n5),(n2,n6),(n3,n7), rows g, g+8
#pragma unroll
                        for (int p = 0; p < 4; ++p) {
                            a[p] = lop3_and_or(w0[wd] >> (4 * p), MASK, MAGIC);
                            c[p] = lop3_and_or(w1[wd] >> (4 * p), MASK, MAGIC);
                            if (!EXACT) {
                                a[p] = bf16x2_fma(bf16x2_sub(a[p], MAGIC), s2a, b2a);
                                c[p] = bf16x2_fma(bf16x2_sub(c[p], MAGIC), s2b, b2b);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < NT; ++j) {
                            const uint4 xu = lds128(xa[j] + wd * 16);
                            if (wd == 0) mma_bf16_z(d0[j], a[0], c[0], a[1], c[1], xu.x, xu.y);
                            else if (wd == 1) mma_bf16_z(d1[j], a[0], c[0], a[1], c[1], xu.x, xu.y);
                            else if (wd & 1) mma_bf16(d1[j], a[0], c[0], a[1], c[1], xu.x, xu.y);
                            else mma_bf16(d0[j], a[0], c[0], a[1], c[1], xu.x, xu.y);
                            if (wd & 1) mma_bf16(d1[j], a[2], c[2], a[3], c[3], xu.z, xu.w);
                            else mma_bf16(d0[j], a[2], c[2], a[3], c[3], xu.z, xu.w);
                        }
                    }
                    }
                    if (EXACT) {
                        const float sc0 = __uint_as_float(s0 << 16);
                        const float bt0 = __fmaf_rn(-OFF, sc0, __uint_as_float(b0 << 16));
                        const float sc1 = __uint_as_float(s1 << 16);
                        const float bt1 = __fmaf_rn(-OFF, sc1, __uint_as_float(b1 << 16));
#pragma unroll
                        for (int j = 0; j < NT; ++j) {
                            const float xs0 = ldsf32(xsa + (2 * j) * xs_row);
                            acc[j][0] = __fmaf_rn(sc0, d0[j][0] + d1[j][0], __fmaf_rn(bt0, xs0, acc[j][0]));
                            acc[j][2] = __fmaf_rn(sc1, d0[j][2] + d1[j][2], __fmaf_rn(bt1, xs0, acc[j][2]));
                            if (PAIR || 2u * j + 1u < M) {  // CTA-uniform: the odd activation row exists
                                const float xs1 = ldsf32(xsa + (2 * j + 1) * xs_row);
                                acc[j][1] = __fmaf_rn(sc0, d0[j][1] + d1[j][1], __fmaf_rn(bt0, xs1, acc[j][1]));
                                acc[j][3] = __fmaf_rn(sc1, d0[j][3] + d1[j][3], __fmaf_rn(bt1, xs1, acc[j][3]));
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < NT; ++j)
#pragma unroll
                            for (int e = 0; e < 4; ++e) acc[j][e] += d0[j][e] + d1[j][e];
                    }
                    // next step of this warp: 4 steps (16 chunks) further along the row
                    qa += 256u;
                    sa += sb_step;
                    lc += 16u;
                    xsa += 64u;
#pragma unroll
                    for (int j = 0; j < NT; ++j) xa[j] += 4u * STEP_UNITS * 16u;
                }
            }
            if (ok) {
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_addr(&empty_bars[stage]));  // stage consumed
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) xb[j] += xadv[j];
            xsp += xs_adv;
        }
        // back to k-slab 0 of the row
#pragma unroll
        for (int j = 0; j < NT; ++j) xb[j] -= kslabs_v * xadv[j] + kp * (xadv[j] >> kshift);
        xsp -= kslabs_v * xs_adv + kp * 256u;

#ifdef MIORI_TMA_TRACE
        if (tile_it == 0) TMA_MARK(5);
#endif
        // ---- tile complete: quad sum (EXACT), then 4 partials per output through shared memory
        constexpr int WS = Red<MP>::WS;
        float* buf = gred + (size_t)(tile_it & 1u) * 4 * WS;
        float* mine = buf + (size_t)wg * WS;
        if (PAIR) {
            // lanes t and t^2 hold the two chunk pairs of the same two activation rows
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[0][e] += __shfl_xor_sync(0xFFFFFFFFu, acc[0][e], 2);
            if (t < 2u) {  // t = 0: rows 0, 1; t = 1: rows 2, 3
                mine[g * MP + 2 * t] = acc[0][0];
                mine[g * MP + 2 * t + 1] = acc[0][1];
                mine[(g + 8) * MP + 2 * t] = acc[0][2];
                mine[(g + 8) * MP + 2 * t + 1] = acc[0][3];
            }
        } else if (EXACT) {
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = acc[j][e];
                    v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
                    v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
                    acc[j][e] = v;
                }
            if (t == 0) {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    mine[g * MP + 2 * j] = acc[j][0];
                    mine[g * MP + 2 * j + 1] = acc[j][1];
                    mine[(g + 8) * MP + 2 * j] = acc[j][2];
                    mine[(g + 8) * MP + 2 * j + 1] = acc[j][3];
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                mine[g * MP + 8 * j + 2 * t] = acc[j][0];
                mine[g * MP + 8 * j + 2 * t + 1] = acc[j][1];
                mine[(g + 8) * MP + 8 * j + 2 * t] = acc[j][2];
                mine[(g + 8) * MP + 8 * j + 2 * t + 1] = acc[j][3];
            }
        }
        named_barrier(1u + grp, 128u);
        const uint32_t gt = wg * 32u + lane;  // thread index inside the group
#pragma unroll
        for (uint32_t base = 0; base < 16u * MP * 4u; base += 128u) {
            const uint32_t idx = base + gt;
            const uint32_t o = idx >> 2, w = idx & 3u;  // output o = m*16 + r, partial of warp w
            // GATED enumerates the outputs as o = (m*8 + r')*2 + half, tile row r = r' + 8 half:
            // gate and up of an output sit in neighbouring quads (neighbouring threads below)
            const uint32_t r = GATED ? ((o >> 1) & 7u) + ((o & 1u) << 3) : o & 15u, m = o >> 4;
            float v = buf[(size_t)w * WS + r * MP + m];
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
            const uint32_t row = tile * 16u + r;
            if constexpr (GATED) {
                const float up = __shfl_down_sync(0xFFFFFFFFu, v, 4);
                if (kpar > 1u) {
                    if (w == 0) kred[((size_t)(tile_it & 1u) * GROUPS + grp) * (16 * MP) + o] = v;
                } else if (w == 0 && (o & 1u) == 0u && m < M && ok) {
                    store_gated(m, tile * 8u + r, v, up);
                }
            } else if (kpar > 1u) {
                if (w == 0) kred[((size_t)(tile_it & 1u) * GROUPS + grp) * (16 * MP) + o] = v;
            } else if (w == 0 && m < M && row < N && ok) {
                store_out(m, row, v);
            }
        }
        if (kpar > 1u) {
            // the kpar groups of this tile meet; the first of them sums the partials in order
            named_barrier(5u + (grp >> kshift), kpar * 128u);
            if (kp == 0u) {
                const float* kr = kred + ((size_t)(tile_it & 1u) * GROUPS + grp) * (16 * MP);
                for (uint32_t o = gt; o < 16u * MP; o += 128u) {
                    float v = kr[o];
                    for (uint32_t j = 1; j < kpar; ++j) v += kr[(size_t)j * (16 * MP) + o];
                    if constexpr (GATED) {  // 16 MP is a multiple of 32: whole warps run this loop
                        const float up = __shfl_down_sync(0xFFFFFFFFu, v, 1);
                        const uint32_t m = o >> 4;
                        if ((o & 1u) == 0u && m < M && ok) store_gated(m, tile * 8u + ((o >> 1) & 7u), v, up);
                    } else {
                        const uint32_t r = o & 15u, m = o >> 4, row = tile * 16u + r;
                        if (m < M && row < N && ok) store_out(m, row, v);
                    }
                }
            }
        }
#ifdef MIORI_TMA_TRACE
        if (tile_it == 0) TMA_MARK(6);
#endif
        ++tile_it;
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
    }

    TMA_MARK(3);
    if (abort_flag) {  // let copies still in flight land before the CTA's memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
    }
    if constexpr (POSTNORM) {  // every thread of the CTA gets here: no early exits above
        __shared__ float pn_part[neighbors::NORM_THREADS / 32];
        __shared__ uint32_t pn_last;
        __threadfence();  // this thread's rows of v are visible before the CTA reports in
        __syncthreads();
        if (threadIdx.x == 0) {
            pn_last = atomicAdd(pn.arrivals, 1u) == gridDim.x - 1u ? 1u : 0u;
            __threadfence();
        }
        __syncthreads();
        if (pn_last && threadIdx.x < (uint32_t)neighbors::NORM_THREADS) {
            float* out = reinterpret_cast<float*>(y);
            for (uint32_t m = 0; m < M; ++m) {
                const size_t at = (size_t)m * N;
                if (N <= 8u * (uint32_t)neighbors::NORM_THREADS)
                    neighbors::post_norm_add_row_regs<9, true, 8>(pn.residual + at, out + at, pn.gamma, out + at, N,
                                                                  pn.eps, pn_part);
                else
                    neighbors::post_norm_add_row<9, true>(pn.residual + at, out + at, pn.gamma, out + at, N, pn.eps,
                                                          pn_part);
                neighbors::norm_sync<9>();  // pn_part is reused by the next row
            }
            if (threadIdx.x == 0) *pn.arrivals = 0u;  // ready for the next launch
        }
    } else if constexpr (ARGMAX) {  // every thread of the CTA gets here: no early exits above
        unsigned long long k = my_best;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, k, o);
            k = other > k ? other : k;
        }
        __shared__ unsigned long long warp_keys[WARPS + 1];
        if (lane == 0) warp_keys[warp] = k;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (uint32_t w = 1; w <= (uint32_t)WARPS; ++w) k = warp_keys[w] > k ? warp_keys[w] : k;
            if (k != 0ull) atomicMax(best, k);  // one candidate per CTA
            unsigned int* arrived = reinterpret_cast<unsigned int*>(best + 1);
            __threadfence();
            if (atomicAdd(arrived, 1u) == gridDim.x - 1u) {  // the last CTA: every candidate is in
                __threadfence();
                const unsigned long long win = atomicExch(best, 0ull);  // read, and reset for the next launch
                *arrived = 0u;
                uint32_t* pairs = reinterpret_cast<uint32_t*>(best) + 4;
                const size_t base = (size_t)(reinterpret_cast<uint8_t*>(pairs) - (pa.local + PEER_CTL_BYTES)) / 4u;
                peer_argmax_exchange(pa, pairs, base, peer_best_from_key(win));
            }
        }
    } else if constexpr (SHARDED) {
        if (world > 1u) {  // every thread of the CTA gets here: no early exits above
            const uint32_t e = peer_epoch(pa);
            __syncthreads();
            peer_collect<OUT_BF16>(pa, e, y_off, M, n_total, row0, N);
            __syncthreads();
            if (threadIdx.x == 0) peer_finish(pa, e);
            TMA_MARK(7);  // tracing build: the peers' rows are in y
        }
    }
}

template <int BITS, bool EXACT, int NT, bool PAIR>
size_t fixed_smem(uint32_t K) {
    constexpr int KC = 16 * 4 * (128 / BITS);
    constexpr int MP = EXACT ? (PAIR ? 4 : 2 * NT) : 8 * NT;
    const uint32_t kslabs = (K + KC - 1) / KC, steps_p = kslabs * 16;
    size_t bytes = (size_t)MP * (steps_p * STEP_UNITS + 1) * 16 + ZERO_BYTES;
    if (EXACT) bytes += (size_t)MP * steps_p * 4 * 4;
    bytes += (size_t)GROUPS * Red<MP>::GROUP_FLOATS * 4;
    bytes += (size_t)2 * GROUPS * 16 * MP * 4;  // partial outputs of groups that share a tile
    return bytes;
}

// Placement of an N-sharded launch's output: peers (world <= 1: none, y is a plain pointer),
// rows of the whole output, this rank's first row, and the offset of y inside every arena.
struct Shard {
    PeerArgs pa = {};
    uint32_t n_total = 0, row0 = 0;
    size_t y_off = 0;
    // arg-max epilogue (one activation row): 16 bytes of zeroed scratch {key, arrivals} followed by
    // the (2 world + 2) words of the candidates and the winner, inside the local arena; null: off
    unsigned long long* best = nullptr;
    // gated epilogue (4-bit weights, one GPU): rows [0, N/2) are the gate and [N/2, N) the up
    // projection, y is bf16 [M][N/2] of silu(gate) * up
    bool gated = false;
    // post-norm epilogue (4-bit weights, fp32 out, up to four rows, one GPU); residual null: off
    PostNorm post;
    // norm prologue (4-bit weights, up to four rows, one GPU; fp32 out or the gated epilogue): x is
    // fp32; gamma null: off
    PreNorm pre;
};

// Launch plan: CTAs, active groups and stages per group; ngrp == 0 means the TMA path cannot
// take the problem.
struct Plan {
    uint32_t grid, ngrp, nsg, kpar;
    bool pad = false;  // raise the shared-memory request above half an SM (see plan_stages)
    bool roomy;  // one CTA per SM and few tiles: use the instantiation with the larger register budget
};
template <int BITS, bool EXACT, int NT, bool PAIR>
Plan plan_stages(uint32_t N, uint32_t K, uint32_t group) {
    constexpr int KC = 16 * 4 * (128 / BITS);
    Plan p = {0, 0, 0, 1, false, false};
    if ((K / group) % 8 != 0) return p;  // scale rows must have a 16-byte pitch for TMA
    const size_t fixed = fixed_smem<BITS, EXACT, NT, PAIR>(K);
    const uint32_t tiles = (N + 15) / 16, kslabs = (K + KC - 1) / KC;
    const uint32_t sms = (uint32_t)sm_count();
    // Long streams (many tiles per SM) launch two CTAs per SM, each sized for half an SM, for
    // latency hiding.  Everything else launches at most one CTA per SM, and the one- and two-row
    // kernels then also claim more than half of the SM's shared memory, so that no second CTA of
    // any kernel of this family can join it.  Sharing an SM with the successor of a
    // dependent-launch chain looks attractive (it prefetches while this one computes) and is
    // 5-10 % faster while every launch has the same footprint, but the placement is not stable:
    // after a launch with another footprint the successor's CTAs double up on the SMs that were
    // free and leave others without one, every later launch inherits the skew, and a 24-layer
    // chain of four shapes ran 17 % slower than the sum of its parts.  With the SM to itself a CTA
    // starts as its predecessor's CTA exits, fills a ring of up to 200 KB during the ~1.5 us
    // hand-over between the grids, and the placement is one CTA per SM whatever ran before.
    const size_t half = 112 * 1024, hard = 208 * 1024;
    const bool fits_half = fixed + 4 * STAGE_BYTES <= half;
    if (!fits_half && fixed + 2 * STAGE_BYTES > hard) return p;
    const bool two_per_sm = fits_half && NT == 1 && tiles * kslabs > 6 * sms;
    const bool alone = !two_per_sm && EXACT && NT == 1 && !PAIR;
    const bool whole = !fits_half || alone;
    const uint32_t st = (uint32_t)(((whole ? hard : half) - fixed) / STAGE_BYTES);
    p.grid = std::min<uint32_t>(tiles, two_per_sm ? 2 * sms : sms);
    p.roomy = !two_per_sm && (tiles <= 2 * sms || alone);
    p.pad = alone;
    const uint32_t tiles_cta = (tiles + p.grid - 1) / p.grid;  // tiles of the busiest CTA
    // few tiles per CTA and a long K: let 2 or 4 groups share a tile, each taking every
    // kpar-th k-slab
    while (p.kpar * 2 <= (uint32_t)GROUPS && tiles_cta * p.kpar * 2 <= (uint32_t)GROUPS &&
           kslabs % (p.kpar * 2) == 0 && st >= p.kpar * 2)
        p.kpar *= 2;
    const uint32_t vtiles = tiles_cta * p.kpar;
    p.ngrp = std::min<uint32_t>(std::min<uint32_t>(GROUPS, st), vtiles);
    p.ngrp -= p.ngrp % p.kpar;
    const uint32_t sets = (vtiles + p.ngrp - 1) / p.ngrp;
    p.nsg = std::min<uint32_t>(st / p.ngrp, sets * (kslabs / p.kpar));  // no more than a group needs
    if (p.ngrp * p.nsg > (uint32_t)MAX_STAGES) p.nsg = MAX_STAGES / p.ngrp;
    return p;
}

template <int BITS, bool EXACT, int NT, bool PAIR>
int launch_one(Plan plan, const void* q, const void* s, const void* b, const void* x, void* y,
               uint32_t N, uint32_t K, uint32_t M, uint32_t group, uint32_t flags,
               cudaStream_t stream, const Shard& sh) {
    constexpr int KC = 16 * 4 * (128 / BITS);
    const size_t smem = fixed_smem<BITS, EXACT, NT, PAIR>(K) + (size_t)plan.ngrp * plan.nsg * STAGE_BYTES;
    const uint32_t grid = plan.grid;
    const bool pdl = (flags & MIORI_LAUNCH_PDL) != 0;
    const uint32_t gshift = group == 32 ? 5u : 6u;
    // K within one slab: plain bulk copies (rows of a tile are contiguous); else tiled TMA
    const bool linear = K <= (uint32_t)KC && !(flags & MIORI_TUNE_GEMV_TILED);
    CUtensorMap tq, ts, tb;
    const uint32_t box_rows = sh.gated ? 8 : 16;  // gated: a tile is two boxes, one from each half
    int rc = make_tmap_2d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, (uint64_t)K * BITS / 32, N,
                          ROW_BYTES / 4, box_rows, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    rc = make_tmap_2d(&ts, s, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, K / group, N, KC / group, box_rows,
                      CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    rc = make_tmap_2d(&tb, b, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, K / group, N, KC / group, box_rows,
                      CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    const uint8_t* ql = linear ? reinterpret_cast<const uint8_t*>(q) : nullptr;
    cudaError_t e = cudaSuccess;
#define MIORI_TMA_LAUNCH(OB, SH, AM, GT, PN) MIORI_TMA_LAUNCH_N(OB, SH, AM, GT, PN, false)
#define MIORI_TMA_LAUNCH_N(OB, SH, AM, GT, PN, NM)                                               \
    do {                                                                                         \
        auto kern = roomy ? gemv_tma_kernel<BITS, EXACT, NT, OB, SH, NT == 1, PAIR, AM, GT, PN, NM>  \
                          : gemv_tma_kernel<BITS, EXACT, NT, OB, SH, false, PAIR, AM, GT, PN, NM>;   \
        e = cudaSuccess;                                                                         \
        if (smem_l > 48 * 1024)                                                                  \
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_l); \
        if (e == cudaSuccess)                                                                    \
            e = launch(kern, dim3(grid), dim3(THREADS), smem_l, stream, pdl, tq, ts, tb, ql,     \
                       reinterpret_cast<const uint16_t*>(s), reinterpret_cast<const uint16_t*>(b), \
                       reinterpret_cast<const uint16_t*>(x), y, N, K, M, gshift, plan.ngrp, plan.nsg, plan.kpar, \
                       sh.pa, placed ? sh.n_total : N, placed ? sh.row0 : 0u, sh.y_off, sh.best, sh.post, sh.pre); \
    } while (0)
    const bool sharded = sh.pa.world > 1;
    constexpr bool can_argmax = EXACT && NT == 1 && !PAIR;  // the one- and two-row kernels
    const bool argmax = sh.best != nullptr;
    if (argmax && (!can_argmax || M != 1))
        return fail(MIORI_E_INVALID, "the arg-max epilogue takes one activation row");
    const bool placed = sharded || argmax;  // y is a slice of an n_total-row output
    const bool roomy = NT == 1 && plan.roomy;
    const size_t smem_l = plan.pad ? std::max<size_t>(smem, 120 * 1024) : smem;
    if (sh.gated && (BITS != 4 || sharded || argmax || N % 16 != 0))
        return fail(MIORI_E_INVALID, "the gated epilogue takes 4-bit weights with N a multiple of 16 on one GPU");
    const bool postnorm = sh.post.residual != nullptr;
    if (postnorm && (BITS != 4 || !EXACT || sharded || argmax || sh.gated || (flags & MIORI_OUT_BF16)))
        return fail(MIORI_E_INVALID, "the post-norm epilogue takes 4-bit weights, up to four rows, fp32 out, one GPU");
    if constexpr (can_argmax) {
        if (argmax) {
            if (flags & MIORI_OUT_BF16) MIORI_TMA_LAUNCH(true, true, true, false, false);
            else MIORI_TMA_LAUNCH(false, true, true, false, false);
        }
    }
    const bool normed = sh.pre.gamma != nullptr;
    if (normed && (BITS != 4 || !EXACT || sharded || argmax || postnorm || (!sh.gated && (flags & MIORI_OUT_BF16))))
        return fail(MIORI_E_INVALID, "the norm prologue takes 4-bit weights, up to four rows, one GPU, fp32 out "
                                     "or the gated epilogue");
    if constexpr (BITS == 4 && EXACT) {
        if (normed) {
            if (sh.gated) MIORI_TMA_LAUNCH_N(true, false, false, true, false, true);
            else MIORI_TMA_LAUNCH_N(false, false, false, false, false, true);
        }
    }
    if constexpr (BITS == 4) {
        if (sh.gated && !normed) MIORI_TMA_LAUNCH(true, false, false, true, false);
    }
    if constexpr (BITS == 4 && EXACT) {
        if (postnorm) MIORI_TMA_LAUNCH(false, false, false, false, true);
    }
    if (!argmax && !sh.gated && !postnorm && !normed) {
        if (flags & MIORI_OUT_BF16) {
            if (sharded) MIORI_TMA_LAUNCH(true, true, false, false, false);
            else MIORI_TMA_LAUNCH(true, false, false, false, false);
        } else {
            if (sharded) MIORI_TMA_LAUNCH(false, true, false, false, false);
            else MIORI_TMA_LAUNCH(false, false, false, false, false);
        }
    }
#undef MIORI_TMA_LAUNCH
#undef MIORI_TMA_LAUNCH_N
    if (e != cudaSuccess) return cuda_fail(e, "gemv_tma launch");
    return MIORI_OK;
}

// Try the TMA path; returns 1 if this problem is not eligible (nothing launched).
template <int BITS>
int try_launch(const void* q, const void* s, const void* b, const void* x, void* y, uint32_t N,
               uint32_t K, uint32_t M, uint32_t group, uint32_t flags, cudaStream_t stream,
               const Shard& sh = Shard()) {
    Plan pl;
#define MIORI_TMA_TRY(EX, NTV, PR)                                                               \
    do {                                                                                         \
        pl = plan_stages<BITS, EX, NTV, PR>(N, K, group);                                        \
        if (pl.ngrp == 0) return 1;                                                              \
        return launch_one<BITS, EX, NTV, PR>(pl, q, s, b, x, y, N, K, M, group, flags, stream, sh); \
    } while (0)
    if (M <= 2) MIORI_TMA_TRY(true, 1, false);
    if constexpr (BITS == 4) {
        // three and four rows at group 64: one column set instead of two (13-21 % faster while K
        // fits one slab; over several slabs the two column sets measured 7-12 % faster); one and
        // two rows stay on the per-chunk columns, which stage half as much x
        if (M <= 4 && group == 64 && K <= 2048) MIORI_TMA_TRY(true, 1, true);
    }
    if (M <= 4) MIORI_TMA_TRY(true, 2, false);
    if constexpr (BITS == 8) {
        return 1;
    } else {
        if (M <= 8) MIORI_TMA_TRY(false, 1, false);
        if (M <= 16) MIORI_TMA_TRY(false, 2, false);
        MIORI_TMA_TRY(false, 4, false);
    }
#undef MIORI_TMA_TRY
}

}  // namespace gemvtma
}  // namespace miori_b200
