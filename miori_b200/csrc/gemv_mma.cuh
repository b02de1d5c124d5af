// Weight-streaming GEMV for 1 <= M <= 32 activation rows, HBM-bound by design.
//
// A warp owns a tile of 16 output rows.  Lane (g = lane/4, t = lane%4) streams, with one
// 128-bit load per row, the packed codes of rows g and g+8 for the 16-byte chunk
// (4*step + t) of the row (32 four-bit or 16 eight-bit codes).  Codes are turned into
// bf16 pairs in registers with one shift+LOP3 per pair (code | 0x4300 == 128+code, exact in
// bf16) and fed straight to mma.sync.m16n8k16 as the A operand; the k index inside an MMA
// is a fixed permutation of the chunk, and the activations are staged once per CTA in
// shared memory in that same permuted order (plus an XOR swizzle of 16-byte units so that
// the B-fragment loads do not collide on banks).  fp32 accumulation happens in the MMA.
//
//   EXACT  (M <= 4): the eight MMA columns are (chunk lane t, activation row m), with x
//          zeroed in the columns of the other lanes' chunks, so every lane gets the raw
//          sum_k (128+code)*x of ITS OWN chunk and applies the group's fp32 scale and bias
//          itself: y += s*D + (b - 128*s)*sum(x).  Same arithmetic class as the
//          reference's gemv4/gemv4_b (fp32 dequantization, fp32 accumulation).
//   PRESCALED (4 < M <= 32, 4-bit): A = bf16(code*s + b) by one bf16x2 fma, columns are
//          activation rows; this is what the reference's wide-batch path multiplies too
//          (its bf16 weight cache, src/batch.cpp:223-230).
// 8-bit codes use the same extraction: each byte is split into two nibbles that multiply
// x and 16*x (both staged), so one accumulator receives (128+lo)*x + 16*(128+hi)*x.
//
// The 8 warps of a CTA split K in 128-bit-chunk steps (step = 4 chunks per quad), prefetch
// the next work item's weights before reducing the current one, and with a programmatic
// dependent launch they issue the first weight loads BEFORE waiting for the predecessor
// kernel (weights are immutable; only x and y depend on it).  A row's result is summed in
// a fixed order, so it does not depend on M or on the launch shape.
#pragma once
#include "common.cuh"

namespace miori_b200 {
namespace gemvmma {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int SPW = 2;  // steps per warp per work item (loads in flight per lane: 2*SPW)

__device__ __forceinline__ uint32_t swz(uint32_t u, uint32_t m) {
    return u ^ (((u >> 3) & 1u) | ((m & 1u) << 1));
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a&b)|c
    return r;
}
__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t bf16x2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The fp16 forms of the same MMA (8-bit codes of the TMA kernel travel as fp16 1024 + code).
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    const float z = 0.0f;
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
}

// Same MMA with a zero accumulator input: starts a chain without clearing registers first.
__device__ __forceinline__ void mma_bf16_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                           uint32_t a3, uint32_t b0, uint32_t b1) {
    const float z = 0.0f;
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
}

struct Frag {          // one step of one lane: two rows' chunks plus their group parameters
    uint4 w0, w1;      // rows g and g+8
    uint32_t sb0, sb1; // (scale | bias << 16) bf16 bits for rows g and g+8
};

template <int BITS>
__device__ __forceinline__ void load_frag(Frag& f, const uint4* __restrict__ q,
                                          const uint16_t* __restrict__ s,
                                          const uint16_t* __restrict__ b, uint32_t row0,
                                          uint32_t row1, uint32_t chunk, uint32_t chunks,
                                          uint32_t ng, uint32_t gshift) {
    constexpr int CW = 128 / BITS;
    if (chunk < chunks) {
        f.w0 = __ldg(q + (size_t)row0 * chunks + chunk);
        f.w1 = __ldg(q + (size_t)row1 * chunks + chunk);
        const uint32_t g = (chunk * CW) >> gshift;
        f.sb0 = (uint32_t)__ldg(s + (size_t)row0 * ng + g) | ((uint32_t)__ldg(b + (size_t)row0 * ng + g) << 16);
        f.sb1 = (uint32_t)__ldg(s + (size_t)row1 * ng + g) | ((uint32_t)__ldg(b + (size_t)row1 * ng + g) << 16);
    } else {
        f.w0 = make_uint4(0u, 0u, 0u, 0u);
        f.w1 = f.w0;
        f.sb0 = 0u;
        f.sb1 = 0u;
    }
}

// One step of one warp: 16 rows x (4 chunks) against NT column tiles.  `step` is the global
// step index along K (it addresses the staged activations); acc is updated in place.
template <int BITS, bool EXACT, int NT>
__device__ __forceinline__ void mma_step(const uint4& q0, const uint4& q1, uint32_t sb0,
                                         uint32_t sb1, uint32_t step, uint32_t t,
                                         const uint4* __restrict__ xs, const float* __restrict__ xsum,
                                         uint32_t upr, uint32_t cpr, const uint32_t (&mrow)[NT],
                                         const bool (&active)[NT], float (&acc)[NT][4]) {
    constexpr float OFF = BITS == 4 ? 128.0f : 2176.0f;  // sum of the 128 offsets per code
    constexpr uint32_t MASK = 0x000F000Fu, MAGIC = 0x43004300u;  // bf16 128.0 in both halves
    const uint32_t w0[4] = {q0.x, q0.y, q0.z, q0.w};
    const uint32_t w1[4] = {q1.x, q1.y, q1.z, q1.w};
    // two independent accumulation chains (even / odd words) halve the MMA dependency depth
    float d0[NT][4], d1[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        d0[j][0] = d0[j][1] = d0[j][2] = d0[j][3] = 0.0f;
        d1[j][0] = d1[j][1] = d1[j][2] = d1[j][3] = 0.0f;
    }
    uint32_t s2a = 0, b2a = 0, s2b = 0, b2b = 0;
    if (!EXACT) {
        s2a = __byte_perm(sb0, 0u, 0x1010); b2a = __byte_perm(sb0, 0u, 0x3232);
        s2b = __byte_perm(sb1, 0u, 0x1010); b2b = __byte_perm(sb1, 0u, 0x3232);
    }
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) {
        uint32_t a[4], c[4];  // pairs (n0,n4),(n1,n5),(n2,n6),(n3,n7) of rows g, g+8
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            a[p] = lop3_and_or(w0[wd] >> (4 * p), MASK, MAGIC);
            c[p] = lop3_and_or(w1[wd] >> (4 * p), MASK, MAGIC);
            if (!EXACT) {
                a[p] = bf16x2_fma(bf16x2_sub(a[p], MAGIC), s2a, b2a);
                c[p] = bf16x2_fma(bf16x2_sub(c[p], MAGIC), s2b, b2b);
            }
        }
        const uint32_t u = step * 16u + t * 4u + wd;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            uint4 xu = make_uint4(0u, 0u, 0u, 0u);
            if (active[j]) xu = xs[(size_t)mrow[j] * upr + swz(u, mrow[j])];
            if (wd & 1) {
                mma_bf16(d1[j], a[0], c[0], a[1], c[1], xu.x, xu.y);
                mma_bf16(d1[j], a[2], c[2], a[3], c[3], xu.z, xu.w);
            } else {
                mma_bf16(d0[j], a[0], c[0], a[1], c[1], xu.x, xu.y);
                mma_bf16(d0[j], a[2], c[2], a[3], c[3], xu.z, xu.w);
            }
        }
    }
    if (EXACT) {
        const float sc0 = bf16lo(sb0), bt0 = __fmaf_rn(-OFF, sc0, bf16hi(sb0));
        const float sc1 = bf16lo(sb1), bt1 = __fmaf_rn(-OFF, sc1, bf16hi(sb1));
        const uint32_t chunk = step * 4u + t;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const float xs0 = xsum[(size_t)(2 * j) * cpr + chunk];
            const float xs1 = xsum[(size_t)(2 * j + 1) * cpr + chunk];
            acc[j][0] = __fmaf_rn(sc0, d0[j][0] + d1[j][0], __fmaf_rn(bt0, xs0, acc[j][0]));
            acc[j][1] = __fmaf_rn(sc0, d0[j][1] + d1[j][1], __fmaf_rn(bt0, xs1, acc[j][1]));
            acc[j][2] = __fmaf_rn(sc1, d0[j][2] + d1[j][2], __fmaf_rn(bt1, xs0, acc[j][2]));
            acc[j][3] = __fmaf_rn(sc1, d0[j][3] + d1[j][3], __fmaf_rn(bt1, xs1, acc[j][3]));
        }
    } else {
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[j][e] += d0[j][e] + d1[j][e];
    }
}

// Stage the activations for the MMA B operand: x permuted to the k order of the A fragments
// (and 16*x beside x for 8-bit codes), 16-byte units XOR-swizzled; for EXACT also the fp32
// sum of x over every chunk.  All threads of the CTA call this; the caller synchronises.
template <int BITS, bool EXACT, int MP>
__device__ __forceinline__ void stage_x(const uint16_t* __restrict__ x, uint4* xs, float* xsum,
                                        uint32_t M, uint32_t K, uint32_t upr, uint32_t cpr,
                                        uint32_t chunks, uint32_t nthreads) {
    constexpr int CW = 128 / BITS, KU = BITS == 4 ? 8 : 4;
    for (uint32_t i = threadIdx.x; i < (uint32_t)MP * upr; i += nthreads) {
        const uint32_t m = i / upr, u = i - m * upr;
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        if (m < M && u * KU < K) {
            if (BITS == 4) {
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + (size_t)m * K) + u);
                o.x = __byte_perm(v.x, v.z, 0x5410);  // (x0,x4)
                o.y = __byte_perm(v.x, v.z, 0x7632);  // (x1,x5)
                o.z = __byte_perm(v.y, v.w, 0x5410);  // (x2,x6)
                o.w = __byte_perm(v.y, v.w, 0x7632);  // (x3,x7)
            } else {
                const uint2 v = __ldg(reinterpret_cast<const uint2*>(x + (size_t)m * K) + u);
                const uint32_t x02 = __byte_perm(v.x, v.y, 0x5410);  // (x0,x2)
                const uint32_t x13 = __byte_perm(v.x, v.y, 0x7632);  // (x1,x3)
                const uint32_t sixteen = 0x41804180u, zero = 0u;     // bf16 16.0 pair
                o.x = x02;
                o.y = bf16x2_fma(x02, sixteen, zero);
                o.z = x13;
                o.w = bf16x2_fma(x13, sixteen, zero);
            }
        }
        xs[(size_t)m * upr + swz(u, m)] = o;
    }
    if (EXACT) {
        for (uint32_t i = threadIdx.x; i < (uint32_t)MP * cpr; i += nthreads) {
            const uint32_t m = i / cpr, c = i - m * cpr;
            float sum = 0.0f;
            if (m < M && c < chunks) {
                const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)m * K + (size_t)c * CW);
#pragma unroll
                for (int j = 0; j < CW / 8; ++j) {
                    const uint4 v = __ldg(xp + j);
                    sum += bf16lo(v.x); sum += bf16hi(v.x); sum += bf16lo(v.y); sum += bf16hi(v.y);
                    sum += bf16lo(v.z); sum += bf16hi(v.z); sum += bf16lo(v.w); sum += bf16hi(v.w);
                }
            }
            xsum[i] = sum;
        }
    }
}

// End of a 16-row tile: sum the quad lanes (EXACT) and then the NWARPS warps' partial sums in
// a fixed order through shared memory, store y[m][tile*16 + r], and clear acc.  Contains two
// CTA-wide barriers; every thread of the CTA must call it.
template <bool EXACT, int NT, bool OUT_BF16, int NWARPS, int MP>
__device__ __forceinline__ void reduce_store(float (&acc)[NT][4], float* red, uint32_t warp,
                                             uint32_t g, uint32_t t, uint32_t tile, void* y,
                                             uint32_t N, uint32_t M) {
    if (EXACT) {
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
                float* r0 = red + ((size_t)warp * 16 + g) * MP + 2 * j;
                float* r1 = red + ((size_t)warp * 16 + g + 8) * MP + 2 * j;
                r0[0] = acc[j][0]; r0[1] = acc[j][1];
                r1[0] = acc[j][2]; r1[1] = acc[j][3];
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            float* r0 = red + ((size_t)warp * 16 + g) * MP + 8 * j + 2 * t;
            float* r1 = red + ((size_t)warp * 16 + g + 8) * MP + 8 * j + 2 * t;
            r0[0] = acc[j][0]; r0[1] = acc[j][1];
            r1[0] = acc[j][2]; r1[1] = acc[j][3];
        }
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < 16u * MP; i += NWARPS * 32) {
        const uint32_t m = i >> 4, r = i & 15u;  // consecutive threads -> consecutive rows
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) v += red[((size_t)w * 16 + r) * MP + m];
        const uint32_t row = tile * 16u + r;
        if (m < M && row < N) {
            if (OUT_BF16)
                reinterpret_cast<uint16_t*>(y)[(size_t)m * N + row] = (uint16_t)float_to_bf16_bits(v);
            else
                reinterpret_cast<float*>(y)[(size_t)m * N + row] = v;
        }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
}

template <int BITS, bool EXACT, int NT, bool OUT_BF16>
__global__ void __launch_bounds__(THREADS)
gemv_mma_kernel(const uint4* __restrict__ q, const uint16_t* __restrict__ s,
                const uint16_t* __restrict__ b, const uint16_t* __restrict__ x,
                void* __restrict__ y, uint32_t N, uint32_t K, uint32_t M, uint32_t gshift) {
    constexpr int CW = 128 / BITS;          // codes per 16-byte chunk
    constexpr int SK = 4 * CW;              // k per step (one chunk per quad lane)
    constexpr int MP = EXACT ? 2 * NT : 8 * NT;  // staged activation rows
    constexpr int KU = BITS == 4 ? 8 : 4;   // k per 16-byte unit of staged x

    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t chunks = K / CW, ng = K >> gshift;
    const uint32_t steps = (chunks + 3u) >> 2;
    const uint32_t segs = (steps + WARPS * SPW - 1) / (WARPS * SPW);  // work items per tile
    const uint32_t upr = steps * (SK / KU);                            // staged units per row
    const uint32_t cpr = steps * 4u;                                   // staged chunks per row
    const uint32_t tiles = (N + 15u) >> 4;

    extern __shared__ uint4 smem[];
    uint4* xs = smem;                                                   // [MP][upr]
    float* xsum = reinterpret_cast<float*>(xs + (size_t)MP * upr);      // [MP][cpr] (EXACT)
    float* red = xsum + (EXACT ? (size_t)MP * cpr : 0);                 // [WARPS][16][MP]

    pdl_launch_dependents();

    // first work item's weights: issued before waiting for the predecessor kernel
    Frag cur[SPW], nxt[SPW];
    uint32_t tile = blockIdx.x, seg = 0;
    auto rows = [&](uint32_t tl, uint32_t& r0, uint32_t& r1) {
        r0 = min(tl * 16u + g, N - 1u);
        r1 = min(tl * 16u + g + 8u, N - 1u);
    };
    auto load_item = [&](Frag (&f)[SPW], uint32_t tl, uint32_t sg) {
        uint32_t r0, r1;
        rows(tl, r0, r1);
#pragma unroll
        for (int i = 0; i < SPW; ++i) {
            const uint32_t step = (sg * SPW + i) * WARPS + warp;
            load_frag<BITS>(f[i], q, s, b, r0, r1, step * 4u + t, chunks, ng, gshift);
        }
    };
    if (tile < tiles) load_item(cur, tile, 0);

    pdl_wait_prior();

    stage_x<BITS, EXACT, MP>(x, xs, xsum, M, K, upr, cpr, chunks, THREADS);
    __syncthreads();

    // B-fragment addressing of this lane
    const uint32_t n = lane >> 2;
    uint32_t mrow[NT];
    bool active[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        mrow[j] = EXACT ? (2u * j + (n & 1u)) : (8u * j + n);
        active[j] = EXACT ? ((n >> 1) == t) : true;
    }

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

    while (tile < tiles) {
        // prefetch the next work item
        uint32_t ntile = tile, nseg = seg + 1;
        if (nseg == segs) { nseg = 0; ntile = tile + gridDim.x; }
        if (ntile < tiles) load_item(nxt, ntile, nseg);

#pragma unroll
        for (int i = 0; i < SPW; ++i) {
            const uint32_t step = (seg * SPW + i) * WARPS + warp;
            if (step < steps)
                mma_step<BITS, EXACT, NT>(cur[i].w0, cur[i].w1, cur[i].sb0, cur[i].sb1, step, t, xs,
                                          xsum, upr, cpr, mrow, active, acc);
        }

        if (seg + 1 == segs)
            reduce_store<EXACT, NT, OUT_BF16, WARPS, MP>(acc, red, warp, g, t, tile, y, N, M);

#pragma unroll
        for (int i = 0; i < SPW; ++i) cur[i] = nxt[i];
        tile = ntile;
        seg = nseg;
    }
}

template <int BITS, bool EXACT, int NT>
size_t smem_bytes(uint32_t K) {
    constexpr int CW = 128 / BITS, SK = 4 * CW, KU = BITS == 4 ? 8 : 4;
    constexpr int MP = EXACT ? 2 * NT : 8 * NT;
    const uint32_t chunks = K / CW, steps = (chunks + 3) / 4;
    size_t bytes = (size_t)MP * steps * (SK / KU) * 16;
    if (EXACT) bytes += (size_t)MP * steps * 4 * 4;
    bytes += (size_t)WARPS * 16 * MP * 4;
    return bytes;
}

template <int BITS, bool EXACT, int NT>
int launch_one(const void* q, const void* s, const void* b, const void* x, void* y, uint32_t N,
               uint32_t K, uint32_t M, uint32_t group, uint32_t flags, cudaStream_t stream) {
    const size_t smem = smem_bytes<BITS, EXACT, NT>(K);
    const uint32_t tiles = (N + 15u) / 16u;
    // CTAs per SM by shared memory and registers (<= 3 resident), persistent over the tiles
    uint32_t per_sm = (uint32_t)(200 * 1024 / (smem + 1024));
    per_sm = per_sm < 1 ? 1 : (per_sm > 3 ? 3 : per_sm);
    uint32_t grid = (uint32_t)sm_count() * per_sm;
    if (grid > tiles) grid = tiles;
    const bool pdl = (flags & MIORI_LAUNCH_PDL) != 0;
    const uint32_t gshift = group == 32 ? 5u : 6u;
    cudaError_t e;
#define MIORI_MMA_LAUNCH(OB)                                                                     \
    do {                                                                                         \
        auto kern = gemv_mma_kernel<BITS, EXACT, NT, OB>;                                        \
        e = cudaSuccess;                                                                         \
        if (smem > 48 * 1024)                                                                    \
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e == cudaSuccess)                                                                    \
            e = launch(kern, dim3(grid), dim3(THREADS), smem, stream, pdl,                       \
                       reinterpret_cast<const uint4*>(q), reinterpret_cast<const uint16_t*>(s),  \
                       reinterpret_cast<const uint16_t*>(b), reinterpret_cast<const uint16_t*>(x), \
                       y, N, K, M, gshift);                                                      \
    } while (0)
    if (flags & MIORI_OUT_BF16) MIORI_MMA_LAUNCH(true); else MIORI_MMA_LAUNCH(false);
#undef MIORI_MMA_LAUNCH
    if (e != cudaSuccess) return cuda_fail(e, "gemv_mma launch");
    return MIORI_OK;
}

// True if the tensor-core GEMV can take this problem (otherwise the SIMT path runs).
template <int BITS>
bool supported(uint32_t K, uint32_t M, bool force_exact) {
    const size_t limit = 200 * 1024;
    if (M <= 2) return smem_bytes<BITS, true, 1>(K) <= limit;
    if (M <= 4) return smem_bytes<BITS, true, 2>(K) <= limit;
    if (force_exact || BITS == 8) return false;
    if (M <= 8) return smem_bytes<4, false, 1>(K) <= limit;
    if (M <= 16) return smem_bytes<4, false, 2>(K) <= limit;
    return smem_bytes<4, false, 4>(K) <= limit;
}

template <int BITS>
int launch(const void* q, const void* s, const void* b, const void* x, void* y, uint32_t N,
           uint32_t K, uint32_t M, uint32_t group, uint32_t flags, cudaStream_t stream) {
    if (M <= 2) return launch_one<BITS, true, 1>(q, s, b, x, y, N, K, M, group, flags, stream);
    if (M <= 4) return launch_one<BITS, true, 2>(q, s, b, x, y, N, K, M, group, flags, stream);
    if (M <= 8) return launch_one<4, false, 1>(q, s, b, x, y, N, K, M, group, flags, stream);
    if (M <= 16) return launch_one<4, false, 2>(q, s, b, x, y, N, K, M, group, flags, stream);
    return launch_one<4, false, 4>(q, s, b, x, y, N, K, M, group, flags, stream);
}

}  // namespace gemvmma
}  // namespace miori_b200
