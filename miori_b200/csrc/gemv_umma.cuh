// Decode GEMV on the 5th-generation tensor cores, weights streamed packed from HBM.
//
// y[m][n] = sum_g s[n][g] * (sum_{k in g} code[n][k] * x[m][k]) + b[n][g] * sum_{k in g} x[m][k]
//
// The inner sums are what a tensor core is for, so they run as tcgen05.mma with the WEIGHTS as
// the A operand held in tensor memory and the activations as a small B operand in shared memory:
//   * a tile is 128 output rows (= the 128 TMEM lanes); a stage is 128 codes of every row of the
//     tile (64 bytes per row, 8 KiB), brought into a shared-memory ring by one 2-D TMA copy
//     (64-byte swizzle, so the thread that owns row r reads its 16-byte pieces conflict-free);
//   * thread r of an unpack warpgroup turns its row's 4-bit codes into bf16 pairs 128+code
//     (one LOP3 per pair, shifts apart) and writes them with tcgen05.st into the A slot of its
//     warpgroup: 64 TMEM columns per stage.  Nothing but packed codes ever crosses shared memory;
//   * one thread issues eight 128 x 16 x 16 MMAs per stage (A from TMEM, B = the staged x through
//     a no-swizzle K-major descriptor).  Every scale group gets its own 16- or 32-column fp32
//     accumulator, so D[row][m] is the raw sum of (128+code) * x over ONE group;
//   * the same thread r reads its row's accumulators back (tcgen05.ld) and applies the fp32 scale
//     and bias of the group itself: y += s*D + (b - 128*s) * sum(x).  That is fp32 dequantization
//     and fp32 accumulation, the arithmetic class of the reference's gemv4 / gemv4_b
//     (shaders/ops.metal:6-42, shaders/batch.metal:145-188), for every M from 1 to 32; a row's
//     value depends neither on M nor on the number of CTAs.
// Two unpack warpgroups (4 warps each: a warp may only touch its own 32 TMEM lanes) take
// alternate stages; their partial sums are added in a fixed order at the end of a tile.
//
// Shapes with few tiles split K over the CTAs of a thread-block cluster: CTA r of the cluster
// handles k in [r*kc, (r+1)*kc), and the partials meet through distributed shared memory -- CTA r
// receives rows [r*128/cs, (r+1)*128/cs) of every peer, adds them in rank order and stores them.
//
// Weights are immutable, so under programmatic dependent launch the ring is filled and the first
// stages are unpacked BEFORE the kernel waits for its predecessor; only the staging of x and
// everything after it is ordered behind griddepcontrol.wait.  Every wait on a barrier is bounded.
#pragma once
#include "common.cuh"
#include "tma_host.cuh"

#include <algorithm>

namespace miori_b200 {
namespace gemvumma {

constexpr int TILE_N = 128;                       // rows per tile = TMEM lanes
constexpr int KS = 128;                           // codes per row and stage
constexpr int STAGE_BYTES = TILE_N * KS / 2;      // 8 KiB of packed codes
constexpr int A_COLS = KS / 2;                    // TMEM columns of one unpacked stage (bf16 pairs)
constexpr int UNPACK_WARPS = 8;                   // two warpgroups of four
constexpr int STAGER_WARPS = 4;                   // stage x, then issue the MMAs
constexpr int WARP_TMA = UNPACK_WARPS, WARP_STAGE0 = UNPACK_WARPS + 1;
constexpr int THREADS = (UNPACK_WARPS + 1 + STAGER_WARPS) * 32;  // 416
constexpr int STAGERS = STAGER_WARPS * 32;
constexpr int MAX_RING = 24;
constexpr int X_BLOCK_PAD = 16;  // bytes between consecutive 8-k blocks of the staged x beyond
                                 // their rows: consecutive blocks land in different bank groups

// ---- tensor-memory access of one warp: 32 lanes x X consecutive 32-bit columns ---------------
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15])
        : "memory");
}
template <int X>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[X]) {
    static_assert(X == 1 || X == 4 || X == 8 || X == 16 || X == 32, "column counts in use");
    if constexpr (X == 1) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r[0]) : "r"(taddr) : "memory");
    } else if constexpr (X == 4) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
    } else if constexpr (X == 8) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                       "=r"(r[6]), "=r"(r[7]) : "r"(taddr) : "memory");
    } else if constexpr (X == 16) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
              "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
              "=r"(r[13]), "=r"(r[14]), "=r"(r[15]) : "r"(taddr) : "memory");
    } else {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
              "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
              "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
              "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
              "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
              "=r"(r[31]) : "r"(taddr) : "memory");
    }
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[tmem] * B[smem descriptor]: 128 x N x 16, bf16 operands, fp32 accumulators.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                        uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same, issued by one elected lane of a converged warp: operands then stay in the uniform
// datapath, which issues a good deal faster than a lone lane of a diverged warp.
__device__ __forceinline__ void umma_ts_elect(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                              uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_arrive(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(bar)
                 : "memory");
}
// K-major operand without swizzle: 8-row x 16-byte core matrices, `lbo` bytes between the two
// core matrices along K, `sbo` bytes between 8-row groups.
__device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version of sm_100
    return d;
}
__device__ __forceinline__ uint32_t lop3_and_or_u(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a&b)|c
    return r;
}
__device__ __forceinline__ uint4 lds_v4(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds_v2(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void bar_named(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void cluster_arrive_wait() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;"
                 ::: "memory");
}
// store into the same shared-memory offset of CTA `rank` of this cluster
__device__ __forceinline__ void st_cluster_f32(uint32_t local_addr, uint32_t rank, float v) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "st.shared::cluster.f32 [ra], %2;\n\t}"
        ::"r"(local_addr), "r"(rank), "f"(v)
        : "memory");
}

#ifdef MIORI_UMMA_TRACE
// Cycle counters of CTA 0 for profiling by hand (a build with -DMIORI_UMMA_TRACE only).
__device__ long long g_umma_trace[32];
#define UMMA_T0(var) const long long var = clock64()
#define UMMA_ADD(slot, var) do { tr_acc[slot] += clock64() - (var); } while (0)
#define UMMA_DECL long long tr_acc[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}
#define UMMA_FLUSH(lo, hi) do { if (blockIdx.x == 0 && lane == 0) for (int z = lo; z <= hi; ++z) g_umma_trace[z] = tr_acc[z]; } while (0)
#else
#define UMMA_T0(var) do { } while (0)
#define UMMA_ADD(slot, var) do { } while (0)
#define UMMA_DECL do { } while (0)
#define UMMA_FLUSH(lo, hi) do { } while (0)
#endif

// Launch geometry, decided on the host.
struct Geo {
    uint32_t N, K, M;
    uint32_t gshift;     // 5 or 6: log2 of the scale group
    uint32_t kc;         // codes per row handled by one CTA (K / cs), a multiple of KS
    uint32_t cs;         // CTAs per cluster = K splits (1, 2, 4 or 8)
    uint32_t ring;       // stages of the code ring
    uint32_t nb;         // TMEM slots per warpgroup (1 or 2)
    uint32_t tmem_cols;  // power of two >= 32
    uint32_t sb_box;     // scales per row delivered by one TMA box (a multiple of 8)
    uint32_t sb_bufs;    // scale buffers: 2 when a CTA walks several tiles, else 1
    uint32_t out_bf16;
    uint32_t n_total;    // row pitch of y in elements (N, or the whole output when sharded)
    uint32_t row0;       // first output column of this launch inside y
    uint32_t clusters;   // clusters in the grid (host side only)
};

// Shared-memory carve-up (bytes from a 1024-byte aligned base), identical on host and device.
struct Smem {
    uint32_t ring, sb, xs, xsum, wgred, recv, total;
};
template <int MACC>
__host__ __device__ inline Smem smem_layout(const Geo& g) {
    constexpr uint32_t NCS = MACC <= 8 ? 8u : (MACC <= 16 ? 16u : 32u);  // staged rows of x
    Smem s;
    uint32_t at = 0;
    s.ring = at;
    at += g.ring * STAGE_BYTES;
    s.sb = at;  // [tiles in flight][scale, bias][128 rows][sb_box] bf16
    at += g.sb_bufs * 2u * TILE_N * g.sb_box * 2u;
    at = (at + 1023u) & ~1023u;
    s.xs = at;  // [kc/8 blocks][NCS rows][16 bytes] + pad per block, + one spare block
    at += (g.kc / 8u + 1u) * (NCS * 16u + X_BLOCK_PAD);
    at = (at + 127u) & ~127u;
    s.xsum = at;  // [kc >> gshift groups][MACC] fp32
    at += (g.kc >> g.gshift) * MACC * 4u;
    at = (at + 127u) & ~127u;
    s.wgred = at;  // [2][128 rows][MACC] fp32: second warpgroup's partials, alternating per tile
    at += 2u * TILE_N * MACC * 4u;
    s.recv = at;   // [cs][128 / cs rows][MACC] fp32: partials received from the cluster
    at += g.cs > 1u ? TILE_N * MACC * 4u : 0u;
    s.total = at + 1024u;  // slack for aligning the base
    return s;
}

template <int MACC>
__global__ void __launch_bounds__(THREADS, MACC <= 8 ? 2 : 1)
gemv_umma_kernel(const __grid_constant__ CUtensorMap tmap_q,
                 const __grid_constant__ CUtensorMap tmap_s,
                 const __grid_constant__ CUtensorMap tmap_b, const uint16_t* __restrict__ x,
                 void* __restrict__ y, const Geo geo) {
    constexpr uint32_t NCS = MACC <= 8 ? 8u : (MACC <= 16 ? 16u : 32u);  // staged rows of x
    constexpr uint32_t NC = MACC <= 16 ? 16u : 32u;                        // MMA N = columns per group
    constexpr uint32_t XBLK = NCS * 16u + X_BLOCK_PAD;                      // bytes per 8-k block of x
    constexpr uint32_t MASK = 0x000F000Fu, MAGIC = 0x43004300u;             // bf16 128.0 in both halves
    // instruction descriptor: D = f32, A = B = bf16, both K-major, shape 128 x NC
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((NC >> 3) << 17) | ((128u >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bars[MAX_RING];
    __shared__ __align__(8) uint64_t empty_bars[MAX_RING];
    __shared__ __align__(8) uint64_t sb_full[2], sb_empty[2];
    __shared__ __align__(8) uint64_t a_ready[2][2], mma_done[2][2];
    __shared__ __align__(8) uint64_t x_ready;
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile uint32_t abort_flag;

    const Smem L = smem_layout<MACC>(geo);
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t N = geo.N, M = geo.M, gshift = geo.gshift, kc = geo.kc, cs = geo.cs;
    const uint32_t gps = (uint32_t)KS >> gshift;         // scale groups per stage: 2 or 4
    const uint32_t nst = kc / KS;                         // stages per tile
    const uint32_t slot_cols = A_COLS + gps * NC;         // one slot: A stage + its accumulators
    const uint32_t rank = cs > 1u ? blockIdx.x % cs : 0u; // CTA rank in its cluster = K split
    const uint32_t cluster = blockIdx.x / cs, nclusters = gridDim.x / cs;
    const uint32_t tiles = (N + TILE_N - 1) / TILE_N;
    const uint32_t k0 = rank * kc;                        // first code of this CTA's range
    const uint32_t my_tiles = cluster < tiles ? (tiles - cluster + nclusters - 1) / nclusters : 0u;

    pdl_launch_dependents();
    UMMA_T0(t_start);
    UMMA_DECL;

    if (threadIdx.x == 0) {
        abort_flag = 0u;
        for (uint32_t i = 0; i < geo.ring; ++i) {
            mbar_init(smem_addr(&full_bars[i]), 1);
            mbar_init(smem_addr(&empty_bars[i]), 4);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_addr(&sb_full[i]), 1);
            mbar_init(smem_addr(&sb_empty[i]), UNPACK_WARPS);
            for (int j = 0; j < 2; ++j) {
                mbar_init(smem_addr(&a_ready[i][j]), 4);
                mbar_init(smem_addr(&mma_done[i][j]), 2);
            }
        }
        mbar_init(smem_addr(&x_ready), STAGERS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_s) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
    }
    if (warp == WARP_TMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_addr(&tmem_base_slot)), "r"(geo.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    // K split: no CTA may be written to through distributed shared memory before it runs; every
    // thread arrives here and waits right before its first remote store (or at the end)
    bool cluster_waited = false;
    if (cs > 1u) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

    if (warp == WARP_TMA) {
        // ---- producer: scales and biases of a tile, then its code stages, as far ahead as the
        // ring allows.  Nothing here depends on the predecessor kernel.
        if (lane == 0) {
            uint32_t gi = 0;
            bool ok = true;
            // the box starts on the 16-byte boundary at or below this CTA's first scale
            const int sb_c0 = (int)((k0 >> gshift) & ~7u);
            const uint32_t sb_bytes = TILE_N * geo.sb_box * 2u;
            for (uint32_t ti = 0; ti < my_tiles && ok; ++ti) {
                const uint32_t row = (cluster + ti * nclusters) * TILE_N, buf = ti % geo.sb_bufs;
                const uint32_t use = ti / geo.sb_bufs;
                if (use >= 1u) ok = mbar_wait(smem_addr(&sb_empty[buf]), (use - 1u) & 1u, &abort_flag, 0x41);
                if (!ok) break;
                const uint32_t sbar = smem_addr(&sb_full[buf]);
                const uint32_t sdst = base + L.sb + buf * 2u * sb_bytes;
                mbar_expect_tx(sbar, 2u * sb_bytes);
                tma_load_2d(sdst, &tmap_s, sb_c0, (int)row, sbar);
                tma_load_2d(sdst + sb_bytes, &tmap_b, sb_c0, (int)row, sbar);
                for (uint32_t it = 0; it < nst; ++it, ++gi) {
                    const uint32_t r = gi % geo.ring;
                    if (gi >= geo.ring) {
                        UMMA_T0(tw);
                        ok = mbar_wait(smem_addr(&empty_bars[r]), (gi / geo.ring - 1u) & 1u, &abort_flag, 0x42);
                        UMMA_ADD(0, tw);
                        if (!ok) break;
                    }
                    const uint32_t bar = smem_addr(&full_bars[r]);
                    mbar_expect_tx(bar, STAGE_BYTES);
                    tma_load_2d(base + L.ring + r * STAGE_BYTES, &tmap_q, (int)((k0 + it * KS) / 8u),
                                (int)row, bar);
                }
            }
        }
    } else if (warp >= WARP_STAGE0) {
        // ---- x stagers: zero the rows no activation fills, wait for the predecessor, then copy
        // x[m][k0 .. k0 + kc) into the B-operand layout (8-k blocks, the 8 values of a block in the
        // order the unpack gives the codes of a word: 0,4,1,5,2,6,3,7) and add up x per scale
        // group in fp32.
        const uint32_t st = threadIdx.x - WARP_STAGE0 * 32u;
        const uint32_t blocks = kc / 8u;
        const uint32_t xs = base + L.xs;
        for (uint32_t i = st; i < (blocks + 1u) * (XBLK / 16u); i += STAGERS) {
            const uint32_t blk = i / (XBLK / 16u), u = i - blk * (XBLK / 16u);
            if (u >= M || blk == blocks)
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(xs + blk * XBLK + u * 16u), "r"(0u) : "memory");
        }
        pdl_wait_prior();
        const uint32_t lanes_per_group = 1u << (gshift - 3u);  // 8-k blocks per scale group: 4 or 8
        for (uint32_t i0 = st - lane; i0 < M * blocks; i0 += STAGERS) {
            const uint32_t i = i0 + lane;  // blocks is a multiple of 16: a warp never straddles rows unevenly
            const uint32_t m = i / blocks, kb = i - m * blocks;
            float sum = 0.0f;
            if (i < M * blocks) {
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + (size_t)m * geo.K + k0) + kb);
                const uint32_t o0 = __byte_perm(v.x, v.z, 0x5410);  // (x0,x4)
                const uint32_t o1 = __byte_perm(v.x, v.z, 0x7632);  // (x1,x5)
                const uint32_t o2 = __byte_perm(v.y, v.w, 0x5410);  // (x2,x6)
                const uint32_t o3 = __byte_perm(v.y, v.w, 0x7632);  // (x3,x7)
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
                             ::"r"(xs + kb * XBLK + m * 16u), "r"(o0), "r"(o1), "r"(o2), "r"(o3) : "memory");
                sum = ((bf16lo(v.x) + bf16hi(v.x)) + (bf16lo(v.y) + bf16hi(v.y))) +
                      ((bf16lo(v.z) + bf16hi(v.z)) + (bf16lo(v.w) + bf16hi(v.w)));
            }
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
            if (lanes_per_group == 8u) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
            if (i < M * blocks && (kb & (lanes_per_group - 1u)) == 0u)
                asm volatile("st.shared.f32 [%0], %1;"
                             ::"r"(base + L.xsum + ((kb >> (gshift - 3u)) * MACC + m) * 4u), "f"(sum) : "memory");
        }
        // rows of the group sums that no activation fills
        for (uint32_t i = st; i < (kc >> gshift) * MACC; i += STAGERS)
            if (i % MACC >= M)
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(base + L.xsum + i * 4u), "f"(0.0f) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the MMA reads x through the async proxy
        mbar_arrive(smem_addr(&x_ready));
        if (warp == WARP_STAGE0) UMMA_ADD(3, t_start);

        // ---- then the four warps issue the MMAs.  Issuing one tcgen05.mma costs a warp some 50
        // cycles whatever its size, so the eight small MMAs of a stage are shared out: warp iw takes
        // the stages of warpgroup iw >> 1 and, of each, the four k-blocks of half iw & 1.  The two
        // halves of a stage belong to different scale groups, so no accumulator is ever written by
        // two warps and every sum keeps its order.
        const uint32_t iw = warp - WARP_STAGE0, wg = iw >> 1, half = iw & 1u;
        bool ok = mbar_wait(smem_addr(&x_ready), 0u, &abort_flag, 0x43);
        ok = __all_sync(0xFFFFFFFFu, ok);
        const uint32_t per_group = 8u / gps;  // MMAs per scale group: 4 (group 64) or 2 (group 32)
        uint32_t c = 0;                       // stages of this warpgroup issued so far
        for (uint32_t ti = 0; ti < my_tiles && ok; ++ti) {
            for (uint32_t it = wg; it < nst; it += 2u, ++c) {
                const uint32_t slot = c % geo.nb, use = c / geo.nb;
                UMMA_T0(tw);
                ok = mbar_wait(smem_addr(&a_ready[wg][slot]), use & 1u, &abort_flag, 0x44);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (iw == 0) UMMA_ADD(1, tw);
                if (!ok) break;
                UMMA_T0(ti0);
                tc_fence_after();
                const uint32_t a_t = tmem_base + (wg * geo.nb + slot) * slot_cols;
                const uint32_t d_t = a_t + A_COLS;
                const uint32_t xb = base + L.xs + it * 16u * XBLK;
#pragma unroll
                for (uint32_t jj = 0; jj < 4u; ++jj) {
                    const uint32_t j = half * 4u + jj;
                    const uint64_t bdesc = smem_desc_kmajor(xb + j * 2u * XBLK, XBLK, 128u);
                    umma_ts_elect(d_t + (j / per_group) * NC, a_t + j * 8u, bdesc, IDESC, j % per_group);
                }
                if (lane == 0) umma_arrive(smem_addr(&mma_done[wg][slot]));
                __syncwarp();
                if (iw == 0) UMMA_ADD(2, ti0);
            }
        }
    } else {
        // ---- unpack warpgroups: thread = output row of the tile = TMEM lane
        const uint32_t wg = warp >> 2, quad = warp & 3u;
        const uint32_t r = quad * 32u + lane;                       // row inside the tile
        const uint32_t t_lane = tmem_base + ((quad * 32u) << 16);   // this warp's lanes
        const uint32_t q_row = r * 64u, q_swz = (r >> 1) & 3u;      // 64-byte swizzle of the code stage
        const uint32_t sb_pitch = geo.sb_box * 2u;
        // swizzle of the scale rows follows their byte length: 128 -> r & 7, 64 -> (r >> 1) & 3,
        // 32 -> (r >> 2) & 1, 16 -> none
        const uint32_t sb_swz = sb_pitch == 128u ? (r & 7u) : sb_pitch == 64u ? ((r >> 1) & 3u)
                              : sb_pitch == 32u ? ((r >> 2) & 1u) : 0u;
        const uint32_t sb_first = (k0 >> gshift) & 7u;  // this CTA's first scale inside its box
        const uint32_t sb_bytes = TILE_N * sb_pitch;
        float acc[MACC];
#pragma unroll
        for (int m = 0; m < MACC; ++m) acc[m] = 0.0f;
        bool ok = true, have_x = false;
        uint32_t mine = 0;     // stages this warpgroup has unpacked so far (all tiles)
        uint32_t drained = 0;  // ... and read back

        // read back stage number `d` of this warpgroup (tile-local stage index it_d, scale buffer sbuf)
        auto drain = [&](uint32_t d, uint32_t it_d, uint32_t sbuf) {
            const uint32_t slot = d % geo.nb, use = d / geo.nb;
            if (ok && !have_x) {
                UMMA_T0(tx);
                ok = mbar_wait(smem_addr(&x_ready), 0u, &abort_flag, 0x45);
                have_x = true;
                if (warp == 0) UMMA_ADD(9, tx);
            }
            UMMA_T0(tw);
            if (ok) ok = mbar_wait(smem_addr(&mma_done[wg][slot]), use & 1u, &abort_flag, 0x46);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (warp == 0) UMMA_ADD(4, tw);
            if (!ok) return;
            UMMA_T0(td);
            tc_fence_after();
            const uint32_t d_t = t_lane + (wg * geo.nb + slot) * slot_cols + A_COLS;
            // this row's scales and biases of the stage: gps consecutive bf16 each
            const uint32_t off = (sb_first + it_d * gps) * 2u;
            const uint32_t sa = base + L.sb + sbuf * 2u * sb_bytes + r * sb_pitch +
                                (((off >> 4) ^ sb_swz) << 4) + (off & 15u);
            uint32_t sw[2], bw[2];
            if (gps == 2u) {
                sw[0] = lds_u32(sa);
                bw[0] = lds_u32(sa + sb_bytes);
                sw[1] = bw[1] = 0u;
            } else {
                const uint2 s2 = lds_v2(sa), b2 = lds_v2(sa + sb_bytes);
                sw[0] = s2.x; sw[1] = s2.y; bw[0] = b2.x; bw[1] = b2.y;
            }
            const uint32_t xsa = base + L.xsum + it_d * gps * MACC * 4u;
            auto apply = [&](uint32_t gq, const uint32_t (&dv)[MACC]) {
                const uint32_t s16 = (gq & 1u) ? (sw[gq >> 1] >> 16) : (sw[gq >> 1] & 0xFFFFu);
                const uint32_t b16 = (gq & 1u) ? (bw[gq >> 1] >> 16) : (bw[gq >> 1] & 0xFFFFu);
                const float sc = bf16_bits_to_float(s16);
                const float bt = __fmaf_rn(-128.0f, sc, bf16_bits_to_float(b16));
#pragma unroll
                for (int m = 0; m < MACC; ++m) {
                    float xsv;
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(xsv) : "r"(xsa + (gq * MACC + m) * 4u));
                    acc[m] = __fmaf_rn(sc, __uint_as_float(dv[m]), __fmaf_rn(bt, xsv, acc[m]));
                }
            };
            if constexpr (MACC <= 4) {
                // all accumulators of the stage in flight at once
                uint32_t dv[4][MACC];
#pragma unroll
                for (uint32_t gq = 0; gq < 4u; ++gq)
                    if (gq < gps) tmem_ld<MACC>(d_t + gq * NC, dv[gq]);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (uint32_t gq = 0; gq < 4u; ++gq)
                    if (gq < gps) apply(gq, dv[gq]);
            } else {
                // wide batches: one group at a time keeps the register count in bounds
#pragma unroll 1
                for (uint32_t gq = 0; gq < gps; ++gq) {
                    uint32_t dv[MACC];
                    tmem_ld<MACC>(d_t + gq * NC, dv);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    apply(gq, dv);
                }
            }
            tc_fence_before();  // the accumulators may be overwritten once this warp signals again
            if (warp == 0) UMMA_ADD(5, td);
        };

        for (uint32_t ti = 0; ti < my_tiles; ++ti) {
            const uint32_t tile = cluster + ti * nclusters, sbuf = ti % geo.sb_bufs;
            if (ok) ok = mbar_wait(smem_addr(&sb_full[sbuf]), (ti / geo.sb_bufs) & 1u, &abort_flag, 0x47);
            ok = __all_sync(0xFFFFFFFFu, ok);
            uint32_t pend_it[2] = {0u, 0u};  // tile-local stage index of the stages not yet read back
            for (uint32_t it = wg; it < nst; it += 2u) {
                const uint32_t slot = mine % geo.nb;
                if (mine - drained == geo.nb) {  // the slot still holds an undrained stage
                    drain(drained, pend_it[drained % 2u], sbuf);
                    ++drained;
                }
                const uint32_t gi = ti * nst + it, ring = gi % geo.ring;
                UMMA_T0(tf);
                if (ok) ok = mbar_wait(smem_addr(&full_bars[ring]), (gi / geo.ring) & 1u, &abort_flag, 0x48);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (warp == 0) UMMA_ADD(6, tf);
                UMMA_T0(tu);
                if (ok) {
                    const uint32_t st = base + L.ring + ring * STAGE_BYTES + q_row;
                    const uint32_t a_t = t_lane + (wg * geo.nb + slot) * slot_cols;
#pragma unroll
                    for (uint32_t c = 0; c < 4u; ++c) {
                        const uint4 w = lds_v4(st + ((c ^ q_swz) << 4));
                        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
                        uint32_t o[16];
#pragma unroll
                        for (int i = 0; i < 4; ++i)
#pragma unroll
                            for (int p = 0; p < 4; ++p)
                                o[4 * i + p] = lop3_and_or_u(ww[i] >> (4 * p), MASK, MAGIC);
                        tmem_st16(a_t + c * 16u, o);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(smem_addr(&a_ready[wg][slot]));
                        mbar_arrive(smem_addr(&empty_bars[ring]));
                    }
                }
                if (warp == 0) UMMA_ADD(7, tu);
                pend_it[mine % 2u] = it;
                ++mine;
            }
            while (drained < mine) {  // the tile's last stages
                drain(drained, pend_it[drained % 2u], sbuf);
                ++drained;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_addr(&sb_empty[sbuf]));
            UMMA_T0(tt);

            // ---- tile complete: warpgroup 1 hands its partials to warpgroup 0
            const uint32_t wr = base + L.wgred + ((ti & 1u) * TILE_N + r) * MACC * 4u;
            if (wg == 1u) {
#pragma unroll
                for (int m = 0; m < MACC; ++m)
                    asm volatile("st.shared.f32 [%0], %1;" ::"r"(wr + m * 4u), "f"(acc[m]) : "memory");
            }
            bar_named(1u, UNPACK_WARPS * 32u);
            if (wg == 0u) {
#pragma unroll
                for (int m = 0; m < MACC; ++m) {
                    float v;
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(wr + m * 4u));
                    acc[m] += v;
                }
                const uint32_t row = tile * TILE_N + r;
                if (cs == 1u) {
                    if (row < N && ok) {
#pragma unroll
                        for (int m = 0; m < MACC; ++m) {
                            if ((uint32_t)m < M) {
                                const size_t idx = (size_t)m * geo.n_total + geo.row0 + row;
                                if (geo.out_bf16) reinterpret_cast<uint16_t*>(y)[idx] = (uint16_t)float_to_bf16_bits(acc[m]);
                                else reinterpret_cast<float*>(y)[idx] = acc[m];
                            }
                        }
                    }
                } else {
                    // row r is finished by CTA r / rpc of the cluster: partial of K split `rank`
                    if (!cluster_waited) {
                        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
                        cluster_waited = true;
                    }
                    const uint32_t rpc = TILE_N / cs, owner = r / rpc, lr = r - owner * rpc;
                    const uint32_t dst = base + L.recv + ((rank * rpc + lr) * MACC) * 4u;
#pragma unroll
                    for (int m = 0; m < MACC; ++m) st_cluster_f32(dst + m * 4u, owner, acc[m]);
                }
            }
#pragma unroll
            for (int m = 0; m < MACC; ++m) acc[m] = 0.0f;
            if (warp == 0) UMMA_ADD(10, tt);
        }
    }

    if (cs > 1u) {
        // every CTA of the cluster has one tile; the K-split partials of its rows have been written
        // into this CTA's shared memory by all ranks (its own included) once the barrier completes
        __syncwarp();
        if (!cluster_waited) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        cluster_arrive_wait();
        const uint32_t rpc = TILE_N / cs;
        const uint32_t tile = cluster;
        if (tile < tiles && !abort_flag) {
            for (uint32_t i = threadIdx.x; i < rpc * MACC; i += THREADS) {
                const uint32_t m = i / rpc, lr = i - m * rpc;
                float v = 0.0f;
                for (uint32_t src = 0; src < cs; ++src) {
                    float p;
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(p) : "r"(base + L.recv + ((src * rpc + lr) * MACC + m) * 4u));
                    v = src == 0u ? p : v + p;
                }
                const uint32_t row = tile * TILE_N + rank * rpc + lr;
                if (m < M && row < N) {
                    const size_t idx = (size_t)m * geo.n_total + geo.row0 + row;
                    if (geo.out_bf16) reinterpret_cast<uint16_t*>(y)[idx] = (uint16_t)float_to_bf16_bits(v);
                    else reinterpret_cast<float*>(y)[idx] = v;
                }
            }
        }
    }

    // teardown: on abort give copies and MMAs in flight time to land before TMEM is freed
    __syncwarp();
    if (warp == 0) { UMMA_ADD(8, t_start); UMMA_FLUSH(4, 10); }
    if (warp == WARP_TMA) UMMA_FLUSH(0, 0);
    if (warp == WARP_STAGE0) UMMA_FLUSH(1, 3);
    if (abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == WARP_TMA) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"(geo.tmem_cols)
                     : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------------

struct Placement {  // where the output goes when the launch computes a slice of a wider y
    uint32_t n_total = 0, row0 = 0;
};

// Geometry for a problem, or cs == 0 if this kernel cannot take it.  `n_plan` is the row count
// the K split is chosen for (the whole output when the launch is one shard of it, so that a
// row is computed by the same arithmetic on any number of GPUs).
template <int MACC>
inline Geo plan(uint32_t N, uint32_t K, uint32_t M, uint32_t group, uint32_t flags, uint32_t n_plan) {
    Geo g = {};
    g.N = N; g.K = K; g.M = M;
    g.gshift = group == 32 ? 5u : 6u;
    g.out_bf16 = (flags & MIORI_OUT_BF16) ? 1u : 0u;
    g.n_total = N; g.row0 = 0;
    if (K % KS != 0 || (K / group) % 8 != 0 || K / 8 > 0x7FFFFFFFu / 8) return g;
    const uint32_t sms = (uint32_t)sm_count();
    const uint32_t tiles_plan = (n_plan + TILE_N - 1) / TILE_N;
    // K split: double the CTAs per cluster while every CTA still gets an SM of its own and keeps
    // at least 256 codes per row; a CTA's scales must fit one TMA box (256 per row at most)
    uint32_t cs = 1;
    while (cs < 8u && tiles_plan * cs * 2u <= sms && (K / (cs * 2u)) % KS == 0 && K / (cs * 2u) >= 256u) cs *= 2u;
    const uint32_t forced = (flags >> MIORI_TUNE_UMMA_SPLIT_SHIFT) & 15u;  // tuning override
    if (forced == 1u || forced == 2u || forced == 4u || forced == 8u) {
        if ((K / forced) % KS != 0) return g;
        cs = forced;
    }
    while ((K / cs) / group + 7u > 256u && cs < 8u && (K / (cs * 2u)) % KS == 0) cs *= 2u;
    if ((K / cs) / group + 7u > 256u) return g;
    const uint32_t tiles = (N + TILE_N - 1) / TILE_N;
    g.cs = cs;
    g.kc = K / cs;
    // a CTA's scales start (k0 / group) % 8 elements into its TMA box, which begins on a 16-byte
    // boundary: the box covers up to 7 scales more than the CTA uses when K splits unevenly
    const uint32_t per_cta = g.kc / group;
    const uint32_t lead = (cs > 1u && per_cta % 8u != 0u) ? 7u : 0u;
    g.sb_box = (per_cta + lead + 7u) / 8u * 8u;
    const uint32_t gps = KS / group;
    constexpr uint32_t NC = MACC <= 16 ? 16u : 32u;
    const uint32_t slot_cols = A_COLS + gps * NC;
    // two TMEM slots per warpgroup when one CTA owns the SM, one when two CTAs share it
    const bool compact = MACC <= 8;
    g.nb = 2;
    uint32_t cols = 2u * g.nb * slot_cols;
    if (compact && cols > 256u) { g.nb = 1; cols = 2u * slot_cols; }
    if (cols > 512u) { g.nb = 1; cols = 2u * slot_cols; }
    uint32_t pc = 32;
    while (pc < cols) pc *= 2u;
    g.tmem_cols = pc;
    // ring: what shared memory allows (half an SM for the compact instantiations), at most what
    // the CTA will ever stream
    const uint32_t nst = g.kc / KS;
    // long streams run two CTAs per SM (the compact instantiations are sized for half an SM)
    g.clusters = cs > 1u ? tiles : std::min<uint32_t>(tiles, (compact && tiles >= 4u * sms) ? 2u * sms : sms);
    const uint32_t tiles_cta = (tiles + g.clusters - 1) / g.clusters;
    g.sb_bufs = tiles_cta > 1u ? 2u : 1u;
    g.ring = 1;
    const size_t fixed = smem_layout<MACC>(g).total - STAGE_BYTES;
    // half an SM where that leaves room for four stages, else the whole SM
    const size_t budget = (compact && fixed + 4u * STAGE_BYTES <= 110u * 1024u) ? 110u * 1024u : 220u * 1024u;
    if (fixed + 2u * STAGE_BYTES > budget) { g.cs = 0; return g; }
    uint32_t ring = (uint32_t)((budget - fixed) / STAGE_BYTES);
    ring = std::min<uint32_t>(ring, (uint32_t)MAX_RING);
    ring = std::min<uint32_t>(ring, std::max<uint32_t>(2u, nst * tiles_cta));
    g.ring = ring;
    return g;
}

template <int MACC>
inline int launch_one(const Geo& g, const void* q, const void* s, const void* b, const void* x, void* y,
                      uint32_t group, uint32_t flags, cudaStream_t stream) {
    CUtensorMap tq, ts, tb;
    int rc = make_tmap_2d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, g.K / 8, g.N, KS / 8, TILE_N,
                          CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
    const uint32_t sb_bytes = g.sb_box * 2u;
    const CUtensorMapSwizzle sw = sb_bytes == 128u ? CU_TENSOR_MAP_SWIZZLE_128B
                                : sb_bytes == 64u  ? CU_TENSOR_MAP_SWIZZLE_64B
                                : sb_bytes == 32u  ? CU_TENSOR_MAP_SWIZZLE_32B
                                                   : CU_TENSOR_MAP_SWIZZLE_NONE;
    rc = make_tmap_2d(&ts, s, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, g.K / group, g.N, g.sb_box, TILE_N, sw);
    if (rc) return rc;
    rc = make_tmap_2d(&tb, b, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, g.K / group, g.N, g.sb_box, TILE_N, sw);
    if (rc) return rc;
    const uint32_t clusters = g.clusters;
    const size_t smem = smem_layout<MACC>(g).total;
    auto kern = gemv_umma_kernel<MACC>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "gemv_umma attribute");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(clusters * g.cs);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned na = 0;
    if (g.cs > 1u) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = g.cs;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (flags & MIORI_LAUNCH_PDL) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    e = cudaLaunchKernelEx(&cfg, kern, tq, ts, tb, reinterpret_cast<const uint16_t*>(x), y, g);
    if (e != cudaSuccess) return cuda_fail(e, "gemv_umma launch");
    return MIORI_OK;
}

// Try this kernel for packed 4-bit weights; returns 1 if the problem is not eligible (nothing
// launched), 0 if launched, negative on failure.
inline int try_launch(const void* q, const void* s, const void* b, const void* x, void* y, uint32_t N,
                      uint32_t K, uint32_t M, uint32_t group, uint32_t flags, cudaStream_t stream,
                      const Placement& pl = Placement()) {
#define MIORI_UMMA_TRY(MA)                                                                  \
    do {                                                                                    \
        Geo g = plan<MA>(N, K, M, group, flags, pl.n_total ? pl.n_total : N);               \
        if (g.cs == 0) return 1;                                                            \
        if (pl.n_total) { g.n_total = pl.n_total; g.row0 = pl.row0; }                       \
        return launch_one<MA>(g, q, s, b, x, y, group, flags, stream);                      \
    } while (0)
    if (M == 1) MIORI_UMMA_TRY(1);
    if (M <= 4) MIORI_UMMA_TRY(4);
    if (M <= 8) MIORI_UMMA_TRY(8);
    if (M <= 16) MIORI_UMMA_TRY(16);
    MIORI_UMMA_TRY(32);
#undef MIORI_UMMA_TRY
}

}  // namespace gemvumma
}  // namespace miori_b200
