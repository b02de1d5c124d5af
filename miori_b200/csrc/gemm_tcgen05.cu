// Prefill GEMM on the 5th-generation tensor cores: C[M][N] = A[M][K] * Bc[N][K]^T,
// bf16 operands (both K-major), fp32 accumulation in tensor memory.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer: 128-byte-swizzled [128 x 64] A and [BN x 64] B tiles into a
//               STAGES-deep shared-memory ring (cp.async.bulk.tensor, mbarrier tx-count)
//   warp 1      MMA issuer: one thread issues tcgen05.mma (128 x BN x 16 per instruction)
//               from shared-memory descriptors into one of two TMEM accumulators;
//               tcgen05.commit releases ring slots and publishes finished accumulators
//   warps 2..5  epilogue: tcgen05.ld the accumulator (lane = row of C, column = column of
//               C), convert, and store 128 contiguous bytes per thread; overlaps the next
//               tile's main loop through the second accumulator
// Tiles are visited in groups of 16 row blocks so that the A rows of a group and the
// whole B matrix stay in L2.  Out-of-range rows/columns are zero-filled by TMA on load and
// masked on store, so any M >= 1 and any N % 8 == 0 work with the same code; a row of C
// therefore never depends on M (the reference's tile-shape invariance, src/main.cpp:1403-1443).
// Every wait is bounded: on expiry the kernel records an error, drains and returns.
#include "common.cuh"
#include "tma_host.cuh"

#include <algorithm>
#include <mutex>

namespace miori_b200 {
namespace gemm {

constexpr int BM = 128;       // rows of C per tile = UMMA M = TMEM lanes
constexpr int BK = 64;        // bf16 per 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int GROUP_M = 16;   // row blocks per L2 group
constexpr int THREADS = 192;
// epilogue staging: each of the four epilogue warps owns two 32-row x 128-byte buffers
constexpr int OUT_BUF_BYTES = 32 * 128;
constexpr int OUT_STAGE_BYTES = 4 * 2 * OUT_BUF_BYTES;

template <int BN>
struct Cfg {
    static constexpr int STAGES = BN == 256 ? 4 : 6;
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TMEM_COLS = 2 * BN;  // two accumulators (256 or 512: powers of two)
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_STAGE_BYTES + 1024 /*alignment slack*/ + 256;
};

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: rows of 128 bytes, 8-row
// atoms 1024 bytes apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);   // start address, 16-byte units
    d |= (uint64_t)1 << 16;                      // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;            // stride byte offset
    d |= (uint64_t)1 << 46;                      // version
    d |= (uint64_t)2 << 61;                      // SWIZZLE_128B
    return d;
}

// Instruction descriptor: D=f32, A=B=bf16, both K-major, shape 128 x BN.
template <int BN>
__device__ __forceinline__ constexpr uint32_t umma_idesc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
           ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

struct TileCoord {
    uint32_t m_blk, n_blk;
};
__device__ __forceinline__ TileCoord tile_coord(uint32_t t, uint32_t m_blocks, uint32_t n_blocks) {
    const uint32_t per_group = GROUP_M * n_blocks;
    const uint32_t group = t / per_group;
    const uint32_t first_m = group * GROUP_M;
    const uint32_t gm = min((uint32_t)GROUP_M, m_blocks - first_m);
    const uint32_t r = t - group * per_group;
    TileCoord c;
    c.m_blk = first_m + r % gm;
    c.n_blk = r / gm;
    return c;
}

// Epilogue of one warp for one tile: its 32 accumulator rows (TMEM lanes) x BN columns go to
// global memory through shared memory and TMA stores, 128 bytes of a row at a time (32 fp32 or
// 64 bf16 columns).  Each lane writes its row's 128 bytes into a 32 x 128-byte buffer with the
// 128-byte swizzle (conflict-free), lane 0 hands the buffer to the TMA engine, and the warp
// moves on to its other buffer; the store clips rows >= M and columns >= N.  `fill` counts the
// buffers this warp has handed over so far (selects the buffer and throttles reuse).
template <bool OUT_BF16, int BN>
__device__ __forceinline__ void epilogue_rows(uint32_t taddr, uint32_t row0, uint32_t col0,
                                              uint32_t M, uint32_t N, bool bf16_out, uint32_t slice,
                                              const CUtensorMap* tmap_c, uint32_t bufs,
                                              uint32_t& fill, uint32_t lane) {
    if (row0 >= M) return;
    const uint32_t sw = lane & 7u;  // swizzle: 16-byte unit u of row r sits at unit u ^ (r & 7)
    const uint32_t cols_per_fill = (OUT_BF16 && bf16_out) ? 64u : 32u;
#pragma unroll 1
    for (uint32_t c = 0; c < (uint32_t)BN && col0 + c < N; c += cols_per_fill) {
        const uint32_t buf = bufs + (fill & 1u) * OUT_BUF_BYTES;
        if (fill >= 2u) {  // the store issued two fills ago must have finished reading this buffer
            if (lane == 0) tma_store_wait_read<1>();
            __syncwarp();
        }
        const uint32_t rowp = buf + lane * 128u;
        uint32_t r[32];
        tmem_ld32(taddr + c, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (OUT_BF16 && bf16_out) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (h == 1) {
                    tmem_ld32(taddr + c + 32u, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t v[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        v[e] = float_to_bf16_bits(__uint_as_float(r[8 * j + 2 * e])) |
                               (float_to_bf16_bits(__uint_as_float(r[8 * j + 2 * e + 1])) << 16);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                 ::"r"(rowp + ((((uint32_t)(4 * h + j)) ^ sw) << 4)), "r"(v[0]),
                                   "r"(v[1]), "r"(v[2]), "r"(v[3])
                                 : "memory");
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                             ::"r"(rowp + ((((uint32_t)j) ^ sw) << 4)), "r"(r[4 * j]),
                               "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3])
                             : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            tma_store_3d(tmap_c, (int)(col0 + c), (int)row0, (int)slice, buf);
            tma_store_commit();
        }
        ++fill;
    }
}

template <int BN, bool OUT_BF16>
__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_c, uint32_t splits, uint32_t M,
                         uint32_t N, uint32_t K, uint32_t a_box_rows) {
    using C = Cfg<BN>;
    // Bytes one k-block delivers: the A box holds only a_box_rows rows when M is small (a box
    // that reaches far past the tensor's last row is served slowly); the rest of the 128-row A
    // region then keeps stale bytes, which only feed accumulator lanes nobody reads.
    const uint32_t stage_tx = a_box_rows * BK * 2u + (uint32_t)C::B_BYTES;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile uint32_t abort_flag;

    const uint32_t raw = smem_addr(smem_raw);
    const uint32_t tiles_base = (raw + 1023u) & ~1023u;            // 1024-byte aligned ring
    const uint32_t out_stage = tiles_base + C::STAGES * C::STAGE_BYTES;  // epilogue staging
    const uint32_t bars = out_stage + OUT_STAGE_BYTES;                    // barriers after it
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * C::STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * C::STAGES + 2 + a); };

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t m_blocks = (M + BM - 1) / BM, n_blocks = (N + BN - 1) / BN;
    // split-K: work item t covers k-blocks [kb0, kb1) of output tile t / splits and writes its
    // fp32 partial to slice t % splits of the workspace (splits == 1: straight to C)
    const uint32_t tiles = m_blocks * n_blocks * splits;
    const uint32_t k_blocks = (K + BK - 1) / BK;  // TMA zero-fills a ragged last block

    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        abort_flag = 0u;
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_c) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_addr(&tmem_base_slot)), "r"((uint32_t)C::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    // A may be produced, and C read, by the preceding kernel.  The cache is immutable, so the
    // producer first issues the B tiles of its first k-blocks (the ring is empty: no waits) and
    // only then joins the wait; under programmatic dependent launch that fetch overlaps the
    // predecessor's tail.
    if (threadIdx.x != 0) pdl_wait_prior();

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0, pre = 0;
            bool ok = true;
            if (blockIdx.x < tiles) {
                const TileCoord tc = tile_coord(blockIdx.x / splits, m_blocks, n_blocks);
                const uint32_t sp = blockIdx.x % splits;
                const uint32_t kb0 = sp * k_blocks / splits, kb1 = (sp + 1u) * k_blocks / splits;
                pre = min((uint32_t)C::STAGES, kb1 - kb0);
                for (uint32_t i = 0; i < pre; ++i) {
                    mbar_expect_tx(full_bar(i), stage_tx);
                    tma_load_2d(tiles_base + i * C::STAGE_BYTES + C::A_BYTES, &tmap_b,
                                (int)((kb0 + i) * BK), (int)(tc.n_blk * BN), full_bar(i));
                }
            }
            pdl_wait_prior();
            for (uint32_t t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const TileCoord tc = tile_coord(t / splits, m_blocks, n_blocks);
                const uint32_t sp = t % splits;
                const uint32_t kb0 = sp * k_blocks / splits, kb1 = (sp + 1u) * k_blocks / splits;
                for (uint32_t kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1u;
                    const uint32_t sa = tiles_base + s * C::STAGE_BYTES;
                    if (it >= pre) {
                        if (!(ok = mbar_wait(empty_bar(s), ph ^ 1u, &abort_flag, 1))) break;
                        mbar_expect_tx(full_bar(s), stage_tx);
                        tma_load_2d(sa + C::A_BYTES, &tmap_b, (int)(kb * BK), (int)(tc.n_blk * BN),
                                    full_bar(s));
                    }
                    tma_load_2d(sa, &tmap_a, (int)(kb * BK), (int)(tc.m_blk * BM), full_bar(s));
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc<BN>();
            uint32_t it = 0, tile_it = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++tile_it) {
                const uint32_t acc = tile_it & 1u, aph = (tile_it >> 1) & 1u;
                if (!(ok = mbar_wait(tempty_bar(acc), aph ^ 1u, &abort_flag, 2))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + acc * BN;
                const uint32_t sp = t % splits;
                const uint32_t kb0 = sp * k_blocks / splits, kb1 = (sp + 1u) * k_blocks / splits;
                for (uint32_t kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1u;
                    if (!(ok = mbar_wait(full_bar(s), ph, &abort_flag, 3))) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = tiles_base + s * C::STAGE_BYTES;
                    const uint64_t adesc = umma_desc_sw128(sa);
                    const uint64_t bdesc = umma_desc_sw128(sa + C::A_BYTES);
#pragma unroll
                    for (uint32_t k = 0; k < BK / UMMA_K; ++k) {
                        // advance 32 bytes (16 bf16) inside the swizzled 128-byte row
                        umma_f16(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb > kb0) || (k != 0u));
                    }
                    umma_commit(empty_bar(s));  // slot reusable once these MMAs have read it
                }
                if (ok) umma_commit(tfull_bar(acc));  // accumulator complete
            }
        }
    } else {
        const uint32_t quad = warp & 3u;  // TMEM lane quadrant this warp may read
        const uint32_t bufs = out_stage + quad * 2u * OUT_BUF_BYTES;
        uint32_t tile_it = 0, fill = 0;
        bool ok = true;
        for (uint32_t t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++tile_it) {
            const TileCoord tc = tile_coord(t / splits, m_blocks, n_blocks);
            const uint32_t acc = tile_it & 1u, aph = (tile_it >> 1) & 1u;
            ok = mbar_wait(tfull_bar(acc), aph, &abort_flag, 4);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // split-K partials are fp32 slices of the workspace; the last argument picks the slice
            epilogue_rows<OUT_BF16, BN>(tmem_base + ((quad * 32u) << 16) + acc * BN,
                                        tc.m_blk * BM + quad * 32u, tc.n_blk * BN, M, N,
                                        splits == 1u, t % splits, &tmap_c, bufs, fill, lane);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
        if (lane == 0) tma_store_wait_all();  // stores complete before shared memory goes away
    }

    // teardown: on abort give in-flight copies and MMAs time to land before freeing TMEM
    __syncwarp();
    if (abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)C::TMEM_COLS)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------
// Two-CTA variant: a cluster of two CTAs (one SM pair) computes a 256 x 256 tile with
// tcgen05.mma.cta_group::2.  CTA r of the pair owns rows [128r, 128r+128) of the tile (its A
// tile and its TMEM accumulator) and loads only rows [128r, 128r+128) of the B tile; the MMA,
// issued by CTA 0, reads both halves of B out of the two CTAs' shared memory.  Per k-block
// every SM therefore pulls 32 KB through L2 for a 128 x 256 x 64 block of work instead of
// 48 KB, which is what keeps the tensor pipe fed.  TMA loads of both CTAs complete on CTA 0's
// "full" barrier (no multicast is involved); CTA 0 releases stages and publishes
// accumulators to both CTAs with tcgen05.commit ... multicast::cluster.
namespace pair {

constexpr int BN = 256;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;         // 16 KB: this CTA's 128 rows of A
constexpr int B_BYTES = (BN / 2) * BK * 2;   // 16 KB: this CTA's 128 rows of B
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 2 * BN;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_STAGE_BYTES + 1024 + 256;
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;"
                 ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                                 uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                              uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive on the same barrier offset in both CTAs of the pair once the MMAs issued so far finish
__device__ __forceinline__ void umma_commit_both(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
        "[%0], %1;"
        ::"r"(bar), "h"(mask)
        : "memory");
}
// arrive on a barrier of CTA 0 from either CTA of the pair
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar_local) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, 0;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(bar_local)
        : "memory");
}

template <bool OUT_BF16>
__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                              const __grid_constant__ CUtensorMap tmap_b,
                              const __grid_constant__ CUtensorMap tmap_c, uint32_t splits,
                              uint32_t M, uint32_t N, uint32_t K) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile uint32_t abort_flag;

    const uint32_t raw = smem_addr(smem_raw);
    const uint32_t tiles_base = (raw + 1023u) & ~1023u;
    const uint32_t out_stage = tiles_base + STAGES * STAGE_BYTES;
    const uint32_t bars = out_stage + OUT_STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t rank = cluster_ctarank();           // 0 = leader of the pair
    const uint32_t pair_id = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const uint32_t m_blocks = (M + 2 * BM - 1) / (2 * BM), n_blocks = (N + BN - 1) / BN;
    const uint32_t tiles = m_blocks * n_blocks * splits;
    const uint32_t k_blocks = (K + BK - 1) / BK;  // TMA zero-fills a ragged last block

    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        abort_flag = 0u;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);    // leader's copy is the one in use: one expect_tx arrival
            mbar_init(empty_bar(s), 1);   // one multicast commit from the leader
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);   // one multicast commit from the leader
            mbar_init(tempty_bar(a), 8);  // leader's copy: four epilogue warps of each CTA
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_c) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_addr(&tmem_base_slot)), "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();  // both CTAs' barriers exist before any remote arrive or multicast commit
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (threadIdx.x != 0) pdl_wait_prior();

    if (warp == 0) {
        if (lane == 0) {
            // producer of this CTA: its A rows and its half of the B rows, both completing on
            // the leader's full barrier.  As in the single-CTA kernel the B tiles of the first
            // k-blocks are issued before the dependency wait.
            uint32_t it = 0, pre = 0;
            bool ok = true;
            if (pair_id < tiles) {
                const TileCoord tc = tile_coord(pair_id / splits, m_blocks, n_blocks);
                const uint32_t sp = pair_id % splits;
                const uint32_t kb0 = sp * k_blocks / splits, kb1 = (sp + 1u) * k_blocks / splits;
                pre = min((uint32_t)STAGES, kb1 - kb0);
                for (uint32_t i = 0; i < pre; ++i) {
                    if (rank == 0) mbar_expect_tx(full_bar(i), 2u * STAGE_BYTES);
                    tma_load_2d_pair(tiles_base + i * STAGE_BYTES + A_BYTES, &tmap_b,
                                     (int)((kb0 + i) * BK), (int)(tc.n_blk * BN + rank * (BN / 2)),
                                     full_bar(i) & PEER_MASK);
                }
            }
            pdl_wait_prior();
            for (uint32_t t = pair_id; t < tiles && ok; t += pairs) {
                const TileCoord tc = tile_coord(t / splits, m_blocks, n_blocks);
                const uint32_t sp = t % splits;
                const uint32_t kb0 = sp * k_blocks / splits, kb1 = (sp + 1u) * k_blocks / splits;
                for (uint32_t kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                    const uint32_t sa = tiles_base + s * STAGE_BYTES;
                    const uint32_t fb = full_bar(s) & PEER_MASK;
                    if (it >= pre) {
                        if (!(ok = mbar_wait(empty_bar(s), ph ^ 1u, &abort_flag, 0x21))) break;
                        if (rank == 0) mbar_expect_tx(full_bar(s), 2u * STAGE_BYTES);
                        tma_load_2d_pair(sa + A_BYTES, &tmap_b, (int)(kb * BK),
                                         (int)(tc.n_blk * BN + rank * (BN / 2)), fb);
                    }
                    tma_load_2d_pair(sa, &tmap_a, (int)(kb * BK),
                                     (int)(tc.m_blk * 2 * BM + rank * BM), fb);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // the pair's single MMA issuer
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                       ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            uint32_t it = 0, tile_it = 0;
            bool ok = true;
            for (uint32_t t = pair_id; t < tiles && ok; t += pairs, ++tile_it) {
                const uint32_t acc = tile_it & 1u, aph = (tile_it >> 1) & 1u;
                if (!(ok = mbar_wait(tempty_bar(acc), aph ^ 1u, &abort_flag, 0x22))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + acc * BN;
                const uint32_t sp = t % splits;
                const uint32_t kb0 = sp * k_blocks / splits, kb1 = (sp + 1u) * k_blocks / splits;
                for (uint32_t kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                    if (!(ok = mbar_wait(full_bar(s), ph, &abort_flag, 0x23))) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = tiles_base + s * STAGE_BYTES;
                    const uint64_t adesc = umma_desc_sw128(sa);
                    const uint64_t bdesc = umma_desc_sw128(sa + A_BYTES);
#pragma unroll
                    for (uint32_t k = 0; k < BK / UMMA_K; ++k)
                        umma_f16_pair(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc,
                                      (kb > kb0) || (k != 0u));
                    umma_commit_both(empty_bar(s));
                }
                if (ok) umma_commit_both(tfull_bar(acc));
            }
        }
    } else {
        const uint32_t quad = warp & 3u;
        const uint32_t bufs = out_stage + quad * 2u * OUT_BUF_BYTES;
        uint32_t tile_it = 0, fill = 0;
        bool ok = true;
        for (uint32_t t = pair_id; t < tiles && ok; t += pairs, ++tile_it) {
            const TileCoord tc = tile_coord(t / splits, m_blocks, n_blocks);
            const uint32_t acc = tile_it & 1u, aph = (tile_it >> 1) & 1u;
            ok = mbar_wait(tfull_bar(acc), aph, &abort_flag, 0x24);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            epilogue_rows<OUT_BF16, BN>(tmem_base + ((quad * 32u) << 16) + acc * BN,
                                        tc.m_blk * 2 * BM + rank * BM + quad * 32u, tc.n_blk * BN,
                                        M, N, splits == 1u, t % splits, &tmap_c, bufs, fill, lane);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(tempty_bar(acc));
        }
        if (lane == 0) tma_store_wait_all();
    }

    __syncwarp();
    if (abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();  // the peer may still signal this CTA's barriers or read its shared memory
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

}  // namespace pair

// Sum the split-K partials in slice order (deterministic) and write C as fp32 or bf16.
template <bool OUT_BF16>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float4* __restrict__ ws, void* __restrict__ Cout, size_t quads,
                     uint32_t splits) {
    pdl_launch_dependents();
    pdl_wait_prior();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads;
         i += (size_t)gridDim.x * blockDim.x) {
        float4 a = ws[i];
        for (uint32_t s = 1; s < splits; ++s) {
            const float4 b = ws[(size_t)s * quads + i];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        if (OUT_BF16) {
            uint2 o;
            o.x = float_to_bf16_bits(a.x) | (float_to_bf16_bits(a.y) << 16);
            o.y = float_to_bf16_bits(a.z) | (float_to_bf16_bits(a.w) << 16);
            reinterpret_cast<uint2*>(Cout)[i] = o;
        } else {
            reinterpret_cast<float4*>(Cout)[i] = a;
        }
    }
}

// Row pitches in elements (0: dense).
struct Ld {
    uint32_t a = 0, b = 0, c = 0;
};

// [rows][K] bf16 row-major (rows `pitch` elements apart, 0: dense), box = [box_rows][64],
// 128-byte swizzle, zero fill out of range.
static int make_tmap(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K,
                     uint32_t box_rows, uint32_t pitch) {
    return make_tmap_2d(map, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, rows, BK, box_rows,
                        CU_TENSOR_MAP_SWIZZLE_128B, pitch);
}

// Tensor map the epilogue stores through: C itself ([1][M][N], fp32 or bf16), or the split-K
// workspace ([splits][M][N] fp32).  Boxes are 32 rows x 128 bytes with the 128-byte swizzle.
static int make_tmap_out(CUtensorMap* map, void* Cm, float* ws, uint32_t M, uint32_t N,
                         uint32_t splits, bool bf16, uint32_t ldc) {
    if (splits > 1)
        return make_tmap_3d(map, ws, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, N, M, splits, 32, 32,
                            CU_TENSOR_MAP_SWIZZLE_128B);
    if (bf16)
        return make_tmap_3d(map, Cm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, M, 1, 64, 32,
                            CU_TENSOR_MAP_SWIZZLE_128B, ldc);
    return make_tmap_3d(map, Cm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, N, M, 1, 32, 32,
                        CU_TENSOR_MAP_SWIZZLE_128B, ldc);
}

// Launch the two-CTA kernel: clusters of 2, one pair per SM pair.
static int launch_gemm_pair(const void* A, const void* Bc, void* Cm, uint32_t M, uint32_t N,
                            uint32_t K, uint32_t flags, float* ws, uint32_t splits,
                            cudaStream_t stream, const Ld& ld) {
    CUtensorMap ta, tb, tc;
    int rc = make_tmap(&ta, A, M, K, BM, ld.a);
    if (rc) return rc;
    rc = make_tmap(&tb, Bc, N, K, pair::BN / 2, ld.b);
    if (rc) return rc;
    rc = make_tmap_out(&tc, Cm, ws, M, N, splits, (flags & MIORI_OUT_BF16) != 0, ld.c);
    if (rc) return rc;
    const uint32_t tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + pair::BN - 1) / pair::BN) * splits;
    uint32_t pairs = (uint32_t)sm_count() / 2;
    if (pairs > tiles) pairs = tiles;
    const bool bf16 = (flags & MIORI_OUT_BF16) != 0, pdl = (flags & MIORI_LAUNCH_PDL) != 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = pair::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 2 : 1;
    cudaError_t e;
    if (bf16) {
        auto kern = pair::gemm_bf16_tcgen05_pair_kernel<true>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::SMEM_BYTES);
        if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, splits, M, N, K);
    } else {
        auto kern = pair::gemm_bf16_tcgen05_pair_kernel<false>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::SMEM_BYTES);
        if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, splits, M, N, K);
    }
    if (e != cudaSuccess) return cuda_fail(e, "gemm_bf16_tcgen05_pair launch");
    return MIORI_OK;
}

// Fixed-order reduction of split-K partials into C.
static int launch_reduce(void* Cm, uint32_t M, uint32_t N, uint32_t flags, float* ws, uint32_t splits,
                         cudaStream_t stream) {
    const bool bf16 = (flags & MIORI_OUT_BF16) != 0, pdl = (flags & MIORI_LAUNCH_PDL) != 0;
    const size_t quads = (size_t)M * N / 4;
    const unsigned blocks = (unsigned)std::min<size_t>((quads + 255) / 256, (size_t)sm_count() * 8);
    cudaError_t e;
    if (bf16)
        e = launch(splitk_reduce_kernel<true>, dim3(blocks), dim3(256), 0, stream, pdl,
                   reinterpret_cast<const float4*>(ws), Cm, quads, splits);
    else
        e = launch(splitk_reduce_kernel<false>, dim3(blocks), dim3(256), 0, stream, pdl,
                   reinterpret_cast<const float4*>(ws), Cm, quads, splits);
    if (e != cudaSuccess) return cuda_fail(e, "splitk_reduce launch");
    return MIORI_OK;
}

template <int BN>
static int launch_gemm(const void* A, const void* Bc, void* Cm, uint32_t M, uint32_t N, uint32_t K,
                       uint32_t flags, float* ws, uint32_t splits, cudaStream_t stream, const Ld& ld) {
    using C = Cfg<BN>;
    CUtensorMap ta, tb, tc;
    const uint32_t a_box = M >= (uint32_t)BM ? (uint32_t)BM : (M + 7u) / 8u * 8u;
    int rc = make_tmap(&ta, A, M, K, a_box, ld.a);
    if (rc) return rc;
    rc = make_tmap(&tb, Bc, N, K, BN, ld.b);
    if (rc) return rc;
    rc = make_tmap_out(&tc, Cm, ws, M, N, splits, (flags & MIORI_OUT_BF16) != 0, ld.c);
    if (rc) return rc;
    const uint32_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * splits;
    uint32_t grid = (uint32_t)sm_count();
    if (grid > tiles) grid = tiles;
    const bool bf16 = (flags & MIORI_OUT_BF16) != 0, pdl = (flags & MIORI_LAUNCH_PDL) != 0;
    cudaError_t e;
    if (bf16) {
        auto kern = gemm_bf16_tcgen05_kernel<BN, true>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e == cudaSuccess)
            e = launch(kern, dim3(grid), dim3(THREADS), (size_t)C::SMEM_BYTES, stream, pdl, ta, tb,
                       tc, splits, M, N, K, a_box);
    } else {
        auto kern = gemm_bf16_tcgen05_kernel<BN, false>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e == cudaSuccess)
            e = launch(kern, dim3(grid), dim3(THREADS), (size_t)C::SMEM_BYTES, stream, pdl, ta, tb,
                       tc, splits, M, N, K, a_box);
    }
    if (e != cudaSuccess) return cuda_fail(e, "gemm_bf16_tcgen05 launch");
    if (splits > 1) return launch_reduce(Cm, M, N, flags, ws, splits, stream);
    return MIORI_OK;
}

// Shape checks shared by the GEMM entries.
static int check_gemm_args(const char* op, const void* A, const void* cache, const void* Cm,
                           uint32_t M, uint32_t N, uint32_t K) {
    if (!A || !cache || !Cm) return fail(MIORI_E_INVALID, "%s: null pointer", op);
    if (M == 0 || N == 0 || K == 0)
        return fail(MIORI_E_INVALID, "%s: empty shape M=%u N=%u K=%u", op, M, N, K);
    if (K % 64 != 0) return fail(MIORI_E_INVALID, "%s: K=%u is not a multiple of 64", op, K);
    if (N % 8 != 0) return fail(MIORI_E_INVALID, "%s: N=%u is not a multiple of 8", op, N);
    if (!aligned16(A) || !aligned16(cache) || !aligned16(Cm))
        return fail(MIORI_E_INVALID, "%s: A, cache and C must be 16-byte aligned", op);
    return MIORI_OK;
}

// Tile shape and split count for a problem (workspace of ws_bytes available, 0 = none).
struct GemmPlan {
    bool wide;   // 128 x 256 tiles instead of 128 x 128 (single-CTA kernel)
    bool pair;   // 256 x 256 tiles on SM pairs (two-CTA kernel)
    uint32_t splits;
};

// The plan is the cheapest of {128x128, 128x256, 256x256-on-pairs} x {1..16 K-splits} under a
// small cost model (microseconds):
//   main loop  = waves x k-blocks per work item x time per k-block of that tile shape, where
//                waves = ceil(work items / SMs or SM pairs) -- but never less than the time
//                HBM needs to deliver the cache and A once;
//   split cost = a second (reduction) kernel plus (splits + 1) passes over M x N fp32.
// The per-k-block times are what the kernels sustain on a B200 when L2 feeds them (bigger tiles
// need fewer bytes per flop): 0.31 us for 128x128, 0.375 us for 128x256, 0.315 us for a
// 256x256 pair tile.  Splitting K therefore happens when the tiles alone would leave most SMs
// idle and K is long enough to pay for the reduction, never below 4 k-blocks per split.
static GemmPlan plan_gemm(uint32_t M, uint32_t N, uint32_t K, uint32_t flags, size_t ws_bytes) {
    const uint32_t sms = (uint32_t)sm_count();
    const uint32_t k_blocks = (K + BK - 1) / BK;
    const size_t mn = (size_t)M * N;
    struct Shape {
        bool wide, pair, allowed;
        uint32_t tiles, units;
        double t_kb;
    };
    const uint32_t m128 = (M + 127) / 128, m256 = (M + 255) / 256;
    const uint32_t n128 = (N + 127) / 128, n256 = (N + 255) / 256;
    const bool force_narrow = flags & MIORI_TUNE_GEMM_NARROW, force_wide = flags & MIORI_TUNE_GEMM_WIDE;
    const bool force_pair = flags & MIORI_TUNE_GEMM_PAIR, no_pair = flags & MIORI_TUNE_GEMM_NOPAIR;
    const bool forced = force_narrow || force_wide || force_pair;
    Shape shapes[3] = {
        {false, false, !forced || force_narrow, m128 * n128, sms, 0.31},
        {true, false, !forced || force_wide, m128 * n256, sms, 0.375},
        {false, true, ((!forced && M > 128) || force_pair) && !no_pair, m256 * n256, sms / 2, 0.315},
    };
    const double t_hbm = ((double)N * K * 2 + (double)M * K * 2) / 6.5e6;  // us at 6.5 TB/s
    uint32_t max_s = std::min<uint32_t>(16, std::max<uint32_t>(1, k_blocks / 4));
    if (!ws_bytes) max_s = 1;
    else if (mn) max_s = (uint32_t)std::min<size_t>(max_s, std::max<size_t>(1, ws_bytes / (mn * 4)));
    GemmPlan best = {false, false, 1};
    double best_t = 1e30;
    const uint32_t force_split = (flags >> MIORI_TUNE_GEMM_SPLIT_SHIFT) & 15u;
    for (const Shape& sh : shapes) {
        if (!sh.allowed) continue;
        for (uint32_t sp = 1; sp <= max_s; ++sp) {
            if (force_split && sp != std::min(force_split, max_s)) continue;
            const uint32_t waves = (sh.tiles * sp + sh.units - 1) / sh.units;
            double t = (double)waves * ((k_blocks + sp - 1) / sp) * sh.t_kb;
            if (t < t_hbm) t = t_hbm;
            if (sp > 1) t += 2.0 + (double)(sp + 1) * mn * 4 / 5e6;
            if (t < best_t * 0.97) {  // a later candidate must win by 3 %: prefers fewer splits
                best_t = t;
                best = {sh.wide, sh.pair, sp};
            }
        }
    }
    return best;
}

static int run_plan(const GemmPlan& p, const void* A, const void* cache, void* Cm, uint32_t M,
                    uint32_t N, uint32_t K, uint32_t flags, float* ws, cudaStream_t stream,
                    const Ld& ld = Ld()) {
    if (p.pair) {
        int rc = launch_gemm_pair(A, cache, Cm, M, N, K, flags, ws, p.splits, stream, ld);
        if (rc == MIORI_OK && p.splits > 1) rc = launch_reduce(Cm, M, N, flags, ws, p.splits, stream);
        return rc;
    }
    if (p.wide) return launch_gemm<256>(A, cache, Cm, M, N, K, flags, ws, p.splits, stream, ld);
    return launch_gemm<128>(A, cache, Cm, M, N, K, flags, ws, p.splits, stream, ld);
}

// Any-stride, any-alignment bf16 GEMM with fp32 accumulation: 32 x 32 output tile per CTA,
// K in steps of 32 through shared memory.  Only for operands the TMA path cannot describe.
template <bool OUT_BF16>
__global__ void __launch_bounds__(256)
gemm_bf16_simt_kernel(const uint16_t* __restrict__ A, const uint16_t* __restrict__ B,
                      void* __restrict__ Cout, uint32_t M, uint32_t N, uint32_t K, uint32_t lda,
                      uint32_t ldb, uint32_t ldc) {
    __shared__ float As[32][33], Bs[32][33];
    pdl_launch_dependents();
    pdl_wait_prior();
    const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;  // ty 0..7
    const uint32_t m0 = blockIdx.y * 32u, n0 = blockIdx.x * 32u;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};  // rows ty, ty+8, ty+16, ty+24 of the tile; column tx
    for (uint32_t k0 = 0; k0 < K; k0 += 32u) {
#pragma unroll
        for (uint32_t r = 0; r < 4u; ++r) {
            const uint32_t row = ty + 8u * r, k = k0 + tx;
            const uint32_t m = m0 + row, n = n0 + row;
            As[row][tx] = (m < M && k < K) ? bf16_bits_to_float(A[(size_t)m * lda + k]) : 0.0f;
            Bs[row][tx] = (n < N && k < K) ? bf16_bits_to_float(B[(size_t)n * ldb + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (uint32_t kk = 0; kk < 32u; ++kk) {
            const float b = Bs[tx][kk];
#pragma unroll
            for (uint32_t r = 0; r < 4u; ++r) acc[r] = __fmaf_rn(As[ty + 8u * r][kk], b, acc[r]);
        }
        __syncthreads();
    }
#pragma unroll
    for (uint32_t r = 0; r < 4u; ++r) {
        const uint32_t m = m0 + ty + 8u * r, n = n0 + tx;
        if (m < M && n < N) {
            if (OUT_BF16)
                reinterpret_cast<uint16_t*>(Cout)[(size_t)m * ldc + n] = (uint16_t)float_to_bf16_bits(acc[r]);
            else
                reinterpret_cast<float*>(Cout)[(size_t)m * ldc + n] = acc[r];
        }
    }
}

}  // namespace gemm
}  // namespace miori_b200

using namespace miori_b200;

MIORI_API int miori_gemm_bf16_cache_ws(const void* A, const void* cache, void* Cm, uint32_t M,
                                       uint32_t N, uint32_t K, uint32_t flags, void* workspace,
                                       size_t workspace_bytes, void* stream) {
    int rc = gemm::check_gemm_args("miori_gemm_bf16_cache", A, cache, Cm, M, N, K);
    if (rc) return rc;
    if (workspace && !aligned16(workspace))
        return fail(MIORI_E_INVALID, "miori_gemm_bf16_cache: workspace must be 16-byte aligned");
    const gemm::GemmPlan p = gemm::plan_gemm(M, N, K, flags, workspace ? workspace_bytes : 0);
    float* ws = reinterpret_cast<float*>(workspace);
    return gemm::run_plan(p, A, cache, Cm, M, N, K, flags, ws, (cudaStream_t)stream);
}

MIORI_API int miori_gemm_bf16_cache(const void* A, const void* cache, void* Cm, uint32_t M,
                                    uint32_t N, uint32_t K, uint32_t flags, void* stream) {
    return miori_gemm_bf16_cache_ws(A, cache, Cm, M, N, K, flags, nullptr, 0, stream);
}

MIORI_API int miori_gemm_bf16_strided(const void* A, uint32_t lda, const void* B, uint32_t ldb, void* Cm,
                                      uint32_t ldc, uint32_t M, uint32_t N, uint32_t K, uint32_t flags,
                                      void* stream) {
    const char* op = "miori_gemm_bf16_strided";
    if (!A || !B || !Cm) return fail(MIORI_E_INVALID, "%s: null pointer", op);
    if (M == 0 || N == 0 || K == 0)
        return fail(MIORI_E_INVALID, "%s: empty shape M=%u N=%u K=%u", op, M, N, K);
    if (lda < K || ldb < K || ldc < N)
        return fail(MIORI_E_INVALID, "%s: a row pitch is shorter than its row (lda=%u ldb=%u K=%u ldc=%u N=%u)",
                    op, lda, ldb, K, ldc, N);
    const bool bf16 = (flags & MIORI_OUT_BF16) != 0, pdl = (flags & MIORI_LAUNCH_PDL) != 0;
    const uint32_t csz = bf16 ? 2 : 4;
    // what the TMA descriptors can express: 16-byte aligned bases and row pitches
    const bool tma_ok = aligned16(A) && aligned16(B) && aligned16(Cm) && lda % 8 == 0 && ldb % 8 == 0 &&
                        ((size_t)ldc * csz) % 16 == 0;
    // TMA stores clip at 16-byte granularity, so the tensor-core kernels take the columns up to
    // the last multiple of 16 bytes and the plain kernel the few that remain
    uint32_t n_done = 0;
    if (tma_ok) {
        const uint32_t n_main = N - N % (16u / csz);
        if (n_main) {
            const gemm::GemmPlan p = gemm::plan_gemm(M, n_main, K, flags, 0);
            gemm::Ld ld;
            ld.a = lda;
            ld.b = ldb;
            ld.c = ldc;
            const int rc = gemm::run_plan(p, A, B, Cm, M, n_main, K, flags, nullptr, (cudaStream_t)stream, ld);
            if (rc) return rc;
        }
        n_done = n_main;
    }
    if (n_done == N) return MIORI_OK;
    const uint16_t* Bp = static_cast<const uint16_t*>(B) + (size_t)n_done * ldb;
    void* Cp = static_cast<uint8_t*>(Cm) + (size_t)n_done * csz;
    const uint32_t n_rest = N - n_done;
    const dim3 grid((n_rest + 31) / 32, (M + 31) / 32);
    cudaError_t e;
    if (bf16)
        e = launch(gemm::gemm_bf16_simt_kernel<true>, grid, dim3(256), 0, (cudaStream_t)stream, pdl,
                   static_cast<const uint16_t*>(A), Bp, Cp, M, n_rest, K, lda, ldb, ldc);
    else
        e = launch(gemm::gemm_bf16_simt_kernel<false>, grid, dim3(256), 0, (cudaStream_t)stream, pdl,
                   static_cast<const uint16_t*>(A), Bp, Cp, M, n_rest, K, lda, ldb, ldc);
    if (e != cudaSuccess) return cuda_fail(e, "gemm_bf16_simt launch");
    return MIORI_OK;
}

// ---- split-K GEMM on built-in scratch ------------------------------------------------------
// Some hosts cannot hand this library a workspace because they cannot allocate device memory
// at the point of the call: a decode loop whose device memory was carved up once at start-up,
// or a plug-in living in a process where another runtime owns the allocator.  For them the
// split-K partials go to this fixed array, which every GPU that loads the library carries
// until the process exits.  Host code must not pass the array's name to a kernel (on the host
// the name is only a stand-in); its device address is looked up once per device below.
constexpr size_t kStaticScratchBytes = (size_t)16 << 20;  // 16 MiB
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];

// Device address of g_static_scratch on the current device (looked up on first use there).  As
// for every launch entry, the device current at the call must be the one the stream belongs to.
static int static_scratch_ptr(float** out) {
    static float* ptrs[64];
    static std::mutex mu;
    int dev = 0;
    MIORI_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(MIORI_E_INVALID, "device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lk(mu);
    if (!ptrs[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        ptrs[dev] = static_cast<float*>(p);
    }
    *out = ptrs[dev];
    return MIORI_OK;
}

MIORI_API size_t miori_gemm_static_scratch_bytes(void) { return kStaticScratchBytes; }

MIORI_API int miori_gemm_bf16_cache_static(const void* A, const void* cache, void* Cm, uint32_t M,
                                           uint32_t N, uint32_t K, uint32_t flags, void* stream) {
    int rc = gemm::check_gemm_args("miori_gemm_bf16_cache_static", A, cache, Cm, M, N, K);
    if (rc) return rc;
    // the split count the shape wants with unlimited scratch decides whether it fits
    const gemm::GemmPlan want = gemm::plan_gemm(M, N, K, flags, ~(size_t)0 >> 1);
    const size_t need = want.splits > 1 ? (size_t)want.splits * M * N * sizeof(float) : 0;
    if (need > kStaticScratchBytes)
        return fail(MIORI_E_INVALID,
                    "miori_gemm_bf16_cache_static: M=%u N=%u K=%u needs %zu bytes of scratch (%u "
                    "K-splits), the built-in scratch holds %zu; miori_gemm_bf16_cache runs the shape "
                    "without a K split and without scratch (miori_gemm_bf16_cache_ws splits it given a "
                    "caller workspace)",
                    M, N, K, need, want.splits, kStaticScratchBytes);
    float* ws = nullptr;
    if (want.splits > 1) {
        rc = static_scratch_ptr(&ws);
        if (rc) return rc;
    }
    // every element of every partial slice is written by the GEMM before the reduction reads
    // it, so the previous call's contents never need clearing
    return gemm::run_plan(want, A, cache, Cm, M, N, K, flags, ws, (cudaStream_t)stream);
}

MIORI_API int miori_gemm_plan(uint32_t M, uint32_t N, uint32_t K, size_t workspace_bytes, uint32_t* tile_n,
                              uint32_t* ctas_per_tile, uint32_t* splits) {
    if (M == 0 || N == 0 || K == 0) return fail(MIORI_E_INVALID, "miori_gemm_plan: empty shape");
    const gemm::GemmPlan p = gemm::plan_gemm(M, N, K, 0, workspace_bytes);
    if (tile_n) *tile_n = (p.wide || p.pair) ? 256u : 128u;
    if (ctas_per_tile) *ctas_per_tile = p.pair ? 2u : 1u;
    if (splits) *splits = p.splits;
    return MIORI_OK;
}

MIORI_API size_t miori_gemm_workspace_bytes(uint32_t M, uint32_t N, uint32_t K) {
    if (M == 0 || N == 0 || K < 64) return 0;
    const gemm::GemmPlan p = gemm::plan_gemm(M, N, K, 0, (size_t)16 * M * N * 4);
    return p.splits > 1 ? (size_t)p.splits * M * N * 4 : 0;
}
