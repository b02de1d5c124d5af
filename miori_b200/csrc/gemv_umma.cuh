// Decode GEMV on the 5th-generation tensor cores, weights streamed packed from HBM.
//
//   y[m][n] = sum_g ( s[n][g] * sum_{k in g} code[n][k] * x[m][k]  +  b[n][g] * sum_{k in g} x[m][k] )
//
// The inner sum over a scale group is an INTEGER dot product once x is written in fixed point, and
// that is how it is computed: tcgen05.mma.kind::i8 with the packed codes as the unsigned 8-bit A
// operand held in tensor memory and the activations as signed 8-bit "limbs" in shared memory.
//   * x: every activation row is scaled by the power of two that puts its largest magnitude just
//     below 2^27 (2^20 for M > 8) and rounded to an integer X = l3*2^21 + l2*2^14 + l1*2^7 + l0
//     with 7-bit limbs (the top one signed).  Each limb of each row is one column of the MMA's B
//     operand, so a 128 x 16 x 32 MMA multiplies 128 weight rows by four activation rows' four
//     limbs.  Products and sums are exact in int32; the drain adds the limbs' sums in fp32, undoes
//     the row's power of two and applies the group's fp32 scale and bias: fp32 dequantization
//     with an exact inner sum, the arithmetic class of the reference's gemv4 / gemv4_b / gemv8
//     (shaders/ops.metal:6-82, shaders/batch.metal:145-236) for every M from 1 to 32.  An
//     activation below 2^-20 (2^-13 for M > 8) of the largest in its row keeps fewer than its
//     eight significant bits: absolute error below 2^-28 (2^-21) of that maximum.
//   * weights: a tile is 128 output rows (= the 128 TMEM lanes); a stage is 128 codes of every row.
//     A shared-memory ring is filled by 2-D TMA copies ("slabs") of 128 rows x (128, 256 or 512
//     bytes + 16): the TMA engine serves a box row by row at a cost that hardly depends on the
//     row's length, so rows are long, and the 16 extra bytes make the row pitch in shared memory
//     16 (mod 128), which spreads the rows over the banks without a swizzle.  Thread r of the unpack warpgroup reads its row's 16-byte pieces
//     (conflict-free thanks to that pitch), splits nibbles into bytes with three instructions per
//     word (8-bit codes need none) and writes them with tcgen05.st into an A slot of 32 TMEM
//     columns.  Nothing but packed codes ever crosses shared memory;
//   * two issuer warps share the four MMAs of a stage (issuing one tcgen05.mma costs a warp some
//     50 cycles whatever its size); every scale group has its own accumulator columns, and a group
//     is only ever written by one warp, in k order;
//   * thread r of the drain warpgroup reads its row's accumulators back (tcgen05.ld) and keeps the
//     running sums of its row.  Unpack, MMA and drain are decoupled through slots in tensor
//     memory, so the three run concurrently on different stages.
// A row's value depends neither on the other rows of the batch nor on the number of CTAs; it is
// the same for every M of a class (M <= 8, M <= 16, M <= 32).
//
// Shapes with few tiles split K over the CTAs of a thread-block cluster: CTA r of the cluster
// handles k in [r*kc, (r+1)*kc), and the partials meet through distributed shared memory -- CTA r
// receives rows [r*128/cs, (r+1)*128/cs) of every peer, adds them in rank order and stores them.
// (Each CTA then scales its slice of a row by the slice's own maximum.)
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

constexpr int TILE_N = 128;     // rows per tile = TMEM lanes
// warp roles: 0-7 unpack (two warpgroups taking alternate stages), 8-11 drain, 12-13 issue,
// 14 TMA producer (and tensor-memory allocation)
constexpr int WG_DRAIN = 8, WARP_ISSUE0 = 12, WARP_TMA = 14;
constexpr int THREADS = 15 * 32;   // 480
constexpr int STAGERS = 6 * 32;    // the drain and issuer warps stage x first
constexpr int MAX_RING = 24;
constexpr int MAX_SLOTS = 4;
constexpr int X_BLOCK_PAD = 16;  // bytes between consecutive 16-k blocks of the staged x beyond
                                 // their rows: consecutive blocks land in different bank groups

template <int BITS, int MACC>
struct Cfg {
    static constexpr int L = MACC <= 8 ? 4 : 3;                     // limbs of an activation
    static constexpr int NC = (MACC * L + 15) / 16 * 16;            // MMA N: (row, limb) columns
    // A stage is 128 bytes of every row: 256 four-bit or 128 eight-bit codes.  Every hand-over
    // between the roles costs on the order of a hundred cycles (a load and a branch on it), so
    // stages are as long as tensor memory allows.
    static constexpr int KS = 1024 / BITS;                          // codes per row and stage
    static constexpr int ROW_BYTES = 128;                           // bytes of one row in a stage
    static constexpr int A_COLS = KS / 4;                           // TMEM columns of a stage (4 codes each)
    static constexpr int MMAS = KS / 32;                            // MMAs per stage: 8 or 4
    // rows of x actually staged per 16-k block: with one activation row only 4 of the MMA's 16
    // columns carry limbs; the second group of 8 then re-reads rows 1..8 (row 8 is the zero pad)
    static constexpr int XROWS = MACC == 1 ? 8 : NC;
    static constexpr int XSBO = MACC == 1 ? 16 : 128;               // bytes between the 8-row groups
    static constexpr int XBLK = XROWS * 16 + X_BLOCK_PAD;           // bytes of one 16-k block of x
    static constexpr int TOP_BIT = 7 * L - 1;                       // |X| < 2^TOP_BIT
};

// ---- tensor-memory access of one warp: 32 lanes x X consecutive 32-bit columns ---------------
template <int X>
__device__ __forceinline__ void tmem_st(uint32_t taddr, const uint32_t* r) {
    static_assert(X == 4 || X == 8, "column counts in use");
    if constexpr (X == 4) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};"
                     ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
    } else {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                     ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]),
                       "r"(r[6]), "r"(r[7]) : "memory");
    }
}
template <int X>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t* r) {
    static_assert(X == 4 || X == 16 || X == 32 || X == 48, "column counts in use");
    if constexpr (X == 4) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
    } else if constexpr (X == 16) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
              "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
              "=r"(r[13]), "=r"(r[14]), "=r"(r[15]) : "r"(taddr) : "memory");
    } else if constexpr (X == 32) {
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
    } else {
        tmem_ld<32>(taddr, r);
        tmem_ld<16>(taddr + 32u, r + 32);
    }
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[tmem] * B[smem descriptor]: 128 x N x 32, 8-bit integer operands, int32
// accumulators; issued by one elected lane of a converged warp (operands then stay in the uniform
// datapath, which issues a good deal faster than a lone lane of a diverged warp).
__device__ __forceinline__ void umma_i8_elect(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                              uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the barrier receives one arrival once every MMA this warp's elected lane issued so far is done
__device__ __forceinline__ void umma_arrive_elect(uint32_t bar) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
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
__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_f32(uint32_t a, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}
__device__ __forceinline__ void sts_v2(uint32_t a, uint32_t v0, uint32_t v1) {
    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(a), "r"(v0), "r"(v1) : "memory");
}
__device__ __forceinline__ void bar_named(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
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

// Bounded wait of a whole (converged) warp on one barrier.  Usually the barrier has completed
// already: one try by all lanes settles that in a few tens of cycles.  Otherwise lane 0 polls
// (bounded) and the rest of the warp waits for its verdict.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort,
                                          uint32_t where, uint32_t lane) {
    if (__all_sync(0xFFFFFFFFu, mbar_try(bar, parity))) return true;
    uint32_t ok = 1u;
    if (lane == 0) ok = mbar_wait(bar, parity, abort, where) ? 1u : 0u;
    ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
    return ok != 0u;
}

#ifdef MIORI_UMMA_TRACE
// Cycle counters of CTA 0 for profiling by hand (a build with -DMIORI_UMMA_TRACE only).
__device__ long long g_umma_trace[32];
#define UMMA_T0(var) const long long var = clock64()
#define UMMA_ADD(slot, var) do { tr_acc[slot] += clock64() - (var); } while (0)
#define UMMA_DECL long long tr_acc[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}
#define UMMA_FLUSH(lo, hi) do { if (blockIdx.x == 0 && lane == 0) for (int z = lo; z <= hi; ++z) g_umma_trace[z] = tr_acc[z]; } while (0)
// event log of CTA 0: ev[type * 64 + stage] = cycles since the kernel started (stores do not stall)
__device__ unsigned int g_umma_ev[16 * 64];
#define UMMA_EV(type, j) do { if (blockIdx.x == 0 && lane == 0 && (j) < 64u) g_umma_ev[(type) * 64 + (j)] = (unsigned int)(clock64() - t_start); } while (0)
#else
#define UMMA_EV(type, j) do { } while (0)
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
    uint32_t ring;       // slabs of the code ring
    uint32_t slab_row;   // bytes of one row's codes in a slab: 128, 256 or 512 (the pitch is 16 more)
    uint32_t na, nd;     // A slots and accumulator slots in tensor memory
    uint32_t tmem_cols;  // 256 or 512
    uint32_t sb_box;     // scales per row delivered by one TMA box (a multiple of 8)
    uint32_t sb_bufs;    // scale buffers: 2 when a CTA walks several tiles, else 1
    uint32_t out_bf16;
    uint32_t n_total;    // row pitch of y in elements (N, or the whole output when sharded)
    uint32_t row0;       // first output column of this launch inside y
    uint32_t clusters;   // clusters in the grid (host side only)
    uint32_t norm;       // 1: x is fp32 and is RMS-normalised (times gamma) while it is staged
    float eps;           // ... with this epsilon
};

// Shared-memory carve-up (bytes from a 1024-byte aligned base), identical on host and device.
struct Smem {
    uint32_t ring, sb, xs, xsum, xinv, recv, total;
};
template <int BITS, int MACC>
__host__ __device__ inline Smem smem_layout(const Geo& g) {
    using C = Cfg<BITS, MACC>;
    Smem s;
    uint32_t at = 0;
    s.ring = at;
    at += g.ring * TILE_N * (g.slab_row + 16u);
    at = (at + 1023u) & ~1023u;  // the scale boxes are swizzled: their pattern follows the address
    s.sb = at;  // [tiles in flight][scale, bias][128 rows][sb_box] bf16
    at += g.sb_bufs * 2u * TILE_N * g.sb_box * 2u;
    at = (at + 1023u) & ~1023u;
    s.xs = at;  // [kc/16 blocks][NC rows][16 bytes] + pad per block, + one spare block
    at += (g.kc / 16u + 1u) * C::XBLK;
    at = (at + 127u) & ~127u;
    s.xsum = at;  // [kc >> gshift groups][MACC] fp32: sum of x over the group
    at += (g.kc >> g.gshift) * MACC * 4u;
    at = (at + 127u) & ~127u;
    s.xinv = at;  // [32] fp32 powers of two that undo the rows' scaling, [32] u32 row maxima, and for
                  // the fused norm [32] fp32 rsqrt(mean + eps) and [32][6] partial sums of squares
    at += (3u * 32u + 32u * 6u) * 4u;
    s.recv = at;  // [cs][128 / cs rows][MACC] fp32: partials received from the cluster
    at += g.cs > 1u ? TILE_N * MACC * 4u : 0u;
    s.total = at + 1024u;  // slack for aligning the base
    return s;
}

template <int BITS, int MACC>
__global__ void __launch_bounds__(THREADS, MACC <= 4 ? 2 : 1)
gemv_umma_kernel(const __grid_constant__ CUtensorMap tmap_q,
                 const __grid_constant__ CUtensorMap tmap_s,
                 const __grid_constant__ CUtensorMap tmap_b, const uint16_t* __restrict__ x,
                 const float* __restrict__ xnorm, const uint16_t* __restrict__ gamma,
                 void* __restrict__ y, const Geo geo) {
    using C = Cfg<BITS, MACC>;
    constexpr uint32_t L = C::L, NC = C::NC, XBLK = C::XBLK, KS = C::KS, A_COLS = C::A_COLS;
    // instruction descriptor: D = s32, A = u8, B = s8, both K-major, shape 128 x NC
    constexpr uint32_t IDESC = (2u << 4) | (0u << 7) | (1u << 10) | ((NC >> 3) << 17) | ((128u >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bars[MAX_RING];
    __shared__ __align__(8) uint64_t empty_bars[MAX_RING];
    __shared__ __align__(8) uint64_t sb_full[2], sb_empty[2];
    // stage j may be issued once its A slot is filled (four unpack warps arrive) and its
    // accumulator slot has been read back (four drain warps arrive): go[j % 4]
    __shared__ __align__(8) uint64_t go[MAX_SLOTS];
    __shared__ __align__(8) uint64_t mma_done[MAX_SLOTS];  // stage j completes mma_done[j % 4]
    __shared__ __align__(8) uint64_t x_ready;
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile uint32_t abort_flag;

    const Smem Ls = smem_layout<BITS, MACC>(geo);
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t N = geo.N, M = geo.M, gshift = geo.gshift, kc = geo.kc, cs = geo.cs;
    const uint32_t gps = KS >> gshift;                   // scale groups per stage: 2, 4 or 8
    const uint32_t nst = kc / KS;                         // stages per tile
    const uint32_t d_cols = gps * NC;                     // accumulator columns of one stage
    const uint32_t rank = cs > 1u ? blockIdx.x % cs : 0u; // CTA rank in its cluster = K split
    const uint32_t cluster = blockIdx.x / cs, nclusters = gridDim.x / cs;
    const uint32_t tiles = (N + TILE_N - 1) / TILE_N;
    const uint32_t k0 = rank * kc;                        // first code of this CTA's range
    const uint32_t my_tiles = cluster < tiles ? (tiles - cluster + nclusters - 1) / nclusters : 0u;
    const uint32_t total_stages = my_tiles * nst;
    const uint32_t slab_pitch = geo.slab_row + 16u, slab_bytes = TILE_N * slab_pitch;
    const uint32_t sps = geo.slab_row / (uint32_t)C::ROW_BYTES;  // stages per slab

    pdl_launch_dependents();
    UMMA_T0(t_start);
    UMMA_DECL;

    if (threadIdx.x == 0) {
        abort_flag = 0u;
        for (uint32_t i = 0; i < geo.ring; ++i) {
            mbar_init(smem_addr(&full_bars[i]), 1);
            mbar_init(smem_addr(&empty_bars[i]), sps >= 2u ? 8u : 4u);  // every unpack warp that reads the slab
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_addr(&sb_full[i]), 1);
            mbar_init(smem_addr(&sb_empty[i]), 4);
        }
        for (int i = 0; i < MAX_SLOTS; ++i) {
            mbar_init(smem_addr(&go[i]), 8);
            mbar_init(smem_addr(&mma_done[i]), 2);
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
    const uint32_t tmem_d0 = tmem_base + geo.na * A_COLS;  // accumulator slots follow the A slots
    // K split: no CTA may be written to through distributed shared memory before it runs; every
    // thread arrives here and waits right before its first remote store (or at the end)
    bool cluster_waited = false;
    if (cs > 1u) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

    if (warp == WARP_TMA) {
        // ---- producer: scales and biases of a tile, then its code stages, as far ahead as the
        // ring allows.  Nothing here depends on the predecessor kernel.
        if (lane == 0) {
            uint32_t r = 0, r_par = 1u;  // ring slot and the parity of its previous release
            bool ok = true, wrapped = false;
            // the box starts on the 16-byte boundary at or below this CTA's first scale
            const int sb_c0 = (int)((k0 >> gshift) & ~7u);
            const uint32_t sb_bytes = TILE_N * geo.sb_box * 2u;
            for (uint32_t ti = 0; ti < my_tiles && ok; ++ti) {
                const uint32_t row = (cluster + ti * nclusters) * TILE_N, buf = geo.sb_bufs == 2u ? (ti & 1u) : 0u;
                const uint32_t use = geo.sb_bufs == 2u ? (ti >> 1) : ti;
                if (use >= 1u) ok = mbar_wait(smem_addr(&sb_empty[buf]), (use - 1u) & 1u, &abort_flag, 0x41);
                if (!ok) break;
                const uint32_t sbar = smem_addr(&sb_full[buf]);
                const uint32_t sdst = base + Ls.sb + buf * 2u * sb_bytes;
                mbar_expect_tx(sbar, 2u * sb_bytes);
                tma_load_2d(sdst, &tmap_s, sb_c0, (int)row, sbar);
                tma_load_2d(sdst + sb_bytes, &tmap_b, sb_c0, (int)row, sbar);
                for (uint32_t it = 0; it < nst; it += sps) {
                    if (wrapped) {
                        UMMA_T0(tw);
                        ok = mbar_wait(smem_addr(&empty_bars[r]), r_par, &abort_flag, 0x42);
                        UMMA_ADD(0, tw);
                        if (!ok) break;
                    }
                    const uint32_t bar = smem_addr(&full_bars[r]);
                    mbar_expect_tx(bar, slab_bytes);
                    tma_load_2d(base + Ls.ring + r * slab_bytes, &tmap_q,
                                (int)((k0 + it * KS) * BITS / 32u), (int)row, bar);
                    if (++r == geo.ring) { r = 0; r_par ^= 1u; wrapped = true; }
                }
            }
        }
    } else if (warp < WG_DRAIN) {
        // ---- unpack warpgroup: thread = output row of the tile = TMEM lane.  Packed codes of the
        // stage -> one byte per code -> A slot.  A 4-bit word (codes n0..n7) becomes the two
        // columns (n0,n2,n4,n6) and (n1,n3,n5,n7); x is staged in the same order.
        const uint32_t ug = warp >> 2, quad = warp & 3u;  // unpack warpgroup; TMEM lane quarter
        const uint32_t r = quad * 32u + lane;
        const uint32_t t_lane = tmem_base + ((quad * 32u) << 16);
        const uint32_t q_row = r * slab_pitch;
        bool ok = true, new_slab = true;
        // stage j of the CTA lives in slab j / sps (ring slot `ring`), part j % sps (`half`)
        uint32_t ring = 0, ring_par = 0, half = ug, sa = ug;
        while (half >= sps) { half -= sps; if (++ring == geo.ring) { ring = 0; ring_par ^= 1u; } }
        if (sa >= geo.na) sa -= geo.na;
        for (uint32_t j = ug; j < total_stages; j += 2u) {
            UMMA_T0(tf);
            if (ok && new_slab) ok = warp_wait(smem_addr(&full_bars[ring]), ring_par, &abort_flag, 0x48, lane);
            if (warp == 0) { UMMA_ADD(6, tf); UMMA_EV(0, j); }
            UMMA_T0(ta);
            // the MMAs that read this A slot last (stage j - na) must have completed
            if (ok && j >= geo.na)
                ok = warp_wait(smem_addr(&mma_done[(j - geo.na) & 3u]), ((j - geo.na) >> 2) & 1u, &abort_flag, 0x49, lane);
            if (warp == 0) { UMMA_ADD(4, ta); UMMA_EV(1, j); }
            if (!ok) break;
            UMMA_T0(tu);
            tc_fence_after();
            const uint32_t st = base + Ls.ring + ring * slab_bytes + q_row + half * (uint32_t)C::ROW_BYTES;
            const uint32_t a_t = t_lane + sa * A_COLS;
            if constexpr (BITS == 4) {
#pragma unroll
                for (uint32_t c4 = 0; c4 < 8u; c4 += 4u) {
                    uint4 w[4];
#pragma unroll
                    for (uint32_t c = 0; c < 4u; ++c) w[c] = lds_v4(st + ((c4 + c) << 4));
#pragma unroll
                    for (uint32_t c = 0; c < 4u; ++c) {
                        uint32_t o[8];
                        o[0] = w[c].x & 0x0F0F0F0Fu; o[1] = (w[c].x >> 4) & 0x0F0F0F0Fu;
                        o[2] = w[c].y & 0x0F0F0F0Fu; o[3] = (w[c].y >> 4) & 0x0F0F0F0Fu;
                        o[4] = w[c].z & 0x0F0F0F0Fu; o[5] = (w[c].z >> 4) & 0x0F0F0F0Fu;
                        o[6] = w[c].w & 0x0F0F0F0Fu; o[7] = (w[c].w >> 4) & 0x0F0F0F0Fu;
                        tmem_st<8>(a_t + (c4 + c) * 8u, o);
                    }
                }
            } else {
#pragma unroll
                for (uint32_t c4 = 0; c4 < 8u; c4 += 4u) {
                    uint4 w[4];
#pragma unroll
                    for (uint32_t c = 0; c < 4u; ++c) w[c] = lds_v4(st + ((c4 + c) << 4));
#pragma unroll
                    for (uint32_t c = 0; c < 4u; ++c) {
                        const uint32_t o[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
                        tmem_st<4>(a_t + (c4 + c) * 4u, o);
                    }
                }
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            const bool last_here = half + 2u >= sps;  // this warpgroup's last stage inside the slab
            if (lane == 0) {
                mbar_arrive(smem_addr(&go[j & 3u]));
                if (last_here) mbar_arrive(smem_addr(&empty_bars[ring]));
            }
            if (warp == 0) { UMMA_ADD(7, tu); UMMA_EV(2, j); }
            sa += 2u;
            if (sa >= geo.na) sa -= geo.na;
            half += 2u;
            new_slab = false;
            while (half >= sps) {
                half -= sps;
                new_slab = true;
                if (++ring == geo.ring) { ring = 0; ring_par ^= 1u; }
            }
        }
    } else if (warp < WARP_TMA) {
        // ---- the drain warpgroup and the two issuer warps first stage x
        const uint32_t st = threadIdx.x - WG_DRAIN * 32u;
        const uint32_t units = kc / 8u;         // 16-byte pieces (8 activations) per row
        const uint32_t xs = base + Ls.xs;
        const uint32_t xinv_a = base + Ls.xinv, xmax_a = xinv_a + 32u * 4u;
        // rows of the B operand no activation fills (and the spare block) must read as zero
        {
            const uint32_t per_blk = XBLK / 16u, blocks = kc / 16u;
            for (uint32_t i = st; i < (blocks + 1u) * per_blk; i += STAGERS) {
                const uint32_t blk = i / per_blk, u = i - blk * per_blk;
                if (u >= M * L || blk == blocks)  // (the pad unit after the rows included)
                    asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(xs + blk * XBLK + u * 16u), "r"(0u) : "memory");
            }
            if (st < 32u) asm volatile("st.shared.u32 [%0], %1;" ::"r"(xmax_a + st * 4u), "r"(0u) : "memory");
            for (uint32_t i = st; i < (kc >> gshift) * MACC; i += STAGERS)
                if (i % MACC >= M) sts_f32(base + Ls.xsum + i * 4u, 0.0f);
        }
        bar_named(2u, STAGERS);
        pdl_wait_prior();
        if (warp == WG_DRAIN) UMMA_EV(7, 62u);
        // Fused RMSNorm (shaders/ops.metal:86-115): the activations arrive as fp32; the CTA adds up
        // the squares of each WHOLE row (whatever slice of K it multiplies) in a fixed order, and a
        // unit is then read as bf16(x * rsqrt(mean + eps) * gamma), the value the stand-alone norm
        // would have written for the GEMV to read.
        const uint32_t rinv_a = xmax_a + 32u * 4u;  // [32] fp32: rsqrt(mean(x^2) + eps) per row
        if (geo.norm) {
            const uint32_t part_a = rinv_a + 32u * 4u;  // [32 rows][6 warps] partial sums
            const uint32_t sw = st >> 5;
            for (uint32_t m = 0; m < M; ++m) {
                float ss = 0.0f;
                const float4* row = reinterpret_cast<const float4*>(xnorm + (size_t)m * geo.K);
                for (uint32_t i = st; i < geo.K / 4u; i += STAGERS) {
                    const float4 v = __ldg(row + i);
                    ss = __fmaf_rn(v.x, v.x, ss); ss = __fmaf_rn(v.y, v.y, ss);
                    ss = __fmaf_rn(v.z, v.z, ss); ss = __fmaf_rn(v.w, v.w, ss);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
                if (lane == 0) sts_f32(part_a + (m * 6u + sw) * 4u, ss);
            }
            bar_named(2u, STAGERS);
            if (st < M) {
                float tot = 0.0f;
#pragma unroll
                for (uint32_t w6 = 0; w6 < 6u; ++w6) tot += lds_f32(part_a + (st * 6u + w6) * 4u);
                sts_f32(rinv_a + st * 4u, rsqrtf(tot / (float)geo.K + geo.eps));
            }
            bar_named(2u, STAGERS);
        }
        // one unit = 8 consecutive activations of row m as bf16 pairs
        auto load_unit = [&](uint32_t m, uint32_t u) -> uint4 {
            if (!geo.norm) return __ldg(reinterpret_cast<const uint4*>(x + (size_t)m * geo.K + k0) + u);
            const float4* p = reinterpret_cast<const float4*>(xnorm + (size_t)m * geo.K + k0 + u * 8u);
            const float4 a = __ldg(p), b4 = __ldg(p + 1);
            const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma + k0 + u * 8u));
            const float inv = lds_f32(rinv_a + m * 4u);
            uint4 o;
            o.x = float_to_bf16_bits(a.x * inv * bf16lo(g.x)) | (float_to_bf16_bits(a.y * inv * bf16hi(g.x)) << 16);
            o.y = float_to_bf16_bits(a.z * inv * bf16lo(g.y)) | (float_to_bf16_bits(a.w * inv * bf16hi(g.y)) << 16);
            o.z = float_to_bf16_bits(b4.x * inv * bf16lo(g.z)) | (float_to_bf16_bits(b4.y * inv * bf16hi(g.z)) << 16);
            o.w = float_to_bf16_bits(b4.z * inv * bf16lo(g.w)) | (float_to_bf16_bits(b4.w * inv * bf16hi(g.w)) << 16);
            return o;
        };
        // pass 1: the largest magnitude of every row (bf16 bit patterns order like magnitudes)
        for (uint32_t m = 0; m < M; ++m) {
            uint32_t mx = 0;
            for (uint32_t i = st; i < units; i += STAGERS) {
                const uint4 v = load_unit(m, i);
                const uint32_t a = v.x & 0x7FFF7FFFu, b = v.y & 0x7FFF7FFFu, c = v.z & 0x7FFF7FFFu,
                               d = v.w & 0x7FFF7FFFu;
                mx = max(max(max(mx, a & 0xFFFFu), max(a >> 16, b & 0xFFFFu)),
                         max(max(b >> 16, c & 0xFFFFu), max(max(c >> 16, d & 0xFFFFu), d >> 16)));
            }
            mx = __reduce_max_sync(0xFFFFFFFFu, mx);
            if (lane == 0 && mx) asm volatile("red.shared.max.u32 [%0], %1;" ::"r"(xmax_a + m * 4u), "r"(mx) : "memory");
        }
        bar_named(2u, STAGERS);
        // pass 2: limbs and group sums
        const uint32_t lanes_per_group = 1u << (gshift - 3u);  // units per scale group: 4 or 8
        for (uint32_t m = 0; m < M; ++m)
        for (uint32_t u0 = st - lane; u0 < units; u0 += STAGERS) {
            const uint32_t u = u0 + lane;  // units is a multiple of 16: lane groups never straddle it
            float sum = 0.0f;
            if (u < units) {
                const uint4 v = load_unit(m, u);
                const uint32_t top = lds_u32(xmax_a + m * 4u);
                // the row's largest magnitude, in [2^E, 2^(E+1)), lands in [2^(TOP_BIT-1), 2^TOP_BIT)
                int sh = top >= 0x80u ? (int)C::TOP_BIT - 1 - ((int)(top >> 7) - 127) : 0;
                sh = max(-100, min(100, sh));
                const float mul = __uint_as_float((uint32_t)(127 + sh) << 23);
                if (u == 0u) sts_f32(xinv_a + m * 4u, __uint_as_float((uint32_t)(127 - sh) << 23));
                const float xf[8] = {bf16lo(v.x), bf16hi(v.x), bf16lo(v.y), bf16hi(v.y),
                                     bf16lo(v.z), bf16hi(v.z), bf16lo(v.w), bf16hi(v.w)};
                sum = ((xf[0] + xf[1]) + (xf[2] + xf[3])) + ((xf[4] + xf[5]) + (xf[6] + xf[7]));
                // W[e]: the limbs of activation e, one per byte (top limb signed)
                uint32_t W[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t X = (uint32_t)__float2int_rn(xf[e] * mul);
                    if constexpr (L == 4)
                        W[e] = (X & 0x7Fu) | ((X << 1) & 0x7F00u) | ((X << 2) & 0x7F0000u) | ((X << 3) & 0xFF000000u);
                    else
                        W[e] = (X & 0x7Fu) | ((X << 1) & 0x7F00u) | ((X << 2) & 0xFF0000u);
                }
                // byte order inside the unit: the order the unpack gives a word's codes
                // (4-bit: 0,2,4,6 then 1,3,5,7; 8-bit: 0..7)
                constexpr int S = BITS == 4 ? 2 : 1, O = BITS == 4 ? 1 : 4;
                const uint32_t dst = xs + (u >> 1) * XBLK + (m * L) * 16u + (u & 1u) * 8u;
#pragma unroll
                for (uint32_t l = 0; l < L; ++l) {
                    const uint32_t sel = 0x4040u + l * 0x11u;  // byte l of both operands
                    const uint32_t lo = __byte_perm(__byte_perm(W[0], W[S], sel),
                                                    __byte_perm(W[2 * S], W[3 * S], sel), 0x5410);
                    const uint32_t hi = __byte_perm(__byte_perm(W[O], W[O + S], sel),
                                                    __byte_perm(W[O + 2 * S], W[O + 3 * S], sel), 0x5410);
                    sts_v2(dst + l * 16u, lo, hi);
                }
            }
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
            if (lanes_per_group == 8u) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
            if (u < units && (u & (lanes_per_group - 1u)) == 0u)
                sts_f32(base + Ls.xsum + ((u >> (gshift - 3u)) * MACC + m) * 4u, sum);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the MMA reads x through the async proxy
        mbar_arrive(smem_addr(&x_ready));
        if (warp == WG_DRAIN) { UMMA_ADD(3, t_start); UMMA_EV(7, 0u); }
        bool ok = warp_wait(smem_addr(&x_ready), 0u, &abort_flag, 0x43, lane);

        if (warp >= WARP_ISSUE0) {
            // ---- issuers: warp h issues the first or the second half of every stage's MMAs.  A scale
            // group is one or two consecutive MMAs and never straddles the halves: an accumulator is
            // only ever written by one warp, in k order.
            const uint32_t h = warp - WARP_ISSUE0;
            // MMAs per scale group: group / 32 = 2 or 1; their log2
            const uint32_t pg_shift = gshift - 5u;
            uint32_t sa = 0, sd = 0, it = 0;
            for (uint32_t j = 0; j < total_stages && ok; ++j) {
                UMMA_T0(tw);
                ok = warp_wait(smem_addr(&go[j & 3u]), (j >> 2) & 1u, &abort_flag, 0x44, lane);
                if (h == 0) { UMMA_ADD(1, tw); UMMA_EV(3, j); }
                if (!ok) break;
                UMMA_T0(ti0);
                tc_fence_after();
                const uint32_t a_t = tmem_base + sa * A_COLS;
                const uint32_t d_t = tmem_d0 + sd * d_cols;
                const uint32_t xb = xs + it * (KS / 16u) * XBLK;  // KS / 16 blocks of 16 k per stage
#pragma unroll
                for (uint32_t jj = 0; jj < (uint32_t)C::MMAS / 2u; ++jj) {
                    const uint32_t q = h * ((uint32_t)C::MMAS / 2u) + jj;
                    const uint64_t bdesc = smem_desc_kmajor(xb + q * 2u * XBLK, XBLK, (uint32_t)C::XSBO);
                    umma_i8_elect(d_t + (q >> pg_shift) * NC, a_t + q * 8u, bdesc, IDESC,
                                  q & ((1u << pg_shift) - 1u));
                }
                umma_arrive_elect(smem_addr(&mma_done[j & 3u]));
                if (h == 0) { UMMA_ADD(2, ti0); UMMA_EV(4, j); }
                if (++sa == geo.na) sa = 0;
                if (++sd == geo.nd) sd = 0;
                if (++it == nst) it = 0;
            }
        } else {
            // ---- drain warpgroup: thread = output row.  accs[m] collects s * (integer sum), accb[m]
            // collects b * sum(x); the row's power of two is undone once, at the end of the tile.
            const uint32_t dw = warp - WG_DRAIN;
            const uint32_t r = dw * 32u + lane;
            const uint32_t t_lane = tmem_d0 + ((dw * 32u) << 16);
            const uint32_t sb_pitch = geo.sb_box * 2u;
            // swizzle of the scale rows follows their byte length: 128 -> r & 7, 64 -> (r >> 1) & 3,
            // 32 -> (r >> 2) & 1, anything else -> none
            const uint32_t sb_swz = sb_pitch == 128u ? (r & 7u) : sb_pitch == 64u ? ((r >> 1) & 3u)
                                  : sb_pitch == 32u ? ((r >> 2) & 1u) : 0u;
            const uint32_t sb_first = (k0 >> gshift) & 7u;  // this CTA's first scale inside its box
            const uint32_t sb_bytes = TILE_N * sb_pitch;
            float accs[MACC], accb[MACC];
#pragma unroll
            for (int m = 0; m < MACC; ++m) accs[m] = accb[m] = 0.0f;
            uint32_t j = 0, sd = 0;
            // the first nd stages find their accumulator slots free
            if (lane == 0)
                for (uint32_t z = 0; z < geo.nd && z < total_stages; ++z) mbar_arrive(smem_addr(&go[z & 3u]));
            for (uint32_t ti = 0; ti < my_tiles; ++ti) {
                const uint32_t tile = cluster + ti * nclusters, sbuf = geo.sb_bufs == 2u ? (ti & 1u) : 0u;
                if (ok) ok = warp_wait(smem_addr(&sb_full[sbuf]), (geo.sb_bufs == 2u ? (ti >> 1) : ti) & 1u, &abort_flag, 0x47, lane);
                for (uint32_t it = 0; it < nst; ++it, ++j) {
                    UMMA_T0(tw);
                    if (ok) ok = warp_wait(smem_addr(&mma_done[j & 3u]), (j >> 2) & 1u, &abort_flag, 0x46, lane);
                    if (dw == 0) { UMMA_ADD(9, tw); UMMA_EV(5, j); }
                    if (!ok) break;
                    UMMA_T0(td);
                    tc_fence_after();
                    // this row's scales and biases of the stage: gps consecutive bf16 each, read one by
                    // one (the row's first scale need not sit on a 16-byte boundary when K is split)
                    const uint32_t sb_row = base + Ls.sb + sbuf * 2u * sb_bytes + r * sb_pitch;
                    const uint32_t e0 = sb_first + it * gps;
                    const uint32_t xsa = base + Ls.xsum + it * gps * MACC * 4u;
                    const uint32_t d_t = t_lane + sd * d_cols;
                    // scale and bias of group gq of the stage
                    auto group_sb = [&](uint32_t gq, float& sc, float& bi) {
                        const uint32_t off = (e0 + gq) * 2u;
                        const uint32_t a = sb_row + (((off >> 4) ^ sb_swz) << 4) + (off & 15u);
                        uint32_t s16, b16;
                        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(s16) : "r"(a));
                        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(b16) : "r"(a + sb_bytes));
                        sc = bf16_bits_to_float(s16);
                        bi = bf16_bits_to_float(b16);
                    };
                    // rows mb .. mb + MB - 1 of group gq from their MB * L accumulator columns
                    auto apply = [&](uint32_t gq, int mb, int MB, const uint32_t* dv, float sc, float bi) {
#pragma unroll
                        for (int m = 0; m < MB; ++m) {
                            float v = (float)(int)dv[m * L + L - 1];
#pragma unroll
                            for (int l = (int)L - 2; l >= 0; --l)
                                v = __fmaf_rn(v, 128.0f, (float)(int)dv[m * L + l]);
                            accs[mb + m] = __fmaf_rn(sc, v, accs[mb + m]);
                            accb[mb + m] = __fmaf_rn(bi, lds_f32(xsa + (gq * MACC + mb + m) * 4u), accb[mb + m]);
                        }
                    };
                    if constexpr (MACC == 1) {
                        // few columns: every group's accumulators in flight at once
                        uint32_t dv[8][MACC * L];
#pragma unroll
                        for (uint32_t gq = 0; gq < 8u; ++gq)
                            if (gq < gps) tmem_ld<MACC * L>(d_t + gq * NC, dv[gq]);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (uint32_t gq = 0; gq < 8u; ++gq) {
                            if (gq < gps) {
                                float sc, bi;
                                group_sb(gq, sc, bi);
                                apply(gq, 0, MACC, dv[gq], sc, bi);
                            }
                        }
                    } else {
#pragma unroll 1
                        for (uint32_t gq = 0; gq < gps; ++gq) {
                            float sc, bi;
                            group_sb(gq, sc, bi);
                            constexpr int MB = MACC < 16 ? MACC : 16;  // up to 16 activation rows at a time
#pragma unroll
                            for (int mb = 0; mb < MACC; mb += MB) {
                                uint32_t dv[MB * L];
                                tmem_ld<MB * L>(d_t + gq * NC + mb * L, dv);
                                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                                apply(gq, mb, MB, dv, sc, bi);
                            }
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    // the slot is free for stage j + nd
                    if (lane == 0 && j + geo.nd < total_stages) mbar_arrive(smem_addr(&go[(j + geo.nd) & 3u]));
                    if (dw == 0) { UMMA_ADD(5, td); UMMA_EV(6, j); }
                    if (++sd == geo.nd) sd = 0;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_addr(&sb_empty[sbuf]));
                UMMA_T0(tt);
                // ---- tile complete
                const uint32_t row = tile * TILE_N + r;
                if (cs == 1u) {
                    if (row < N && ok) {
#pragma unroll
                        for (int m = 0; m < MACC; ++m) {
                            if ((uint32_t)m < M) {
                                const float v = __fmaf_rn(accs[m], lds_f32(xinv_a + m * 4u), accb[m]);
                                const size_t idx = (size_t)m * geo.n_total + geo.row0 + row;
                                if (geo.out_bf16) reinterpret_cast<uint16_t*>(y)[idx] = (uint16_t)float_to_bf16_bits(v);
                                else reinterpret_cast<float*>(y)[idx] = v;
                            }
                        }
                    }
                } else {
                    // row r is finished by CTA r / rpc of the cluster: partial of K split `rank`
                    if (!cluster_waited) {
                        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
                        cluster_waited = true;
                    }
                    const uint32_t rpc_shift = 7u - (31u - (uint32_t)__clz((int)cs)), rpc = 1u << rpc_shift;
                    const uint32_t owner = r >> rpc_shift, lr = r & (rpc - 1u);
                    const uint32_t dst = base + Ls.recv + ((rank * rpc + lr) * MACC) * 4u;
#pragma unroll
                    for (int m = 0; m < MACC; ++m)
                        st_cluster_f32(dst + m * 4u, owner,
                                       (uint32_t)m < M ? __fmaf_rn(accs[m], lds_f32(xinv_a + m * 4u), accb[m]) : 0.0f);
                }
#pragma unroll
                for (int m = 0; m < MACC; ++m) accs[m] = accb[m] = 0.0f;
                if (dw == 0) { UMMA_ADD(10, tt); UMMA_EV(7, 1u + ti); }
            }
        }
    }

    if (cs > 1u) {
        // every CTA of the cluster has one tile; the K-split partials of its rows have been written
        // into this CTA's shared memory by all ranks (its own included) once the barrier completes
        __syncwarp();
        if (!cluster_waited) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        const uint32_t rpc_shift = 7u - (31u - (uint32_t)__clz((int)cs)), rpc = 1u << rpc_shift;
        const uint32_t tile = cluster;
        if (tile < tiles && !abort_flag) {
            for (uint32_t i = threadIdx.x; i < rpc * MACC; i += THREADS) {
                const uint32_t m = i >> rpc_shift, lr = i & (rpc - 1u);
                float v = 0.0f;
                for (uint32_t src = 0; src < cs; ++src) {
                    const float p = lds_f32(base + Ls.recv + ((src * rpc + lr) * MACC + m) * 4u);
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
    if (warp == 0) { UMMA_ADD(8, t_start); UMMA_FLUSH(4, 4); UMMA_FLUSH(6, 8); UMMA_EV(7, 63u); }
    if (warp == WARP_TMA) UMMA_FLUSH(0, 0);
    if (warp == WARP_ISSUE0) UMMA_FLUSH(1, 2);
    if (warp == WG_DRAIN) { UMMA_FLUSH(3, 3); UMMA_FLUSH(5, 5); UMMA_FLUSH(9, 10); }
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
    const void* gamma = nullptr;  // not NULL: x is fp32 and gets the fused RMSNorm with this weight
    float eps = 0.0f;
};

// Geometry for a problem, or cs == 0 if this kernel cannot take it.  `n_plan` is the row count
// the K split is chosen for (the whole output when the launch is one shard of it, so that a
// row is computed by the same arithmetic on any number of GPUs).
template <int BITS, int MACC>
inline Geo plan(uint32_t N, uint32_t K, uint32_t M, uint32_t group, uint32_t flags, uint32_t n_plan) {
    using C = Cfg<BITS, MACC>;
    Geo g = {};
    g.N = N; g.K = K; g.M = M;
    g.gshift = group == 32 ? 5u : 6u;
    g.out_bf16 = (flags & MIORI_OUT_BF16) ? 1u : 0u;
    g.n_total = N; g.row0 = 0;
    constexpr uint32_t KSLOT = 128u * 8u / BITS;  // codes in 128 bytes: the shortest slab row
    if (K % KSLOT != 0 || (K / group) % 8 != 0 || K > (1u << 24)) return g;
    const uint32_t sms = (uint32_t)sm_count();
    const uint32_t tiles_plan = (n_plan + TILE_N - 1) / TILE_N;
    const uint32_t tiles = (N + TILE_N - 1) / TILE_N;
    const uint32_t gps = C::KS / group;
    const bool compact = MACC <= 8;
    // K split: double the CTAs per cluster while every CTA still gets an SM of its own and keeps
    // at least 256 codes per row.  The split is a function of the shape and of the class of M
    // only, because a row's partial sums meet in split order.
    uint32_t cs = 1;
    while (cs < 8u && tiles_plan * cs * 2u <= sms && (K / (cs * 2u)) % KSLOT == 0 && K / (cs * 2u) >= 256u) cs *= 2u;
    const uint32_t forced = (flags >> MIORI_TUNE_UMMA_SPLIT_SHIFT) & 15u;  // tuning override
    if (forced == 1u || forced == 2u || forced == 4u || forced == 8u) {
        if ((K / forced) % KSLOT != 0) return g;
        cs = forced;
    }
    for (;; cs *= 2u) {
        if (cs > 8u || (K / cs) % KSLOT != 0) return g;
        g.cs = cs;
        g.kc = K / cs;
        // a CTA's scales start (k0 / group) % 8 elements into its TMA box, which begins on a
        // 16-byte boundary: the box covers up to 7 scales more than the CTA uses when K splits unevenly
        const uint32_t per_cta = g.kc / group;
        const uint32_t lead = (cs > 1u && per_cta % 8u != 0u) ? 7u : 0u;
        g.sb_box = (per_cta + lead + 7u) / 8u * 8u;
        g.clusters = cs > 1u ? tiles : std::min<uint32_t>(tiles, sms);
        g.sb_bufs = tiles > g.clusters ? 2u : 1u;
        g.ring = 2;
        // slab rows: 256 bytes when the CTA's share of a row divides into them, else 128
        g.slab_row = (g.kc * BITS / 8u) % 256u == 0u ? 256u : 128u;
        // the staged activations and the scales must leave room for two slabs
        if (g.sb_box <= 256u && smem_layout<BITS, MACC>(g).total <= 220u * 1024u) break;
        if (forced) { g.cs = 0; return g; }
    }
    // tensor memory: A slots of 32 columns, accumulator slots of gps * NC columns.  Half of it
    // (256 columns) when that leaves two accumulator slots, so that two CTAs can share an SM.
    const uint32_t d_cols = gps * C::NC;
    constexpr uint32_t A_COLS = C::A_COLS;
    uint32_t cols = 256;
    if (!compact || 2u * A_COLS + 2u * d_cols > 256u) cols = 512;
    if (2u * A_COLS + d_cols > cols) { g.cs = 0; return g; }
    g.na = 4;
    while (g.na > 2u && g.na * A_COLS + 2u * d_cols > cols) --g.na;
    g.nd = std::max<uint32_t>(1u, std::min<uint32_t>((uint32_t)MAX_SLOTS, (cols - g.na * A_COLS) / d_cols));
    g.tmem_cols = cols;
    // ring: what shared memory allows, at most what the CTA will ever stream.  The compact
    // instantiations take half an SM when two slabs fit there, so that two CTAs share an SM: the
    // next kernel of a dependent-launch chain beside this one, or, for long streams, two CTAs of
    // this kernel (the grid then has two CTAs per SM).
    const size_t half_sm = 110u * 1024u, whole_sm = 220u * 1024u;
    bool halved = false;
    // Only for 4-bit codes: with 8-bit codes, one activation row and two CTAs per SM a launch
    // ended in a failure on a B200 whose cause reading the code has not shown, so 8-bit weights
    // always take the whole SM.
    if (compact && cols == 256u && BITS == 4) {
        Geo h = g;
        if (cs == 1u && tiles >= 4u * sms) {  // long stream: two CTAs per SM
            h.clusters = std::min<uint32_t>(tiles, 2u * sms);
            h.sb_bufs = 2u;
        }
        h.ring = 2;
        if (smem_layout<BITS, MACC>(h).total > half_sm) h.slab_row = 128u;  // shorter slabs, same ring depth
        if (smem_layout<BITS, MACC>(h).total <= half_sm) {
            g = h;
            halved = true;
        }
    }
    g.ring = 2;
    const size_t slab = (size_t)TILE_N * (g.slab_row + 16u);
    const size_t fixed = smem_layout<BITS, MACC>(g).total - 2u * slab;
    const uint32_t nst = g.kc * BITS / 8u / g.slab_row;  // slabs per tile
    const uint32_t tiles_cta = (tiles + g.clusters - 1) / g.clusters;
    uint32_t ring = (uint32_t)(((halved ? half_sm : whole_sm) - fixed) / slab);
    ring = std::min<uint32_t>(ring, (uint32_t)MAX_RING);
    ring = std::min<uint32_t>(ring, std::max<uint32_t>(2u, nst * tiles_cta));
    g.ring = ring;
    return g;
}

template <int BITS, int MACC>
inline int launch_one(const Geo& g, const void* q, const void* s, const void* b, const void* x, void* y,
                      uint32_t group, uint32_t flags, cudaStream_t stream, const void* gamma = nullptr) {
    using C = Cfg<BITS, MACC>;
    CUtensorMap tq, ts, tb;
    int rc = make_tmap_2d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, (uint64_t)g.K * BITS / 32, g.N,
                          g.slab_row / 4u + 4u, TILE_N, CU_TENSOR_MAP_SWIZZLE_NONE);
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
    const size_t smem = smem_layout<BITS, MACC>(g).total;
    auto kern = gemv_umma_kernel<BITS, MACC>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "gemv_umma attribute");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(g.clusters * g.cs);
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
    // with the fused norm x is fp32 and travels in its own parameter
    e = cudaLaunchKernelEx(&cfg, kern, tq, ts, tb, reinterpret_cast<const uint16_t*>(g.norm ? nullptr : x),
                           reinterpret_cast<const float*>(g.norm ? x : nullptr),
                           reinterpret_cast<const uint16_t*>(gamma), y, g);
    if (e != cudaSuccess) return cuda_fail(e, "gemv_umma launch");
    return MIORI_OK;
}

// Try this kernel; returns 1 if the problem is not eligible (nothing launched), 0 if launched,
// negative on failure.
template <int BITS>
inline int try_launch(const void* q, const void* s, const void* b, const void* x, void* y, uint32_t N,
                      uint32_t K, uint32_t M, uint32_t group, uint32_t flags, cudaStream_t stream,
                      const Placement& pl = Placement()) {
#define MIORI_UMMA_TRY(MA)                                                                  \
    do {                                                                                    \
        Geo g = plan<BITS, MA>(N, K, M, group, flags, pl.n_total ? pl.n_total : N);         \
        if (g.cs == 0) return 1;                                                            \
        if (pl.n_total) { g.n_total = pl.n_total; g.row0 = pl.row0; }                       \
        if (pl.gamma) { g.norm = 1u; g.eps = pl.eps; }                                      \
        return launch_one<BITS, MA>(g, q, s, b, x, y, group, flags, stream, pl.gamma);      \
    } while (0)
    if (M == 1) MIORI_UMMA_TRY(1);
    if (M <= 4) MIORI_UMMA_TRY(4);
    if (M <= 8) MIORI_UMMA_TRY(8);
    if (M <= 16) MIORI_UMMA_TRY(16);
    {
        Geo g = plan<BITS, 32>(N, K, M, group, flags, pl.n_total ? pl.n_total : N);
        if (g.cs != 0) {
            if (pl.n_total) { g.n_total = pl.n_total; g.row0 = pl.row0; }
            if (pl.gamma) { g.norm = 1u; g.eps = pl.eps; }
            return launch_one<BITS, 32>(g, q, s, b, x, y, group, flags, stream, pl.gamma);
        }
    }
    // the 32-row instantiation does not fit tensor memory (4-bit codes with group 32): two
    // launches of up to 16 rows each
    {
        const uint32_t m0 = 16u, m1 = M - 16u;
        const size_t ypitch = (size_t)(pl.n_total ? pl.n_total : N) * ((flags & MIORI_OUT_BF16) ? 2u : 4u);
        int rc = try_launch<BITS>(q, s, b, x, y, N, K, m0, group, flags, stream, pl);
        if (rc != 0) return rc;
        const void* x1 = pl.gamma ? static_cast<const void*>(static_cast<const float*>(x) + (size_t)m0 * K)
                                  : static_cast<const void*>(static_cast<const uint16_t*>(x) + (size_t)m0 * K);
        return try_launch<BITS>(q, s, b, x1, static_cast<uint8_t*>(y) + m0 * ypitch, N, K, m1, group, flags,
                                stream, pl);
    }
#undef MIORI_UMMA_TRY
}

}  // namespace gemvumma
}  // namespace miori_b200
