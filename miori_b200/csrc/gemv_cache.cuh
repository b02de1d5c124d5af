// Narrow batches against the bf16 weight cache: y[M][N] = x[M][K] (bf16) x cache[N][K]^T, M <= 32.
//
// What the reference's wide-batch path multiplies (its bf16 cache, shaders/gemm_mpp.metal:36-73,
// reached through BatchEngine::linear, src/batch.cpp:223-230) for the batch sizes of a decode
// step.  The tcgen05 GEMM serves these shapes badly: a 128-row tile of A is three quarters empty,
// a projection of 2048 outputs has 16 tiles for 148 SMs, so K has to be split and summed by a
// second kernel, and the launch pays TMEM allocation and a long pipeline fill.  Here the cache is
// streamed once in 16-row tiles, exactly like the packed weights of the decode GEMV -- there are
// 128 tiles where the GEMM had 16 -- with no unpack at all: 16 bytes of a cache row ARE an A
// fragment of mma.sync.m16n8k16 (under the fixed k permutation "slot 2t, 2t+1, 2t+8, 2t+9 of lane
// t = elements 8t .. 8t+3"), and the same 16 bytes of an activation row are the matching B
// fragment, so x needs no permutation either.
//
//   * one CTA per SM, 16 compute warps + 1 producer warp; a stage is 16 rows x 512 k of the cache,
//     one 2-D TMA copy (the tensor is described as 64-bit words so that the box can be 1088 bytes
//     wide: the 64 extra bytes per row make the row pitch 64 (mod 128), which spreads the eight
//     lanes of a quarter-warp over all bank groups without a swizzle);
//   * the ring is filled before griddepcontrol.wait (the cache is immutable);
//   * the activation rows come in NT sets of eight (the MMA's columns).  Warp w owns set w % NT
//     and the k range [32 NT (w / NT), + 32 NT) of every stage, for every tile of the CTA.  Its B
//     fragments are therefore the same for all tiles and live in REGISTERS: after the wait every
//     lane loads its 16 bytes of x per (k-slab, 32-k step) straight from global memory, once -- at
//     most 16 of them, 64 registers -- and x never touches shared memory, which is left to the
//     ring (eight stages, 139 KB in flight per SM);
//   * per stage and 32-k step a warp issues two 16-byte loads (the tile's rows g and g + 8) and two
//     MMAs; after the last slab of a tile the 16 / NT warps that share a set add their 16 x 8
//     partial sums through shared memory in a fixed order, so a row's value depends neither on M
//     nor on the grid.  (Splitting only k over the warps, every warp carrying all sets, needed a
//     16 x 8 NT partial per warp: at 32 rows the exchange cost 6 us of a 23 us launch.)
// Every wait is bounded.
#pragma once
#include "common.cuh"
#include "gemv_mma.cuh"
#include "gemv_tma.cuh"
#include "tma_host.cuh"

namespace miori_b200 {
namespace gemvcache {

constexpr int WARPS = 16;
constexpr int THREADS = (WARPS + 1) * 32;
constexpr int KS = 512;                       // k per stage
constexpr int PITCH = KS * 2 + 64;            // bytes between rows of a stage
constexpr int STAGE_BYTES = 16 * PITCH;       // 17408
constexpr int BOX_WORDS = PITCH / 8;          // box width in 64-bit words
constexpr int MAX_STAGES = 8;
constexpr int MAX_FRAGS = 16;                 // (k-slabs) x (sets of 8 activation rows) held in registers

template <int NT>
struct Cfg {
    static constexpr int MP = 8 * NT;                     // activation rows covered (zero rows past M)
    static constexpr int KP = WARPS / NT;                 // warps that share a set: k parts of a stage
    static constexpr int RED_STRIDE = 16 * 9;             // floats of one warp's 16 x 8 partial, padded rows
    static constexpr int RED_BYTES = WARPS * RED_STRIDE * 4;
};

template <int NT>
size_t smem_bytes(uint32_t nstage) {
    return 128 + (size_t)nstage * STAGE_BYTES + Cfg<NT>::RED_BYTES;
}

constexpr int X_AHEAD = 3;  // streamed x: k-slabs between the load of a fragment and its use

// SLABS = ceil(K / 512) is a template parameter so that the x fragments index registers.
// STREAM: the fragments are loaded per tile, X_AHEAD slabs ahead, instead of once per CTA.
template <int NT, int SLABS, bool OUT_BF16, bool STREAM = false>
__global__ void __launch_bounds__(THREADS, 1)
gemv_cache_kernel(const __grid_constant__ CUtensorMap tmap_w, const uint16_t* __restrict__ x,
                  void* __restrict__ y, uint32_t N, uint32_t K, uint32_t M, uint32_t nstage) {
    constexpr uint32_t slabs = SLABS;
    constexpr int XF = STREAM ? X_AHEAD + 1 : SLABS;  // fragment sets held per lane
    static_assert(NT * XF <= (STREAM ? 20 : MAX_FRAGS), "x fragments held in registers");
    // a slab's slot is s % XF in every tile, so the ring must divide the slabs of a tile
    static_assert(!STREAM || (SLABS > X_AHEAD && SLABS % XF == 0), "streaming is for long rows");
    using C = Cfg<NT>;
    using namespace gemvmma;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bars[MAX_STAGES];
    __shared__ __align__(8) uint64_t empty_bars[MAX_STAGES];
    __shared__ volatile uint32_t abort_flag;

    const uint32_t base = (smem_addr(smem_raw) + 127u) & ~127u;
    const uint32_t ring = base;
    const uint32_t red_a = ring + nstage * (uint32_t)STAGE_BYTES;
    float* red = reinterpret_cast<float*>(smem_raw + (red_a - smem_addr(smem_raw)));

    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t tiles = (N + 15u) / 16u;
    const uint32_t my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1u) / gridDim.x : 0u;
    const uint32_t total = my_tiles * slabs;

    pdl_launch_dependents();

    const bool producer = threadIdx.x == WARPS * 32;
    uint32_t issued = 0, p_tile = 0, p_slab = 0, p_stage = 0, p_round = 0;
    // issue every slab whose stage is free, without blocking
    auto try_refill = [&]() {
        while (issued < total) {
            if (p_round != 0u) {
                if (!mbar_try(smem_addr(&empty_bars[p_stage]), (p_round - 1u) & 1u)) break;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            const uint32_t bar = smem_addr(&full_bars[p_stage]);
            mbar_expect_tx(bar, (uint32_t)STAGE_BYTES);
            tma_load_2d(ring + p_stage * (uint32_t)STAGE_BYTES, &tmap_w, (int)(p_slab * (KS / 4)),
                        (int)((blockIdx.x + p_tile * gridDim.x) * 16u), bar);
            ++issued;
            if (++p_slab == slabs) { p_slab = 0; ++p_tile; }
            if (++p_stage == nstage) { p_stage = 0; ++p_round; }
        }
    };
    if (producer) {
        abort_flag = 0u;
        for (uint32_t i = 0; i < nstage; ++i) {
            mbar_init(smem_addr(&full_bars[i]), 1);
            mbar_init(smem_addr(&empty_bars[i]), WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        try_refill();  // the cache is immutable: its first slabs travel before the dependency wait
    }
    pdl_wait_prior();  // x (and y) belong to the predecessor until here
    // this lane's B fragments: 16 bytes of activation row 8 (warp % NT) + g at
    // k = 512 s + 32 (NT (warp / NT) + i) + 8 t for the NT steps i of the warp's k part
    const uint32_t set = warp % (uint32_t)NT, kpart = warp / (uint32_t)NT;
    uint4 xf[XF][NT];
    // the fragments of k-slab s into slot s % XF
    auto load_x = [&](int s) {
        const uint32_t g = lane >> 2, t = lane & 3u, m = 8u * set + g;
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const uint32_t k = (uint32_t)s * KS + (kpart * NT + i) * 32u + t * 8u;
            xf[s % XF][i] = make_uint4(0u, 0u, 0u, 0u);
            if (warp < WARPS && m < M && k < K)  // K is a multiple of 8: whole pieces
                xf[s % XF][i] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)m * K + k));
        }
    };
#pragma unroll
    for (int s = 0; s < (STREAM ? X_AHEAD : SLABS); ++s) load_x(s);
    __syncthreads();  // barriers initialised before anyone waits on them

    if (producer) {
        const long long t0 = clock64();
        while (issued < total && !abort_flag) {
            try_refill();
            if (clock64() - t0 > 4 * WAIT_LIMIT_CYCLES) {
                abort_flag = 1u;
                device_error(0x6F14u, blockIdx.x, issued);
            }
        }
    }
    if (warp < WARPS) {
        const uint32_t g = lane >> 2, t = lane & 3u;
        const uint32_t a_lane = g * (uint32_t)PITCH + kpart * (NT * 64u) + t * 16u;  // row g, first step of the k part
        bool ok = true;
        uint32_t stage = 0, parity = 0;
        for (uint32_t ti = 0; ti < my_tiles; ++ti) {
            // two accumulation chains (even and odd steps), so that consecutive MMAs do not wait for
            // one another; they meet in a fixed order before the exchange
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, acc2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int s = 0; s < SLABS; ++s) {
                if constexpr (STREAM) {  // the fragments X_AHEAD slabs on (of the next tile past the last slab)
                    if (s + X_AHEAD < SLABS) load_x(s + X_AHEAD);
                    else if (ti + 1u < my_tiles) load_x(s + X_AHEAD - SLABS);
                }
                if (ok) {
                    ok = mbar_wait(smem_addr(&full_bars[stage]), parity, &abort_flag, 0x20);
                    ok = __all_sync(0xFFFFFFFFu, ok);
                }
                if (ok) {
                    const uint32_t st = ring + stage * (uint32_t)STAGE_BYTES + a_lane;
#pragma unroll
                    for (int i = 0; i < NT; ++i) {
                        const uint4 q0 = gemvtma::lds128(st + (uint32_t)i * 64u);
                        const uint4 q1 = gemvtma::lds128(st + (uint32_t)i * 64u + 8u * (uint32_t)PITCH);
                        mma_bf16(acc, q0.x, q1.x, q0.y, q1.y, xf[s % XF][i].x, xf[s % XF][i].y);
                        mma_bf16(acc2, q0.z, q1.z, q0.w, q1.w, xf[s % XF][i].z, xf[s % XF][i].w);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_addr(&empty_bars[stage]));  // stage consumed
                }
                if (++stage == nstage) { stage = 0; parity ^= 1u; }
            }
            // the KP warps of a set meet: partial [kpart][set] is 16 rows x 8 columns; thread (m, r) adds
            // the KP partials of its output in k order
            float* mine = red + (size_t)(kpart * NT + set) * C::RED_STRIDE;
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] += acc2[e];
            mine[g * 9 + 2 * t] = acc[0];
            mine[g * 9 + 2 * t + 1] = acc[1];
            mine[(g + 8) * 9 + 2 * t] = acc[2];
            mine[(g + 8) * 9 + 2 * t + 1] = acc[3];
            asm volatile("bar.sync 1, 512;" ::: "memory");
            const uint32_t row0 = (blockIdx.x + ti * gridDim.x) * 16u;
            for (uint32_t o = threadIdx.x; o < 16u * C::MP; o += WARPS * 32) {
                const uint32_t m = o >> 4, r = o & 15u;
                const float* src = red + (size_t)(m >> 3) * C::RED_STRIDE + r * 9u + (m & 7u);
                float v = src[0];
#pragma unroll
                for (int p = 1; p < C::KP; ++p) v += src[(size_t)p * NT * C::RED_STRIDE];
                if (m < M && row0 + r < N && ok) {
                    if (OUT_BF16) static_cast<uint16_t*>(y)[(size_t)m * N + row0 + r] = (uint16_t)float_to_bf16_bits(v);
                    else static_cast<float*>(y)[(size_t)m * N + row0 + r] = v;
                }
            }
            asm volatile("bar.sync 1, 512;" ::: "memory");  // the partial area is reused by the next tile
        }
    }
    if (abort_flag) {  // let copies still in flight land before the CTA's memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
    }
}

// Try the narrow-batch kernel; returns 1 if the problem is outside its range (nothing launched).
inline int try_launch(const void* x, const void* cache, void* y, uint32_t M, uint32_t N, uint32_t K,
                      uint32_t flags, cudaStream_t stream_) {
    if (M == 0 || M > 32 || K % 8 != 0) return 1;
    const uint32_t slabs = (K + KS - 1) / KS;
    const uint32_t nt = M <= 8 ? 1 : M <= 16 ? 2 : 4;
    // instantiated slab counts; a slab past the end of K is zero-filled by TMA and multiplies zeros
    const uint32_t slabs_t = slabs <= 1 ? 1 : slabs <= 2 ? 2 : slabs <= 4 ? 4 : slabs <= 8 ? 8 : 16;
    if (slabs > 16) return 1;
    const bool stream = slabs_t * nt > (uint32_t)MAX_FRAGS;  // a row's fragments do not fit the registers
    const uint32_t tiles = (N + 15u) / 16u;
    const uint32_t grid = std::min<uint32_t>(tiles, (uint32_t)sm_count());
    const uint32_t nstage =
        std::min<uint32_t>(MAX_STAGES, std::max<uint32_t>(2u, ((tiles + grid - 1) / grid) * slabs_t));
    // more than half of an SM's shared memory, so that no second CTA of a neighbouring launch joins
    // this one (see the placement note in gemv_tma.cuh: plan_stages)
    const size_t need = nt == 1 ? smem_bytes<1>(nstage) : nt == 2 ? smem_bytes<2>(nstage) : smem_bytes<4>(nstage);
    const size_t smem = std::max<size_t>(need, 120 * 1024);
    CUtensorMap tw;
    // rows past the last whole slab are zero-filled by TMA, and so are the x fragments there
    int rc = make_tmap_2d(&tw, cache, CU_TENSOR_MAP_DATA_TYPE_UINT64, 8, K / 4, N, BOX_WORDS, 16,
                          CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    const bool pdl = (flags & MIORI_LAUNCH_PDL) != 0, bf16 = (flags & MIORI_OUT_BF16) != 0;
    cudaError_t e = cudaSuccess;
#define MIORI_CACHE_LAUNCH(NTV, SL, OB)                                                           \
    do {                                                                                          \
        auto kern = gemv_cache_kernel<NTV, SL, OB>;                                               \
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        if (e == cudaSuccess)                                                                     \
            e = launch(kern, dim3(grid), dim3(THREADS), smem, stream_, pdl, tw,                   \
                       static_cast<const uint16_t*>(x), y, N, K, M, nstage);                      \
    } while (0)
#define MIORI_CACHE_SL(NTV, SL) do { if (bf16) MIORI_CACHE_LAUNCH(NTV, SL, true); else MIORI_CACHE_LAUNCH(NTV, SL, false); } while (0)
#define MIORI_CACHE_STREAM(NTV, SL)                                                               \
    do {                                                                                          \
        auto kern = bf16 ? gemv_cache_kernel<NTV, SL, true, true> : gemv_cache_kernel<NTV, SL, false, true>; \
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        if (e == cudaSuccess)                                                                     \
            e = launch(kern, dim3(grid), dim3(THREADS), smem, stream_, pdl, tw,                   \
                       static_cast<const uint16_t*>(x), y, N, K, M, nstage);                      \
    } while (0)
    if (stream) {
        if (nt == 2) MIORI_CACHE_STREAM(2, 16);
        else if (slabs_t == 8) MIORI_CACHE_STREAM(4, 8);
        else MIORI_CACHE_STREAM(4, 16);
    } else if (nt == 1) {
        if (slabs_t == 1) MIORI_CACHE_SL(1, 1); else if (slabs_t == 2) MIORI_CACHE_SL(1, 2);
        else if (slabs_t == 4) MIORI_CACHE_SL(1, 4); else if (slabs_t == 8) MIORI_CACHE_SL(1, 8);
        else MIORI_CACHE_SL(1, 16);
    } else if (nt == 2) {
        if (slabs_t == 1) MIORI_CACHE_SL(2, 1); else if (slabs_t == 2) MIORI_CACHE_SL(2, 2);
        else if (slabs_t == 4) MIORI_CACHE_SL(2, 4); else MIORI_CACHE_SL(2, 8);
    } else {
        if (slabs_t == 1) MIORI_CACHE_SL(4, 1); else if (slabs_t == 2) MIORI_CACHE_SL(4, 2);
        else MIORI_CACHE_SL(4, 4);
    }
#undef MIORI_CACHE_STREAM
#undef MIORI_CACHE_SL
#undef MIORI_CACHE_LAUNCH
    if (e != cudaSuccess) return cuda_fail(e, "gemv_cache launch");
    return MIORI_OK;
}

}  // namespace gemvcache
}  // namespace miori_b200
