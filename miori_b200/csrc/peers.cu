// Host side of the multi-GPU path: per-rank arenas shared through CUDA IPC, the N-sharded GEMV
// entries whose epilogue is the all-gather (peers.cuh), and a stand-alone all-gather kernel for
// outputs produced by another kernel (the cache GEMM).
#include "common.cuh"
#include "gemv_tma.cuh"
#include "peers.cuh"

#include <cstring>

struct miori_peers {
    int rank, world;
    size_t user_bytes;
    uint8_t* mapped[miori_b200::MAX_PEERS];  // [rank] is the local allocation
    bool connected;
};

using namespace miori_b200;

namespace miori_b200 {
namespace peers {

// Send this rank's block of an output -- src[M][n_local] elements, row pitch src_pitch bytes --
// to columns [row0, row0 + n_local) of y[M][n_total] on every rank (a plain copy into its own
// arena, packets into the peers' inboxes), then collect the peers' blocks: the protocol of the
// fused GEMV (peers.cuh) as a kernel of its own.
template <bool BF16>
__global__ void __launch_bounds__(256)
allgather_kernel(const PeerArgs pa, const uint8_t* __restrict__ src, uint32_t src_pitch, size_t y_off,
                 uint32_t M, uint32_t n_total, uint32_t row0, uint32_t n_local) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const uint32_t e = peer_epoch(pa);
    constexpr uint32_t ES = BF16 ? 2u : 4u;
    uint8_t* y = pa.local + PEER_CTL_BYTES + y_off;
    const size_t base = y_off / ES;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)M * n_local;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t m = i / n_local, c = i - m * n_local;
        const size_t idx = m * n_total + row0 + c;
        uint32_t bits;
        if (BF16) {
            bits = *reinterpret_cast<const uint16_t*>(src + m * src_pitch + c * 2u);
            reinterpret_cast<uint16_t*>(y)[idx] = (uint16_t)bits;
        } else {
            bits = *reinterpret_cast<const uint32_t*>(src + m * src_pitch + c * 4u);
            reinterpret_cast<uint32_t*>(y)[idx] = bits;
        }
        for (uint32_t p = 0; p < pa.world; ++p)
            if (p != pa.rank) peer_send(peer_slot(pa, peer_arena(pa, p), e, base + idx), bits, e);
    }
    __syncthreads();
    peer_collect<BF16>(pa, e, y_off, M, n_total, row0, n_local);
    __syncthreads();
    if (threadIdx.x == 0) peer_finish(pa, e);
}

// Greedy sampling over an N-sharded head without gathering the logits: every rank finds the best
// of its own slice, the ranks exchange (value, index) pairs -- two 8-byte packets per rank instead
// of the whole vector -- and every rank reduces the pairs the same way (ties: lowest index, as the
// host loop of src/engine.cpp:740-747).  One cluster of up to 8 CTAs finds the local best; thread
// 0 of its first CTA does the exchange.  The pairs land in the arena at y_off as
// [rank][value, index] followed by the winner [value, index].
template <bool BF16>
__global__ void __launch_bounds__(1024)
argmax_allreduce_kernel(const PeerArgs pa, const void* __restrict__ v, uint32_t n_local, uint32_t index0,
                        size_t y_off) {
    __shared__ neighbors::Best warp_best[32];
    __shared__ __align__(8) neighbors::Best cta_best[neighbors::ARGMAX_CLUSTER];
    pdl_launch_dependents();
    pdl_wait_prior();
    const neighbors::Best mine = neighbors::cluster_argmax<BF16>(v, n_local, index0, warp_best, cta_best);
    if (neighbors::cluster_ctarank() == 0u && threadIdx.x == 0) {
        uint32_t* pairs = reinterpret_cast<uint32_t*>(pa.local + PEER_CTL_BYTES + y_off);
        peer_argmax_exchange(pa, pairs, y_off / 4u, PeerBest{mine.v, mine.i});
    }
}

// The limit of the kernels' waits for a peer, kept in the control block in SM clock cycles.
static int write_wait_limit(const miori_peers* g, double microseconds) {
    int dev = 0, khz = 0;
    MIORI_CUDA(cudaGetDevice(&dev));
    MIORI_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));
    if (khz <= 0) khz = 1965000;
    long long cycles = (long long)(microseconds * 1e-3 * (double)khz);
    if (cycles < 1000) cycles = 1000;
    MIORI_CUDA(cudaMemcpy(g->mapped[g->rank] + CTL_LIMIT * 4, &cycles, sizeof(cycles), cudaMemcpyHostToDevice));
    return MIORI_OK;
}

// The table of mapped arenas the kernels read, in the local control block.
static int write_table(const miori_peers* g) {
    uint8_t* table[MAX_PEERS] = {};
    for (int r = 0; r < g->world; ++r) table[r] = g->mapped[r];
    MIORI_CUDA(cudaMemcpy(g->mapped[g->rank] + PEER_TABLE_OFFSET, table, sizeof(table),
                          cudaMemcpyHostToDevice));
    return MIORI_OK;
}

static int check_peers(const char* op, const miori_peers* g) {
    if (!g) return fail(MIORI_E_INVALID, "%s: null peer group", op);
    if (g->world > 1 && !g->connected)
        return fail(MIORI_E_STATE, "%s: miori_peers_connect has not been called", op);
    return MIORI_OK;
}

static PeerArgs peer_args(const miori_peers* g) {
    PeerArgs pa = {};
    pa.local = g->mapped[g->rank];
    pa.world = (uint32_t)g->world;
    pa.rank = (uint32_t)g->rank;
    pa.user_bytes = g->user_bytes;
    return pa;
}

template <int BITS>
static int gemv_allgather(const char* op, miori_peers* g, const void* q, const void* s, const void* b,
                          const void* x, size_t y_offset, uint32_t n_local, uint32_t row0,
                          uint32_t n_total, uint32_t K, uint32_t M, uint32_t group, uint32_t flags,
                          void* stream, const size_t* best_offset = nullptr) {
    int rc = check_peers(op, g);
    if (rc) return rc;
    if (!q || !s || !b || !x) return fail(MIORI_E_INVALID, "%s: null pointer", op);
    if (group != 32 && group != 64) return fail(MIORI_E_INVALID, "%s: group must be 32 or 64", op);
    if (M == 0 || M > 32) return fail(MIORI_E_INVALID, "%s: M=%u outside 1..32", op, M);
    if (n_local == 0 || K == 0 || K % group != 0 || (size_t)row0 + n_local > n_total)
        return fail(MIORI_E_INVALID, "%s: bad shape n_local=%u row0=%u n_total=%u K=%u", op, n_local,
                    row0, n_total, K);
    if (!aligned16(q) || !aligned16(s) || !aligned16(b) || !aligned16(x) || y_offset % 16 != 0)
        return fail(MIORI_E_INVALID, "%s: q, s, b, x and the y offset must be 16-byte aligned", op);
    const size_t esize = (flags & MIORI_OUT_BF16) ? 2 : 4;
    if (y_offset + (size_t)M * n_total * esize > g->user_bytes)
        return fail(MIORI_E_INVALID, "%s: y (%zu bytes at offset %zu) does not fit the %zu-byte arena",
                    op, (size_t)M * n_total * esize, y_offset, g->user_bytes);
    gemvtma::Shard sh;
    sh.pa = peer_args(g);
    sh.n_total = n_total;
    sh.row0 = row0;
    sh.y_off = y_offset;
    void* y_local = g->mapped[g->rank] + PEER_CTL_BYTES + y_offset;
    if (g->world <= 1) {  // no peers: an ordinary GEMV into the local arena
        sh.pa.world = 0;
        if (row0 != 0 || n_local != n_total)
            return fail(MIORI_E_INVALID, "%s: a single rank holds all rows", op);
    }
    if (best_offset) {  // arg-max epilogue: scratch {key, arrivals}, candidates, winner
        const size_t need = 16 + (size_t)(2 * g->world + 2) * 4;
        if (M != 1) return fail(MIORI_E_INVALID, "%s: one activation row", op);
        if (*best_offset % 16 != 0 || *best_offset + need > g->user_bytes)
            return fail(MIORI_E_INVALID, "%s: %zu bytes at offset %zu do not fit the arena", op, need, *best_offset);
        sh.best = reinterpret_cast<unsigned long long*>(g->mapped[g->rank] + PEER_CTL_BYTES + *best_offset);
    }
    rc = gemvtma::try_launch<BITS>(q, s, b, x, y_local, n_local, K, M, group, flags,
                                   (cudaStream_t)stream, sh);
    if (rc == 1)
        return fail(MIORI_E_INVALID,
                    "%s: shape n_local=%u K=%u M=%u group=%u is outside the fused kernel's range "
                    "(use miori_gemv%d into the arena followed by miori_allgather)",
                    op, n_local, K, M, group, BITS);
    return rc;
}

}  // namespace peers
}  // namespace miori_b200

MIORI_API int miori_peers_create(int rank, int world, size_t arena_bytes, miori_peers** out) {
    if (!out) return fail(MIORI_E_INVALID, "miori_peers_create: null out");
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world)
        return fail(MIORI_E_INVALID, "miori_peers_create: rank %d of world %d (1..%d ranks)", rank, world,
                    MAX_PEERS);
    if (arena_bytes == 0 || arena_bytes % 256 != 0)
        return fail(MIORI_E_INVALID, "miori_peers_create: arena size must be a positive multiple of 256");
    miori_peers* g = new (std::nothrow) miori_peers();
    if (!g) return fail(MIORI_E_NOMEM, "miori_peers_create: out of host memory");
    g->rank = rank;
    g->world = world;
    g->user_bytes = arena_bytes;
    g->connected = world == 1;
    void* p = nullptr;
    // control block, user area, and two inboxes of 8-byte packets (PEER_INBOX_FACTOR x user each)
    const size_t total = PEER_CTL_BYTES + arena_bytes * (1 + 2 * PEER_INBOX_FACTOR);
    cudaError_t e = cudaMalloc(&p, total);
    if (e == cudaSuccess) e = cudaMemset(p, 0, total);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        delete g;
        return e == cudaErrorMemoryAllocation ? fail(MIORI_E_NOMEM, "miori_peers_create: %s", cudaGetErrorString(e))
                                              : cuda_fail(e, "miori_peers_create");
    }
    g->mapped[rank] = static_cast<uint8_t*>(p);
    int rc = peers::write_table(g);
    if (rc == MIORI_OK) rc = peers::write_wait_limit(g, 1.0e6);
    if (rc) {
        cudaFree(p);
        delete g;
        return rc;
    }
    *out = g;
    return MIORI_OK;
}

MIORI_API int miori_peers_set_wait_us(miori_peers* g, uint32_t microseconds) {
    if (!g) return fail(MIORI_E_INVALID, "miori_peers_set_wait_us: null peer group");
    if (microseconds == 0 || microseconds > 10000000u)
        return fail(MIORI_E_INVALID, "miori_peers_set_wait_us: %u us outside 1 us .. 10 s", microseconds);
    return peers::write_wait_limit(g, (double)microseconds);
}

MIORI_API size_t miori_peers_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

MIORI_API int miori_peers_handle(miori_peers* g, void* handle_out) {
    if (!g || !handle_out) return fail(MIORI_E_INVALID, "miori_peers_handle: null argument");
    cudaIpcMemHandle_t h;
    MIORI_CUDA(cudaIpcGetMemHandle(&h, g->mapped[g->rank]));
    std::memcpy(handle_out, &h, sizeof(h));
    return MIORI_OK;
}

MIORI_API int miori_peers_connect(miori_peers* g, const void* handles) {
    if (!g || !handles) return fail(MIORI_E_INVALID, "miori_peers_connect: null argument");
    if (g->connected) return fail(MIORI_E_STATE, "miori_peers_connect: already connected");
    const uint8_t* hs = static_cast<const uint8_t*>(handles);
    for (int r = 0; r < g->world; ++r) {
        if (r == g->rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, hs + (size_t)r * sizeof(h), sizeof(h));
        void* p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int k = 0; k < r; ++k)
                if (k != g->rank && g->mapped[k]) {
                    cudaIpcCloseMemHandle(g->mapped[k]);
                    g->mapped[k] = nullptr;
                }
            return cuda_fail(e, "miori_peers_connect: cudaIpcOpenMemHandle");
        }
        g->mapped[r] = static_cast<uint8_t*>(p);
    }
    int rc = peers::write_table(g);
    if (rc) return rc;
    g->connected = true;
    return MIORI_OK;
}

MIORI_API void* miori_peers_arena(miori_peers* g) {
    return g ? g->mapped[g->rank] + PEER_CTL_BYTES : nullptr;
}

MIORI_API size_t miori_peers_arena_bytes(miori_peers* g) { return g ? g->user_bytes : 0; }

MIORI_API int miori_peers_status(miori_peers* g) {
    if (!g) return fail(MIORI_E_INVALID, "miori_peers_status: null peer group");
    uint32_t ctl[32];
    MIORI_CUDA(cudaMemcpy(ctl, g->mapped[g->rank], sizeof(ctl), cudaMemcpyDeviceToHost));
    if (ctl[CTL_ERR] != 0u)
        return fail(MIORI_E_DEVICE, "rank %d gave up waiting for a peer (code 0x%x) at launch %u", g->rank,
                    ctl[CTL_ERR], ctl[CTL_EPOCH] + 1u);
    return MIORI_OK;
}

MIORI_API int miori_peers_destroy(miori_peers* g) {
    if (!g) return MIORI_OK;
    cudaError_t first = cudaSuccess;
    for (int r = 0; r < g->world; ++r) {
        if (!g->mapped[r]) continue;
        const cudaError_t e = r == g->rank ? cudaFree(g->mapped[r]) : cudaIpcCloseMemHandle(g->mapped[r]);
        if (e != cudaSuccess && first == cudaSuccess) first = e;
    }
    delete g;
    if (first != cudaSuccess) return cuda_fail(first, "miori_peers_destroy");
    return MIORI_OK;
}

MIORI_API int miori_gemv4_allgather(miori_peers* g, const void* q, const void* s, const void* b,
                                    const void* x, size_t y_offset, uint32_t n_local, uint32_t row0,
                                    uint32_t n_total, uint32_t K, uint32_t M, uint32_t group,
                                    uint32_t flags, void* stream) {
    return peers::gemv_allgather<4>("miori_gemv4_allgather", g, q, s, b, x, y_offset, n_local, row0,
                                    n_total, K, M, group, flags, stream);
}

MIORI_API int miori_gemv8_allgather(miori_peers* g, const void* q, const void* s, const void* b,
                                    const void* x, size_t y_offset, uint32_t n_local, uint32_t row0,
                                    uint32_t n_total, uint32_t K, uint32_t M, uint32_t group,
                                    uint32_t flags, void* stream) {
    return peers::gemv_allgather<8>("miori_gemv8_allgather", g, q, s, b, x, y_offset, n_local, row0,
                                    n_total, K, M, group, flags, stream);
}

MIORI_API size_t miori_gemv_argmax_bytes(int world) {
    return world < 1 ? 0 : 16 + (size_t)(2 * world + 2) * 4;
}

MIORI_API int miori_gemv4_argmax(miori_peers* g, const void* q, const void* s, const void* b, const void* x,
                                 size_t y_offset, size_t best_offset, uint32_t n_local, uint32_t row0,
                                 uint32_t n_total, uint32_t K, uint32_t group, uint32_t flags, void* stream) {
    return peers::gemv_allgather<4>("miori_gemv4_argmax", g, q, s, b, x, y_offset, n_local, row0, n_total, K, 1,
                                    group, flags, stream, &best_offset);
}

MIORI_API int miori_gemv8_argmax(miori_peers* g, const void* q, const void* s, const void* b, const void* x,
                                 size_t y_offset, size_t best_offset, uint32_t n_local, uint32_t row0,
                                 uint32_t n_total, uint32_t K, uint32_t group, uint32_t flags, void* stream) {
    return peers::gemv_allgather<8>("miori_gemv8_argmax", g, q, s, b, x, y_offset, n_local, row0, n_total, K, 1,
                                    group, flags, stream, &best_offset);
}

MIORI_API int miori_allgather(miori_peers* g, const void* src, size_t y_offset, uint32_t M,
                              uint32_t n_local, uint32_t row0, uint32_t n_total, uint32_t elem_bytes,
                              uint32_t flags, void* stream) {
    int rc = peers::check_peers("miori_allgather", g);
    if (rc) return rc;
    if (!src || !aligned16(src)) return fail(MIORI_E_INVALID, "miori_allgather: src null or not 16-byte aligned");
    if (elem_bytes != 2 && elem_bytes != 4)
        return fail(MIORI_E_INVALID, "miori_allgather: element size must be 2 or 4 bytes");
    if (M == 0 || n_local == 0 || (size_t)row0 + n_local > n_total)
        return fail(MIORI_E_INVALID, "miori_allgather: bad shape M=%u n_local=%u row0=%u n_total=%u", M,
                    n_local, row0, n_total);
    const size_t row_bytes = (size_t)n_total * elem_bytes, off = (size_t)row0 * elem_bytes,
                 len = (size_t)n_local * elem_bytes;
    if (y_offset % 16 || row_bytes % 16 || off % 16 || len % 16)
        return fail(MIORI_E_INVALID, "miori_allgather: offsets and row blocks must be multiples of 16 bytes");
    if (y_offset + (size_t)M * row_bytes > g->user_bytes)
        return fail(MIORI_E_INVALID, "miori_allgather: y does not fit the arena");
    const size_t elems = (size_t)M * n_local;
    const unsigned blocks = (unsigned)std::min<size_t>((elems + 255) / 256, (size_t)sm_count());
    const bool pdl = (flags & MIORI_LAUNCH_PDL) != 0;
    cudaError_t e;
    if (elem_bytes == 2)
        e = launch(peers::allgather_kernel<true>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, pdl,
                   peers::peer_args(g), static_cast<const uint8_t*>(src), (uint32_t)len, y_offset, M,
                   n_total, row0, n_local);
    else
        e = launch(peers::allgather_kernel<false>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, pdl,
                   peers::peer_args(g), static_cast<const uint8_t*>(src), (uint32_t)len, y_offset, M,
                   n_total, row0, n_local);
    if (e != cudaSuccess) return cuda_fail(e, "miori_allgather launch");
    return MIORI_OK;
}

MIORI_API int miori_argmax_allreduce(miori_peers* g, const void* v, uint32_t n_local, uint32_t index0,
                                     size_t y_offset, uint32_t flags, void* stream) {
    int rc = peers::check_peers("miori_argmax_allreduce", g);
    if (rc) return rc;
    if (!v || n_local == 0) return fail(MIORI_E_INVALID, "miori_argmax_allreduce: empty input");
    const size_t need = (size_t)(2 * g->world + 2) * 4;
    if (y_offset % 16 != 0 || y_offset + need > g->user_bytes)
        return fail(MIORI_E_INVALID, "miori_argmax_allreduce: %zu bytes at offset %zu do not fit the arena", need, y_offset);
    PeerArgs pa = peers::peer_args(g);
    if (g->world <= 1) pa.world = 0;
    const bool pdl = (flags & MIORI_LAUNCH_PDL) != 0;
    cudaError_t e;
    if (flags & MIORI_OUT_BF16)
        e = neighbors::launch_cluster(peers::argmax_allreduce_kernel<true>, neighbors::argmax_ctas(n_local),
                                      neighbors::ARGMAX_THREADS, (cudaStream_t)stream, pdl, pa, v, n_local, index0,
                                      y_offset);
    else
        e = neighbors::launch_cluster(peers::argmax_allreduce_kernel<false>, neighbors::argmax_ctas(n_local),
                                      neighbors::ARGMAX_THREADS, (cudaStream_t)stream, pdl, pa, v, n_local, index0,
                                      y_offset);
    if (e != cudaSuccess) return cuda_fail(e, "miori_argmax_allreduce launch");
    return MIORI_OK;
}
