// Device side of the N-sharded GEMV's fused all-gather.  Every rank (one process per GPU) owns
// an "arena" of device memory that all other ranks map through CUDA IPC:
//
//   [ control block 256 B | user area (outputs, same offsets on every rank) | inbox 0 | inbox 1 ]
//
// A kernel writes the rows it computed into its own copy of y and, for every peer, into that
// peer's inbox as 8-byte packets {value bits, launch number} -- one plain store over NVLink per
// element, which arrives whole, so the packet is its own "ready" flag and no fence, release or
// counter crosses the link (a system-scope fence costs 1.5-3.5 us here; the first version of this
// protocol spent one per CTA).  Before it exits, every CTA of the receiving kernel takes a slice of
// the output, waits (bounded) until the packets of the rows its peers own carry this launch's
// number, and copies the values into y.  When the kernel completes on a rank its whole y is
// there, so anything that follows on the stream may read it.
//
// Launch numbers: every rank runs the same sequence of these kernels, so the per-rank count of
// completed launches (kept in the control block, bumped by the last CTA with local atomics only)
// agrees across ranks without the host, and CUDA graphs replay it.  Inboxes alternate with the
// launch number's parity: a rank can be at most one launch ahead of a peer (its launch e+1
// completes only after the peer's rows of e+1 arrived, which the peer sends after finishing e),
// so a packet of launch e+1 never lands on a slot a peer still reads for launch e.
// All waits are bounded (about a second unless the host sets another limit): on expiry the kernel records a device error, marks the control
// block and stops waiting, so a missing peer costs time but never hangs the GPU.  Only plain
// loads and stores touch peer memory: no multicast, no TMA.
#pragma once
#include "common.cuh"

namespace miori_b200 {

constexpr int MAX_PEERS = 8;
constexpr size_t PEER_CTL_BYTES = 256;      // control block at the start of every arena
constexpr size_t PEER_TABLE_OFFSET = 128;   // MAX_PEERS arena pointers inside the control block
constexpr size_t PEER_INBOX_FACTOR = 4;     // one inbox = 4 x user bytes: 8-byte packets for 2-byte elements
enum : uint32_t { CTL_COUNT = 16, CTL_EPOCH = 17, CTL_ERR = 18, CTL_LIMIT = 20 /* 64-bit: wait limit in cycles */ };

struct PeerArgs {          // by value in kernel parameters
    uint8_t* local;        // this rank's arena; its control block holds, at PEER_TABLE_OFFSET,
                           // every rank's arena as mapped in this process (entry [rank] = local)
    uint32_t world, rank;  // world <= 1: no peers, kernels behave as single-GPU kernels
    size_t user_bytes;     // size of the user area (the inboxes follow it)
};

#ifdef __CUDACC__
__device__ __forceinline__ uint8_t* peer_arena(const PeerArgs& pa, uint32_t p) {
    return reinterpret_cast<uint8_t* const*>(pa.local + PEER_TABLE_OFFSET)[p];
}
__device__ __forceinline__ uint32_t* peer_ctl(const PeerArgs& pa) {
    return reinterpret_cast<uint32_t*>(pa.local);
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// The launch number this kernel runs as.  Stable for the kernel's whole life: only the last CTA
// advances it, after every CTA has finished.  Call after the dependency wait.
__device__ __forceinline__ uint32_t peer_epoch(const PeerArgs& pa) {
    return ld_relaxed_sys(peer_ctl(pa) + CTL_EPOCH) + 1u;
}
// Packet slot of output element `elem` (index into the user area in units of the output's element
// size, i.e. y_off / esize + m * n_total + row) in the inbox of launch e inside `arena`.
__device__ __forceinline__ uint2* peer_slot(const PeerArgs& pa, uint8_t* arena, uint32_t e, size_t elem) {
    uint8_t* inbox = arena + PEER_CTL_BYTES + pa.user_bytes * (1u + (e & 1u) * PEER_INBOX_FACTOR);
    return reinterpret_cast<uint2*>(inbox) + elem;
}
// One element to one peer: value bits (low word) and launch number (high word) as ONE 64-bit
// store.  A scalar 8-byte access is single-copy atomic in the PTX memory model, so a reader sees
// either the whole old packet or the whole new one; a vector store of two words would not
// promise that.
__device__ __forceinline__ void peer_send(uint2* slot, uint32_t bits, uint32_t e) {
    const uint64_t pkt = (uint64_t)bits | ((uint64_t)e << 32);
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(slot), "l"(pkt) : "memory");
}
__device__ __forceinline__ uint64_t peer_load(const uint2* slot) {
    uint64_t pkt;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(pkt) : "l"(slot) : "memory");
    return pkt;
}
// Bounded wait for the packet of launch e in a local slot; false if it never came.
__device__ __forceinline__ bool peer_recv(const PeerArgs& pa, const uint2* slot, uint32_t e, uint32_t& bits) {
    uint64_t pkt = peer_load(slot);
    bits = (uint32_t)pkt;
    if ((uint32_t)(pkt >> 32) == e) return true;
    uint32_t* ctl = peer_ctl(pa);
    // the limit is a field of the control block (miori_peers_set_wait_us; about a second by default)
    const long long limit = *reinterpret_cast<const volatile long long*>(ctl + CTL_LIMIT);
    const long long t0 = clock64();
    for (;;) {
        pkt = peer_load(slot);
        bits = (uint32_t)pkt;
        if ((uint32_t)(pkt >> 32) == e) return true;
        if (ld_relaxed_sys(ctl + CTL_ERR) != 0u) return false;  // someone already gave up
        if (clock64() - t0 > limit) {
            st_relaxed_sys(ctl + CTL_ERR, 0x7E30u);
            device_error(0x7E30u, blockIdx.x, e);
            return false;
        }
        __nanosleep(32);
    }
}
// Every CTA, all threads, after the CTA's own rows are written (a CTA-wide barrier precedes the
// call): copy the peers' rows of y[M][n_total] out of the local inbox.  The grid's threads share
// the M * n_total elements; rows [row0, row0 + n_local) are this rank's own and are skipped.
template <bool OUT_BF16>
__device__ __forceinline__ void peer_collect(const PeerArgs& pa, uint32_t e, size_t y_off, uint32_t M,
                                             uint32_t n_total, uint32_t row0, uint32_t n_local) {
    const size_t total = (size_t)M * n_total, base = y_off / (OUT_BF16 ? 2u : 4u);
    uint8_t* y = pa.local + PEER_CTL_BYTES + y_off;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t row = (uint32_t)(i % n_total);
        if (row - row0 < n_local) continue;
        uint32_t bits;
        if (!peer_recv(pa, peer_slot(pa, pa.local, e, base + i), e, bits)) return;
        if (OUT_BF16) reinterpret_cast<uint16_t*>(y)[i] = (uint16_t)bits;
        else reinterpret_cast<uint32_t*>(y)[i] = bits;
    }
}
// One thread per CTA, after the CTA has collected (a CTA-wide barrier precedes the call): the last
// CTA of the grid advances the launch number.  Local atomics only.
__device__ __forceinline__ void peer_finish(const PeerArgs& pa, uint32_t e) {
    uint32_t* ctl = peer_ctl(pa);
    __threadfence();
    if (atomicAdd(ctl + CTL_COUNT, 1u) != gridDim.x - 1u) return;
    ctl[CTL_COUNT] = 0u;
    st_relaxed_sys(ctl + CTL_EPOCH, e);
}
// Sharded arg-max: a candidate (value, index) per rank; larger value first, then the lower index
// (the first maximum of the unsharded vector, as the host loop of src/engine.cpp:740-747).
struct PeerBest {
    float v;
    uint32_t i;
};
__device__ __forceinline__ PeerBest peer_better(PeerBest a, PeerBest b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
// One thread of the whole grid: offer this rank's candidate to every peer, take theirs, reduce in
// rank order.  `pairs` is this rank's [world][value, index] + winner [value, index] area in its
// arena, `base` the same area's position in 4-byte units of the user area (where the peers'
// packets land).  Returns the winner (this rank's candidate when there are no peers).
__device__ __forceinline__ PeerBest peer_argmax_exchange(const PeerArgs& pa, uint32_t* pairs, size_t base,
                                                         PeerBest mine) {
    const uint32_t world = pa.world > 1u ? pa.world : 1u, rank = pa.world > 1u ? pa.rank : 0u;
    pairs[2u * rank] = __float_as_uint(mine.v);
    pairs[2u * rank + 1u] = mine.i;
    PeerBest all = mine;
    if (pa.world > 1u) {
        const uint32_t e = peer_epoch(pa);
        for (uint32_t p = 0; p < world; ++p) {
            if (p == rank) continue;
            uint8_t* arena = peer_arena(pa, p);
            peer_send(peer_slot(pa, arena, e, base + 2u * rank), __float_as_uint(mine.v), e);
            peer_send(peer_slot(pa, arena, e, base + 2u * rank + 1u), mine.i, e);
        }
        bool ok = true;
        all = PeerBest{-INFINITY, 0xFFFFFFFFu};
        for (uint32_t p = 0; p < world && ok; ++p) {
            PeerBest b = mine;
            if (p != rank) {
                uint32_t vb = 0, ib = 0;
                ok = peer_recv(pa, peer_slot(pa, pa.local, e, base + 2u * p), e, vb) &&
                     peer_recv(pa, peer_slot(pa, pa.local, e, base + 2u * p + 1u), e, ib);
                b = PeerBest{__uint_as_float(vb), ib};
                pairs[2u * p] = vb;
                pairs[2u * p + 1u] = ib;
            }
            if (ok) all = peer_better(all, b);
        }
        __threadfence();
        st_relaxed_sys(peer_ctl(pa) + CTL_EPOCH, e);  // this thread does all the peer work of the launch
    }
    pairs[2u * world] = __float_as_uint(all.v);
    pairs[2u * world + 1u] = all.i;
    return all;
}
// Order-preserving 64-bit key of a candidate: the larger key is the larger value, and among equal
// values the lower index; 0 stands for "none" (NaN never becomes a key).
__device__ __forceinline__ unsigned long long peer_best_key(uint32_t value_bits, uint32_t index) {
    const uint32_t ordered = (value_bits & 0x80000000u) ? ~value_bits : (value_bits | 0x80000000u);
    return ((unsigned long long)ordered << 32) | (unsigned long long)(0xFFFFFFFFu - index);
}
__device__ __forceinline__ PeerBest peer_best_from_key(unsigned long long key) {
    if (key == 0ull) return PeerBest{-INFINITY, 0xFFFFFFFFu};
    const uint32_t ordered = (uint32_t)(key >> 32);
    const uint32_t bits = (ordered & 0x80000000u) ? (ordered ^ 0x80000000u) : ~ordered;
    return PeerBest{__uint_as_float(bits), 0xFFFFFFFFu - (uint32_t)key};
}
// The same for a kernel in which a single thread of the whole grid does the peer work: that
// thread advances the launch number itself.
__device__ __forceinline__ void peer_finish_single(const PeerArgs& pa, uint32_t e) {
    __threadfence();
    st_relaxed_sys(peer_ctl(pa) + CTL_EPOCH, e);
}
#endif

}  // namespace miori_b200
