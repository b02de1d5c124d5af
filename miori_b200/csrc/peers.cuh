// Device side of the N-sharded GEMV's fused all-gather: every rank (one process per GPU) owns
// an "arena" of device memory that all other ranks map through CUDA IPC, with the output
// buffers at the same offsets on every rank.  A kernel writes its rows of y straight into every
// rank's copy with plain peer stores over NVLink; three small counters per rank pair, kept in a
// control block at the start of each arena, order those stores against the readers:
//
//   ready[from]  "rank `from` has reached launch e": everything it enqueued before (the readers
//                of the previous y) is complete, so its copy of y may be overwritten
//   done[from]   "rank `from` has finished writing its rows of launch e into this arena"
//   epoch        launches completed on this rank; every rank runs the same launch sequence, so
//                launch numbers agree without any host involvement (CUDA graphs replay them)
//
// A kernel (1) announces ready(e) to every peer once its stream predecessors are complete,
// (2) before its first remote store waits until every peer has announced ready(e), (3) after its
// last CTA has stored, announces done(e) to every peer and waits for every peer's done(e), so
// "kernel complete" on a rank means "its whole y is complete".  All waits are bounded: after
// about a second they record a device error, mark the control block and give up, so a missing
// peer costs time but never hangs the GPU.  Only plain loads and stores cross the link: no
// multicast, no TMA from or to peer memory.
#pragma once
#include "common.cuh"

namespace miori_b200 {

constexpr int MAX_PEERS = 8;
constexpr size_t PEER_CTL_BYTES = 256;  // control block at the start of every arena
enum : uint32_t { CTL_READY = 0, CTL_DONE = 8, CTL_COUNT = 16, CTL_EPOCH = 17, CTL_ERR = 18 };

constexpr size_t PEER_TABLE_OFFSET = 128;  // MAX_PEERS arena pointers inside the control block

struct PeerArgs {          // by value in kernel parameters
    uint8_t* local;        // this rank's arena; its control block holds, at PEER_TABLE_OFFSET,
                           // every rank's arena as mapped in this process (entry [rank] = local)
    uint32_t world, rank;  // world <= 1: no peers, kernels behave as single-GPU kernels
};

#ifdef __CUDACC__
__device__ __forceinline__ uint8_t* peer_arena(const PeerArgs& pa, uint32_t p) {
    return reinterpret_cast<uint8_t* const*>(pa.local + PEER_TABLE_OFFSET)[p];
}
__device__ __forceinline__ uint32_t* peer_ctl(const PeerArgs& pa, uint32_t p) {
    return reinterpret_cast<uint32_t*>(p == pa.rank ? pa.local : peer_arena(pa, p));
}
// Counters are written and polled with relaxed system-scope accesses; ordering comes from the
// one system-scope fence each CTA executes after its data stores (below) and from kernel
// boundaries.  On B200 over NVLink a system-scope fence or release costs 1.5-3.5 us whether or
// not stores are outstanding, so the protocol spends exactly one per CTA, all in parallel.
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Bounded wait until *p has reached `want` (counters only grow; compared modulo 2^32).
__device__ __forceinline__ bool peer_wait_ge(uint32_t* ctl_local, const uint32_t* p, uint32_t want,
                                             uint32_t code) {
    if ((int32_t)(ld_relaxed_sys(p) - want) >= 0) return true;
    const long long t0 = clock64();
    for (;;) {
        if ((int32_t)(ld_relaxed_sys(p) - want) >= 0) return true;
        if (ld_relaxed_sys(ctl_local + CTL_ERR) != 0u) return false;  // someone already gave up
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            st_relaxed_sys(ctl_local + CTL_ERR, code);
            device_error(code, blockIdx.x, want);
            return false;
        }
        __nanosleep(32);
    }
}
// The launch number this kernel runs as.  Stable for the kernel's whole life: only the last CTA
// advances it, after every CTA has finished.  Call after the dependency wait.
__device__ __forceinline__ uint32_t peer_epoch(const PeerArgs& pa) {
    return ld_relaxed_sys(peer_ctl(pa, pa.rank) + CTL_EPOCH) + 1u;
}
// (1) one thread of the grid, after the dependency wait.  No fence: what the signal vouches
// for -- the completion of this rank's earlier kernels -- is given by the kernel boundary.
__device__ __forceinline__ void peer_announce_ready(const PeerArgs& pa, uint32_t e) {
    for (uint32_t p = 0; p < pa.world; ++p)
        if (p != pa.rank) st_relaxed_sys(peer_ctl(pa, p) + CTL_READY + pa.rank, e);
}
// (2) any thread about to store into peers' arenas (the stores depend on the loads' outcome)
__device__ __forceinline__ void peer_wait_ready(const PeerArgs& pa, uint32_t e) {
    uint32_t* ctl = peer_ctl(pa, pa.rank);
    for (uint32_t p = 0; p < pa.world; ++p)
        if (p != pa.rank && !peer_wait_ge(ctl, ctl + CTL_READY + p, e, 0x7E10u + p)) return;
}
// (3) one thread per CTA, after all of the CTA's stores (a CTA-wide barrier precedes the call)
__device__ __forceinline__ void peer_finish(const PeerArgs& pa, uint32_t e) {
    uint32_t* ctl = peer_ctl(pa, pa.rank);
    __threadfence_system();  // this CTA's peer stores are performed everywhere before it is counted
    if (atomicAdd(ctl + CTL_COUNT, 1u) != gridDim.x - 1u) return;
    // last CTA: every CTA's stores were performed before its increment, which this thread has
    // observed; order that observation before the signals
    __threadfence();
    ctl[CTL_COUNT] = 0u;
    for (uint32_t p = 0; p < pa.world; ++p)
        if (p != pa.rank) st_relaxed_sys(peer_ctl(pa, p) + CTL_DONE + pa.rank, e);
    // the peers' rows were performed in this GPU's memory before their signals left; kernels
    // that follow this one on the stream read them after the kernel boundary
    for (uint32_t p = 0; p < pa.world; ++p)
        if (p != pa.rank && !peer_wait_ge(ctl, ctl + CTL_DONE + p, e, 0x7E20u + p)) break;
    st_relaxed_sys(ctl + CTL_EPOCH, e);
}
#endif

}  // namespace miori_b200
