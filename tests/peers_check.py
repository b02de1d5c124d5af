"""Self-check of the multi-GPU path (a test helper, not part of the package): run one process per
GPU from the repository root, e.g.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29533 tests/peers_check.py

Every rank holds a row shard of the same seeded weights, runs the N-sharded GEMV whose epilogue
stores into all ranks' arenas, and compares its gathered y bit for bit with the single-GPU GEMV
over the whole matrix: eagerly, back to back with programmatic dependent launch, inside a replayed
CUDA graph, for 8-bit weights with bf16 output, for the stand-alone all-gather and for the
exchange of (value, index) pairs that finishes a sharded arg-max.  Exits non-zero on any mismatch
or if a bounded wait expired.

The last part checks the failure path without faulting anything: in a second group whose wait
limit is 20 ms, rank 1 leaves one launch out; every other rank's kernel gives up waiting for
rank 1's rows, returns, and the host reads the error (a device status, then MioriError from
`status()`).  Nobody exits before a host barrier, so no arena is unmapped under a store.
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main() -> int:
    import miori_b200
    from miori_b200 import synth
    from miori_b200.peers import PeerGroup

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("gloo")
    G, N, K = 64, 4096, 2048
    rows = N // world
    r0 = rank * rows
    grp = PeerGroup(rank, world, 16 << 20, dev)
    failures = []

    def host_barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def expect(ok, what):
        if not ok:
            failures.append(what)

    q, s, b = synth.make_weight(N, K, 4, G, seed=11, device=dev)
    qs, ss, bs = q[r0:r0 + rows].contiguous(), s[r0:r0 + rows].contiguous(), b[r0:r0 + rows].contiguous()
    pdl = miori_b200.LAUNCH_PDL
    # the kernels' waits for a peer are bounded (about a second): start level, whatever the ranks'
    # set-up cost was
    host_barrier()

    # eager, several launches in a row into the same y (exercises the ready/done counters)
    for M in (1, 2, 4, 8, 16):
        off = grp.alloc(M * N * 4)
        y = grp.tensor(off, (M, N))
        for it in range(3):
            x = synth.make_activation(M, K, seed=100 * M + it, device=dev)
            grp.gemv_allgather(4, qs, ss, bs, x, off, r0, N, group=G, flags=pdl)
            torch.cuda.synchronize()
            want = miori_b200.gemv4(q, s, b, x, group=G)
            expect(torch.equal(y, want), f"eager M={M} launch {it}")

    # a replayed CUDA graph of dependent launches alternating between two outputs
    M = 4
    offs = [grp.alloc(M * N * 4) for _ in range(2)]
    xs = [synth.make_activation(M, K, seed=900 + i, device=dev) for i in range(2)]

    def chain():
        for i in range(8):
            grp.gemv_allgather(4, qs, ss, bs, xs[i & 1], offs[i & 1], r0, N, group=G, flags=pdl)
    chain()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        chain()
    for _ in range(5):
        g.replay()
    torch.cuda.synchronize()
    for i in range(2):
        expect(torch.equal(grp.tensor(offs[i], (M, N)), miori_b200.gemv4(q, s, b, xs[i], group=G)),
               f"graph replay output {i}")

    # 8-bit weights, bf16 output
    q8, s8, b8 = synth.make_weight(N, K, 8, G, seed=12, device=dev)
    off8 = grp.alloc(2 * N * 2)
    x8 = synth.make_activation(2, K, seed=77, device=dev)
    grp.gemv_allgather(8, q8[r0:r0 + rows].contiguous(), s8[r0:r0 + rows].contiguous(),
                       b8[r0:r0 + rows].contiguous(), x8, off8, r0, N, group=G,
                       flags=pdl | miori_b200.OUT_BF16)
    torch.cuda.synchronize()
    want8 = miori_b200.gemv8(q8, s8, b8, x8, group=G, flags=miori_b200.OUT_BF16)
    expect(torch.equal(grp.tensor(off8, (2, N), torch.bfloat16), want8), "gemv8 bf16")

    # stand-alone all-gather of blocks written by another kernel
    M = 32
    offa = grp.alloc(M * N * 4)
    full = torch.arange(M * N, device=dev, dtype=torch.float32).reshape(M, N) * 0.5 + 3.0
    for it in range(2):
        blk = (full[:, r0:r0 + rows] + it).contiguous()
        grp.allgather(blk, offa, r0, N, flags=pdl)
        torch.cuda.synchronize()
        expect(torch.equal(grp.tensor(offa, (M, N)), full + it), f"allgather {it}")

    # sharded arg-max: every rank offers its best (value, index), all end with the same winner;
    # ties go to the lowest index
    for dt in (torch.float32, torch.bfloat16):
        for it in range(3):
            gen = torch.Generator(device="cpu").manual_seed(500 + it)
            v = torch.randn(N, generator=gen).to(dt)
            if it == 2:  # the same maximum on every rank
                v[torch.arange(world) * rows + 7] = 9.0
            offb = grp.alloc((2 * world + 2) * 4)
            grp.argmax_allreduce(v[r0:r0 + rows].to(dev).contiguous(), r0, offb, flags=pdl)
            torch.cuda.synchronize()
            want_v = float(v.float().max())
            want_i = int(torch.nonzero(v.float() == want_v)[0, 0])
            expect(grp.argmax_result(offb) == (want_i, want_v), f"argmax exchange {dt} case {it}")

    # the head and the greedy pick in one launch: every rank multiplies its rows, the ranks'
    # best candidates meet, and every rank ends with the arg-max of the whole vector
    q8[torch.arange(world) * rows + 5] = q8[3].clone()   # equal rows on every rank: ties across ranks
    s8[torch.arange(world) * rows + 5] = s8[3].clone()
    b8[torch.arange(world) * rows + 5] = b8[3].clone()
    offy = grp.alloc(N * 4)
    offb = grp.alloc(grp.gemv_argmax_bytes())
    for obf in (0, miori_b200.OUT_BF16):
        for it in range(3):
            xh = synth.make_activation(1, K, seed=300 + it, device=dev)
            grp.gemv_argmax(8, q8[r0:r0 + rows].contiguous(), s8[r0:r0 + rows].contiguous(),
                            b8[r0:r0 + rows].contiguous(), xh, offy, offb, r0, N, group=G, flags=pdl | obf)
            torch.cuda.synchronize()
            whole = miori_b200.gemv8(q8, s8, b8, xh, group=G, flags=obf)[0].float()
            want_i = int(torch.nonzero(whole == whole.max())[0, 0])
            expect(grp.gemv_argmax_result(offb) == (want_i, float(whole.max())),
                   f"gemv8_argmax bf16={bool(obf)} launch {it}")
            mine = grp.tensor(offy, (1, N), torch.bfloat16 if obf else torch.float32)[0, r0:r0 + rows].float()
            expect(torch.equal(mine, whole[r0:r0 + rows]), f"gemv8_argmax own rows bf16={bool(obf)} launch {it}")

    try:
        grp.status()
    except Exception as e:  # a bounded wait expired on this rank
        failures.append(str(e))
    expect(miori_b200.lib.miori_device_error_poll() == 0, "device error recorded")
    host_barrier()  # nobody unmaps an arena while a peer may still store into it
    grp.close()

    # the failure path: a peer that never sends.  Rank 1 skips one launch; the others' waits expire.
    if world > 1:
        grp = PeerGroup(rank, world, 1 << 20, dev)
        grp.set_wait_us(20000)
        offe = grp.alloc(N * 4)
        xe = synth.make_activation(1, K, seed=5, device=dev)
        host_barrier()
        grp.gemv_allgather(4, qs, ss, bs, xe, offe, r0, N, group=G)  # a complete launch first
        host_barrier()
        expect(torch.equal(grp.tensor(offe, (1, N)), miori_b200.gemv4(q, s, b, xe, group=G)), "launch before the gap")
        if rank != 1:
            grp.gemv_allgather(4, qs, ss, bs, xe, offe, r0, N, group=G)
        torch.cuda.synchronize()  # returns: the wait is bounded
        raised = False
        try:
            grp.status()
        except miori_b200.MioriError as e:
            raised = "gave up waiting" in str(e)
        code = miori_b200.lib.miori_device_error_poll()
        if rank != 1:
            expect(raised, "status() did not report the expired wait")
            expect(code != 0, "no device error recorded for the expired wait")
        else:
            expect(not raised and code == 0, "the rank that skipped its launch reports an error")
        # the context is still usable after the expiry
        y_after = miori_b200.gemv4(q, s, b, xe, group=G)
        torch.cuda.synchronize()
        expect(bool(torch.isfinite(y_after).all()), "launch after the expired wait")
    bad = torch.tensor([len(failures)])
    if world > 1:
        dist.all_reduce(bad)
    host_barrier()
    if world > 1:
        grp.close()
    if failures:
        print(f"[peers_check rank {rank}] FAILED: {failures}", file=sys.stderr, flush=True)
    if rank == 0:
        print("peers_check: " + ("ok" if int(bad.item()) == 0 else f"{int(bad.item())} failures")
              + f" (world {world})", flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 1 if int(bad.item()) else 0


if __name__ == "__main__":
    sys.exit(main())
