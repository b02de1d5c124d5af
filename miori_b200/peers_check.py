"""Self-check of the multi-GPU path: run one process per GPU, e.g.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29533 -m miori_b200.peers_check

Every rank holds a row shard of the same seeded weights, runs the N-sharded GEMV whose epilogue
stores into all ranks' arenas, and compares its gathered y bit for bit with the single-GPU GEMV
over the whole matrix: eagerly, back to back with programmatic dependent launch, inside a replayed
CUDA graph, for 8-bit weights with bf16 output, and for the stand-alone all-gather.  Exits non-zero
on any mismatch or if a bounded wait expired.
"""
from __future__ import annotations

import os
import sys

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

    def expect(ok, what):
        if not ok:
            failures.append(what)

    q, s, b = synth.make_weight(N, K, 4, G, seed=11, device=dev)
    qs, ss, bs = q[r0:r0 + rows].contiguous(), s[r0:r0 + rows].contiguous(), b[r0:r0 + rows].contiguous()
    pdl = miori_b200.LAUNCH_PDL

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

    try:
        grp.status()
    except Exception as e:  # a bounded wait expired on this rank
        failures.append(str(e))
    expect(miori_b200.lib.miori_device_error_poll() == 0, "device error recorded")
    bad = torch.tensor([len(failures)])
    if world > 1:
        dist.all_reduce(bad)
        dist.barrier()  # nobody unmaps an arena while a peer may still store into it
    torch.cuda.synchronize()
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
