"""Multi-GPU path: N-sharded GEMV with the all-gather fused into the epilogue (peer stores).

One GPU covers the entry points with a world of one rank (the kernel then takes its ordinary
path and writes into the arena).  With two or more GPUs the check runs as one process per GPU;
the ranks compare their gathered outputs bit for bit with the single-GPU GEMV, which the other
GPU tests compare with the oracle.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_world_of_one_writes_into_the_arena(port):
    import numpy as np
    import miori_b200
    from miori_b200 import synth
    from miori_b200.peers import PeerGroup
    from conftest import assert_close, u16, u32

    dev = torch.device("cuda", 0)
    N, K, G = 1024, 2048, 64
    q, s, b = synth.make_weight(N, K, 4, G, seed=5, device=dev)
    grp = PeerGroup(0, 1, 1 << 20, dev)
    try:
        for M in (1, 8):
            x = synth.make_activation(M, K, seed=6 + M, device=dev)
            off = grp.alloc(M * N * 4)
            grp.gemv_allgather(4, q, s, b, x, off, 0, N, group=G)
            torch.cuda.synchronize()
            y = grp.tensor(off, (M, N))
            assert torch.equal(y, miori_b200.gemv4(q, s, b, x, group=G))
            assert_close(y.cpu().numpy(), port.gemv(4, u32(q), u16(s), u16(b), u16(x), G), what=f"M={M}")
        # the stand-alone all-gather degenerates to a copy
        src = torch.randn(4, N, device=dev)
        off = grp.alloc(4 * N * 4)
        grp.allgather(src, off, 0, N)
        torch.cuda.synchronize()
        assert torch.equal(grp.tensor(off, (4, N)), src)
        # argument checks: a y that does not fit, rows outside the matrix
        with pytest.raises(miori_b200.MioriError):
            grp.gemv_allgather(4, q, s, b, x, (1 << 20) - 256, 0, N, group=G)
        with pytest.raises(miori_b200.MioriError):
            grp.gemv_allgather(4, q, s, b, x, 0, 16, N, group=G)
        grp.status()
    finally:
        grp.close()


@pytest.mark.parametrize("bits,out_bf16", [(8, True), (8, False), (4, False)])
def test_head_and_greedy_pick_in_one_launch(bits, out_bf16):
    """miori_gemv{4,8}_argmax with a world of one rank: the logits land in the arena and the
    winner equals the arg-max of those logits (first maximum), launch after launch (the scratch
    resets itself), also when several rows tie and inside a replayed CUDA graph."""
    import miori_b200
    from miori_b200 import synth
    from miori_b200.peers import PeerGroup

    dev = torch.device("cuda", 0)
    N, K, G = 20000, 2048, 64
    q, s, b = synth.make_weight(N, K, bits, G, seed=15, device=dev)
    q[4000:4003] = q[123].clone()  # three more rows equal to row 123: whatever wins, ties exist somewhere
    s[4000:4003] = s[123].clone()
    b[4000:4003] = b[123].clone()
    fn = miori_b200.gemv8 if bits == 8 else miori_b200.gemv4
    flags = miori_b200.OUT_BF16 if out_bf16 else 0
    grp = PeerGroup(0, 1, 1 << 20, dev)
    try:
        off_y = grp.alloc(N * 4)
        off_b = grp.alloc(grp.gemv_argmax_bytes())
        for it in range(4):
            x = synth.make_activation(1, K, seed=30 + it, device=dev)
            grp.gemv_argmax(bits, q, s, b, x, off_y, off_b, 0, N, group=G, flags=flags)
            torch.cuda.synchronize()
            want = fn(q, s, b, x, group=G, flags=flags)[0].float()
            y = grp.tensor(off_y, (1, N), torch.bfloat16 if out_bf16 else torch.float32)[0].float()
            assert torch.equal(y, want)
            idx, val = grp.gemv_argmax_result(off_b)
            first = int(torch.nonzero(want == want.max())[0, 0])
            assert (idx, val) == (first, float(want.max())), f"launch {it}"
        # replayed graph of dependent launches
        x = synth.make_activation(1, K, seed=99, device=dev)
        pdl = miori_b200.LAUNCH_PDL

        def chain():
            for _ in range(5):
                grp.gemv_argmax(bits, q, s, b, x, off_y, off_b, 0, N, group=G, flags=flags | pdl)
        chain()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            chain()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        want = fn(q, s, b, x, group=G, flags=flags)[0].float()
        idx, val = grp.gemv_argmax_result(off_b)
        assert (idx, val) == (int(torch.nonzero(want == want.max())[0, 0]), float(want.max()))
        grp.status()
        assert miori_b200.lib.miori_device_error_poll() == 0
    finally:
        grp.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_gather_bit_exact():
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
         "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(ROOT, "tests", "peers_check.py")],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "peers_check: ok" in r.stdout
