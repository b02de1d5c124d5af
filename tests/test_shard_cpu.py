"""Host logic of the multi-GPU plan on CPU: shard arithmetic, and a world_size-2 gloo run of
the N-sharded GEMV + all-gather and the M-sharded GEMM with the CPU oracle standing in for
the kernels (the oracle is the checker here, not a product path)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from miori_b200 import shard, synth
from conftest import u16, u32


def test_row_ranges_tile_the_rows():
    for total in (1, 15, 16, 17, 2048, 8192, 128000, 131072):
        for world in (1, 2, 3, 4, 8):
            got = [shard.row_range(total, r, world, 16) for r in range(world)]
            assert got[0][0] == 0 and got[-1][1] == total
            for (a0, a1), (b0, b1) in zip(got, got[1:]):
                assert a1 == b0 and a0 <= a1
            assert all(b % 16 == 0 or b == total for b, _ in got)
            sizes = [e - b for b, e in got]
            assert max(sizes) - min(sizes) <= 16 + 15
    assert shard.row_range(8192, 3, 8, 16) == (3072, 4096)
    with pytest.raises(ValueError):
        shard.row_range(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, N, K, M, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle
    orc = oracle.port()
    orc.set_threads(2)
    q, s, b = synth.make_weight(N, K, 4, 64, seed=3)      # same seed on every rank
    x = synth.make_activation(M, K, seed=4)
    ql, sl, bl = shard.shard_weight(q, s, b, rank, world)
    y_local = torch.from_numpy(orc.gemv(4, u32(ql), u16(sl), u16(bl), u16(x), 64)).float()
    y = shard.gather_rows(y_local, N)
    # M-sharded GEMM: every rank multiplies its token rows against the replicated cache
    cache = orc.dequant_rowmajor(4, u32(q), u16(s), u16(b), 64)
    A = synth.make_activation(37, K, seed=5)
    m0, m1 = shard.token_range(37, rank, world)
    c_local = orc.gemm_bf16(u16(A[m0:m1]), cache) if m1 > m0 else np.zeros((0, N))
    if rank == 0:
        want = orc.gemv(4, u32(q), u16(s), u16(b), u16(x), 64)
        np.save(out + ".y.npy", y.numpy())
        np.save(out + ".want.npy", want.astype(np.float32))
        np.save(out + ".c0.npy", c_local)
        np.save(out + ".cfull.npy", orc.gemm_bf16(u16(A), cache)[m0:m1])
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("N", [96, 100])  # equal shards, and a ragged last shard
def test_sharded_gemv_allgather_world2(tmp_path, N):
    out = str(tmp_path / "r")
    mp.spawn(_worker, args=(2, _free_port(), N, 128, 3, out), nprocs=2, join=True)
    y, want = np.load(out + ".y.npy"), np.load(out + ".want.npy")
    assert y.shape == want.shape and np.array_equal(y, want)
    assert np.array_equal(np.load(out + ".c0.npy"), np.load(out + ".cfull.npy"))


def test_split_plan():
    sizes = [3 << 20, 2 << 20, 18 << 20, 9 << 20]
    assert shard.split_plan(sizes, 1, 16 << 20) == [False] * 4
    assert shard.split_plan(sizes, 8, 16 << 20) == [False, False, True, False]
    assert shard.split_plan(sizes, 2, 16 << 20, "all") == [True] * 4
    assert shard.split_plan(sizes, 2, 16 << 20, "none") == [False] * 4
    with pytest.raises(ValueError):
        shard.split_plan(sizes, 2, 1, "some")


def test_argmax_candidate_order():
    nan = float("nan")
    assert shard.better((2.0, 9), (1.0, 0))
    assert shard.better((1.0, 3), (1.0, 4)) and not shard.better((1.0, 4), (1.0, 3))
    assert not shard.better((nan, 0), (-1e30, 5)) and shard.better((-1e30, 5), (nan, 0))


def _argmax_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    got = []
    for case in range(4):
        v = torch.randn(1000, generator=torch.Generator().manual_seed(case))
        if case == 1:    # the same maximum on both ranks: the lower index wins
            v[[17, 600]] = 7.0
        if case == 2:    # the maximum is the very last element
            v[999] = 8.0
        if case == 3:    # one rank holds nothing but NaN
            v[:500] = float("nan")
        r0, r1 = shard.row_range(1000, rank, world, 1)
        idx, val = shard.argmax_exchange(v[r0:r1], r0)
        want = int(torch.argmax(torch.nan_to_num(v, nan=float("-inf"))))
        got.append((idx, val, want, float(v[want])))
    np.save(out + f".{rank}.npy", np.array(got, dtype=np.float64))
    dist.barrier()
    dist.destroy_process_group()


def test_argmax_exchange_world2(tmp_path):
    out = str(tmp_path / "a")
    mp.spawn(_argmax_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    r0, r1 = np.load(out + ".0.npy"), np.load(out + ".1.npy")
    assert np.array_equal(r0, r1)                      # every rank ends with the same winner
    assert np.array_equal(r0[:, 0], r0[:, 2]) and np.array_equal(r0[:, 1], r0[:, 3])
    assert r0[1, 0] == 17 and r0[2, 0] == 999 and r0[3, 0] >= 500
