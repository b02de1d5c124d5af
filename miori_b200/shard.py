"""Partitioning of the quantized-matmul path across the GPUs of one box.

The reference is single-GPU; this is the multi-GPU plan of the B200 build:
  * decode GEMV: output rows N are split contiguously across ranks, every rank holds only its
    rows of q / s / b, x is replicated, and y is reassembled by an all-gather;
  * prefill GEMM and the cache build: token rows M are split across ranks, the weight cache is
    replicated, there is no collective.
Pure host logic (torch.distributed is the plumbing); it runs on CPU tensors with gloo as
well as on CUDA tensors with NCCL.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

ROW_ALIGN = 16  # GEMV kernels work on 16-row tiles; shard boundaries respect them


def row_range(total: int, rank: int, world: int, align: int = 1) -> tuple[int, int]:
    """Contiguous [begin, end) of `total` rows owned by `rank`: blocks of `align` rows are dealt
    as evenly as possible, earlier ranks taking the remainder; the last block may be ragged."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    blocks = (total + align - 1) // align
    base, extra = divmod(blocks, world)
    b0 = rank * base + min(rank, extra)
    b1 = b0 + base + (1 if rank < extra else 0)
    return min(b0 * align, total), min(b1 * align, total)


def shard_weight(q: torch.Tensor, s: torch.Tensor, b: torch.Tensor, rank: int, world: int):
    """This rank's rows of a quantized weight (q [N][words], s/b [N][K/group])."""
    r0, r1 = row_range(q.shape[0], rank, world, ROW_ALIGN)
    return q[r0:r1].contiguous(), s[r0:r1].contiguous(), b[r0:r1].contiguous()


def gather_rows(y_local: torch.Tensor, N: int, group=None) -> torch.Tensor:
    """All-gather the N-sharded GEMV output y_local [M][rows of this rank] into y [M][N].

    Ranks may own different row counts (ragged last shard), so the exchange pads every shard to
    the largest one; with equal shards it is a single all_gather_into_tensor.
    """
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    M = y_local.shape[0]
    sizes = [row_range(N, r, world, ROW_ALIGN) for r in range(world)]
    widest = max(e - b for b, e in sizes)
    send = y_local
    if y_local.shape[1] != widest:
        send = torch.zeros((M, widest), dtype=y_local.dtype, device=y_local.device)
        send[:, :y_local.shape[1]] = y_local
    recv = torch.empty((world * M, widest), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(recv, send.contiguous(), group=group)
    recv = recv.view(world, M, widest)
    out = torch.empty((M, N), dtype=y_local.dtype, device=y_local.device)
    for r, (b0, e0) in enumerate(sizes):
        out[:, b0:e0] = recv[r, :, :e0 - b0]
    return out


def token_range(M: int, rank: int, world: int) -> tuple[int, int]:
    """Rows of A (tokens) this rank multiplies in the M-sharded prefill GEMM."""
    return row_range(M, rank, world, 1)
