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


def split_plan(weight_bytes: list[int], world: int, threshold_bytes: int, mode: str = "policy") -> list[bool]:
    """Which projections of a decode chain are split by output rows.  A split saves
    weight_bytes * (1 - 1/world) of streaming per launch and costs one exchange of y, so it pays
    only above a size; below it every rank computes the whole projection and nothing crosses
    NVLink.  mode: "policy" (by `threshold_bytes`), "all", "none"."""
    if mode not in ("policy", "all", "none"):
        raise ValueError(f"unknown sharding mode {mode!r}")
    if world <= 1 or mode == "none":
        return [False] * len(weight_bytes)
    return [mode == "all" or nbytes >= threshold_bytes for nbytes in weight_bytes]


def better(a: tuple[float, int], b: tuple[float, int]) -> bool:
    """Order of the arg-max candidates (value, index): larger value first, then the lower index,
    so the winner is the first maximum of the unsharded vector; NaN never wins."""
    if a[0] != a[0]:
        return False
    return b[0] != b[0] or a[0] > b[0] or (a[0] == b[0] and a[1] < b[1])


def argmax_exchange(v_local: torch.Tensor, index0: int, group=None) -> tuple[int, float]:
    """Greedy pick over a vector split across ranks: every rank offers its best (value, index),
    the pairs are exchanged (2 words per rank instead of the whole vector) and every rank picks
    the same winner.  Host-side statement of what miori_argmax_allreduce does over peer stores."""
    v = v_local.reshape(-1).float()
    i = int(torch.argmax(torch.nan_to_num(v, nan=float("-inf"))).item()) if v.numel() else 0
    mine = torch.tensor([float(v[i]) if v.numel() else float("nan"), float(index0 + i)], dtype=torch.float64,
                        device=v.device)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return int(mine[1].item()), float(mine[0].item())
    pairs = torch.empty(world * 2, dtype=torch.float64, device=v.device)
    dist.all_gather_into_tensor(pairs, mine, group=group)
    best = (float("nan"), -1)
    for val, idx in pairs.view(world, 2).cpu().tolist():
        if better((val, int(idx)), best):
            best = (val, int(idx))
    return best[1], best[0]
