"""One rank's view of a group of GPUs that share output buffers over NVLink.

Each rank (one process per GPU) owns an arena of device memory that the other ranks map through
CUDA IPC.  Outputs of the N-sharded GEMV live at the same offset in every arena, and the kernel's
epilogue stores its rows into all of them (include/miori_b200.h, "multi-GPU").  The 64-byte
handles travel between the ranks through ``torch.distributed`` (any backend).
"""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import LAUNCH_PDL, OUT_BF16, check, lib  # noqa: F401


class _Raw:
    """A device pointer dressed as a CUDA array for torch.as_tensor."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr,
                                         "data": (ptr, False), "version": 2}


class PeerGroup:
    def __init__(self, rank: int, world: int, arena_bytes: int, device=None):
        self.rank, self.world = rank, world
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            check(lib.miori_peers_create(rank, world, arena_bytes, C.byref(h)))
        self._h = h
        self.arena_bytes = arena_bytes
        self._cursor = 0
        if world > 1:
            self._connect()

    def _connect(self):
        import torch.distributed as dist
        n = lib.miori_peers_handle_bytes()
        mine = (C.c_uint8 * n)()
        check(lib.miori_peers_handle(self._h, mine))
        # gloo moves CPU tensors, nccl CUDA tensors
        on = self.device if dist.get_backend() == "nccl" else torch.device("cpu")
        t = torch.tensor(list(mine), dtype=torch.uint8, device=on)
        out = torch.empty(self.world * n, dtype=torch.uint8, device=on)
        dist.all_gather_into_tensor(out, t)
        blob = bytes(out.cpu().tolist())
        err = None
        try:
            with torch.cuda.device(self.device):
                check(lib.miori_peers_connect(self._h, blob))
        except Exception as e:  # every rank must learn of it: the others would wait below
            err = e
        ok = torch.tensor([0 if err else 1], dtype=torch.int32, device=on)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            raise RuntimeError(f"peer mapping failed on some rank (this rank: {err})")

    def alloc(self, nbytes: int) -> int:
        """Carve `nbytes` out of the arena; every rank must make the same calls in the same order."""
        off = self._cursor
        self._cursor = (off + nbytes + 255) // 256 * 256
        if self._cursor > self.arena_bytes:
            raise MemoryError(f"arena of {self.arena_bytes} bytes exhausted")
        return off

    def tensor(self, offset: int, shape, dtype=torch.float32) -> torch.Tensor:
        """View of the local arena at `offset` (fp32 or bf16)."""
        ptr = lib.miori_peers_arena(self._h) + offset
        if dtype == torch.float32:
            return torch.as_tensor(_Raw(ptr, shape, "<f4"), device=self.device)
        if dtype == torch.bfloat16:
            return torch.as_tensor(_Raw(ptr, shape, "<i2"), device=self.device).view(torch.bfloat16)
        raise TypeError("fp32 or bf16 only")

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def gemv_allgather(self, bits, q, s, b, x, y_offset, row0, n_total, group=32, flags=0):
        """This rank's rows of y = W x, stored into every rank's arena at `y_offset`."""
        fn = lib.miori_gemv4_allgather if bits == 4 else lib.miori_gemv8_allgather
        M, K = x.shape
        check(fn(self._h, q.data_ptr(), s.data_ptr(), b.data_ptr(), x.data_ptr(), y_offset, q.shape[0],
                 row0, n_total, K, M, group, flags, self._stream()))

    def allgather(self, src, y_offset, row0, n_total, flags=0):
        """Copy src[M][n_local] into columns [row0, row0 + n_local) of y at `y_offset` everywhere."""
        M, n_local = src.shape
        check(lib.miori_allgather(self._h, src.data_ptr(), y_offset, M, n_local, row0, n_total,
                                  src.element_size(), flags, self._stream()))

    def argmax_allreduce(self, v, index0, y_offset, flags=0):
        """Greedy pick over an N-sharded vector: v holds this rank's elements, index0 the index of
        its first one.  Returns (index, value) read back from the arena after a synchronize."""
        f = flags | (OUT_BF16 if v.dtype == torch.bfloat16 else 0)
        check(lib.miori_argmax_allreduce(self._h, v.data_ptr(), v.numel(), index0, y_offset, f, self._stream()))

    def argmax_result(self, y_offset):
        """(index, value) left at y_offset by argmax_allreduce (call after synchronizing)."""
        pairs = self.tensor(y_offset, (2 * self.world + 2,)).cpu()
        w = 2 * self.world
        return int(pairs[w + 1:w + 2].view(torch.int32).item()), float(pairs[w].item())

    def gemv_argmax(self, bits, q, s, b, x, y_offset, best_offset, row0, n_total, group=32, flags=0):
        """This rank's rows of y = W x (one row of x) into its own arena, and the greedy pick over
        the whole sharded vector left at best_offset on every rank (see gemv_argmax_result)."""
        fn = lib.miori_gemv4_argmax if bits == 4 else lib.miori_gemv8_argmax
        M, K = x.shape
        if M != 1:
            raise ValueError("gemv_argmax takes one activation row")
        check(fn(self._h, q.data_ptr(), s.data_ptr(), b.data_ptr(), x.data_ptr(), y_offset, best_offset,
                 q.shape[0], row0, n_total, K, group, flags, self._stream()))

    def gemv_argmax_bytes(self) -> int:
        return lib.miori_gemv_argmax_bytes(self.world)

    def gemv_argmax_result(self, best_offset):
        """(index, value) left by gemv_argmax (call after synchronizing)."""
        words = self.tensor(best_offset, (4 + 2 * self.world + 2,)).cpu()
        w = 4 + 2 * self.world
        return int(words[w + 1:w + 2].view(torch.int32).item()), float(words[w].item())

    def set_wait_us(self, microseconds: int):
        """Limit of the kernels' waits for a peer (default about a second)."""
        check(lib.miori_peers_set_wait_us(self._h, microseconds))

    def status(self):
        check(lib.miori_peers_status(self._h))

    def close(self):
        if self._h:
            check(lib.miori_peers_destroy(self._h))
            self._h = None
