"""Tensor-level wrappers over the C ABI.  torch is used for device memory and streams
only; every computation happens in libmiori_b200.so."""
from __future__ import annotations

import torch

from ._lib import OUT_BF16, check, lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if not t.is_cuda:
            raise ValueError("miori_b200 ops need CUDA tensors (there is no CPU path)")
        if not t.is_contiguous():
            raise ValueError("miori_b200 ops need contiguous tensors")


def _gemv(fn, per_word, q, s, b, x, group, flags, out):
    _need_cuda(q, s, b, x)
    if x.dim() == 1:
        x = x.unsqueeze(0)
    M, K = x.shape
    N = q.shape[0]
    if q.shape[1] * per_word != K:
        raise ValueError(f"q has {q.shape[1]} words per row, expected {K // per_word}")
    dt = torch.bfloat16 if flags & OUT_BF16 else torch.float32
    y = out if out is not None else torch.empty((M, N), dtype=dt, device=x.device)
    check(fn(q.data_ptr(), s.data_ptr(), b.data_ptr(), x.data_ptr(), y.data_ptr(), N, K, M, group,
             flags, _stream()))
    return y


def gemv4(q, s, b, x, group=32, flags=0, out=None):
    """y[M][N] for packed 4-bit weights q[N][K/8] (int32 words), s/b[N][K/group] bf16."""
    return _gemv(lib.miori_gemv4, 8, q, s, b, x, group, flags, out)


def gemv8(q, s, b, x, group=32, flags=0, out=None):
    """y[M][N] for packed 8-bit weights q[N][K/4] (int32 words)."""
    return _gemv(lib.miori_gemv8, 4, q, s, b, x, group, flags, out)


def _dequant(fn, per_word, q, s, b, group, out):
    _need_cuda(q, s, b)
    N, K = q.shape[0], q.shape[1] * per_word
    o = out if out is not None else torch.empty((N, K), dtype=torch.bfloat16, device=q.device)
    check(fn(q.data_ptr(), s.data_ptr(), b.data_ptr(), o.data_ptr(), N, K, group, _stream()))
    return o


def dequant4_rowmajor(q, s, b, group=32, out=None):
    return _dequant(lib.miori_dequant4_rowmajor, 8, q, s, b, group, out)


def dequant8_rowmajor(q, s, b, group=32, out=None):
    return _dequant(lib.miori_dequant8_rowmajor, 4, q, s, b, group, out)


def dequant4_cache(q, s, b, group=32, out=None):
    """Layout-opaque bf16 cache for gemm_bf16_cache (returned as a flat bf16 tensor)."""
    _need_cuda(q, s, b)
    N, K = q.shape[0], q.shape[1] * 8
    nbytes = lib.miori_cache_bytes(N, K)
    o = out if out is not None else torch.empty(nbytes // 2, dtype=torch.bfloat16, device=q.device)
    check(lib.miori_dequant4_cache(q.data_ptr(), s.data_ptr(), b.data_ptr(), o.data_ptr(), N, K,
                                   group, _stream()))
    return o


def cache_to_rowmajor(cache, N, K):
    _need_cuda(cache)
    o = torch.empty((N, K), dtype=torch.bfloat16, device=cache.device)
    check(lib.miori_cache_to_rowmajor(cache.data_ptr(), o.data_ptr(), N, K, _stream()))
    return o


def gemm_workspace(M, N, K, device):
    """Scratch tensor of the size miori_gemm_workspace_bytes recommends, or None."""
    nbytes = lib.miori_gemm_workspace_bytes(M, N, K)
    return torch.empty(nbytes // 4, dtype=torch.float32, device=device) if nbytes else None


def gemm_bf16_cache(A, cache, N, flags=0, out=None, workspace=None):
    """C[M][N] = A[M][K] x cache(N,K)^T on the tcgen05 tensor cores (split-K if a workspace
    tensor is given and the shape has few output tiles)."""
    _need_cuda(A, cache)
    M, K = A.shape
    dt = torch.bfloat16 if flags & OUT_BF16 else torch.float32
    Cm = out if out is not None else torch.empty((M, N), dtype=dt, device=A.device)
    wp = workspace.data_ptr() if workspace is not None else None
    wb = workspace.numel() * workspace.element_size() if workspace is not None else 0
    check(lib.miori_gemm_bf16_cache_ws(A.data_ptr(), cache.data_ptr(), Cm.data_ptr(), M, N, K, flags,
                                       wp, wb, _stream()))
    return Cm


def gemm_bf16_strided(A, B, flags=0, out=None):
    """C[M][N] = A[M][K] x B[N][K]^T for bf16 operands whose rows may be strided (views of
    larger tensors, last dimension contiguous); `out` may be a strided view too."""
    if not (A.is_cuda and B.is_cuda):
        raise ValueError("miori_b200 ops need CUDA tensors (there is no CPU path)")
    if A.dtype != torch.bfloat16 or B.dtype != torch.bfloat16:
        raise TypeError("gemm_bf16_strided: bf16 operands expected")
    M, K = A.shape
    N = B.shape[0]
    if B.shape[1] != K or A.stride(1) != 1 or B.stride(1) != 1:
        raise ValueError("gemm_bf16_strided: A [M][K] and B [N][K] with contiguous rows expected")
    dt = torch.bfloat16 if flags & OUT_BF16 else torch.float32
    Cm = out if out is not None else torch.empty((M, N), dtype=dt, device=A.device)
    if Cm.dtype != dt or Cm.shape != (M, N) or Cm.stride(1) != 1:
        raise ValueError("gemm_bf16_strided: bad output tensor")
    check(lib.miori_gemm_bf16_strided(A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0),
                                      Cm.data_ptr(), Cm.stride(0), M, N, K, flags, _stream()))
    return Cm


def gemv_bf16_cache(x, cache, N, flags=0, out=None):
    """y[M][N] = x[M][K] (bf16) against the bf16 cache, M <= 32: the narrow-batch kernel."""
    _need_cuda(x, cache)
    M, K = x.shape
    dt = torch.bfloat16 if flags & OUT_BF16 else torch.float32
    y = out if out is not None else torch.empty((M, N), dtype=dt, device=x.device)
    check(lib.miori_gemv_bf16_cache(x.data_ptr(), cache.data_ptr(), y.data_ptr(), M, N, K, flags, _stream()))
    return y


def linear4(q, s, b, cache, x, group=32, flags=0, out=None, workspace=None):
    """Projection dispatch: packed-weight GEMV up to four rows, the bf16 cache above (narrow-batch
    kernel or tensor-core GEMM by shape; lib.miori_linear4_route tells which)."""
    _need_cuda(q, s, b, x)
    M, K = x.shape
    N = q.shape[0]
    y = out if out is not None else torch.empty((M, N), dtype=torch.float32, device=x.device)
    wp = workspace.data_ptr() if workspace is not None else None
    wb = workspace.numel() * workspace.element_size() if workspace is not None else 0
    check(lib.miori_linear4(q.data_ptr(), s.data_ptr(), b.data_ptr(),
                            cache.data_ptr() if cache is not None else None, x.data_ptr(),
                            y.data_ptr(), N, K, M, group, flags, wp, wb, _stream()))
    return y


def rmsnorm(x, gamma, eps, flags=0, out=None):
    """bf16(x * rsqrt(mean(x^2) + eps) * gamma): x fp32 [rows][n], gamma bf16 [n]."""
    _need_cuda(x, gamma)
    rows, n = x.shape
    y = out if out is not None else torch.empty((rows, n), dtype=torch.bfloat16, device=x.device)
    check(lib.miori_rmsnorm(x.data_ptr(), gamma.data_ptr(), y.data_ptr(), rows, n, float(eps), flags, _stream()))
    return y


def post_norm_add(x, src, gamma, eps, flags=0, out=None):
    """x + src * rsqrt(mean(src^2) + eps) * gamma, fp32 [rows][n]; gamma bf16 [n]."""
    _need_cuda(x, src, gamma)
    rows, n = x.shape
    o = out if out is not None else torch.empty_like(x)
    check(lib.miori_post_norm_add(x.data_ptr(), src.data_ptr(), gamma.data_ptr(), o.data_ptr(), rows, n,
                                  float(eps), flags, _stream()))
    return o


def silu_mul(gate, up, flags=0, out=None):
    """bf16(gate / (1 + exp(-gate)) * up), fp32 inputs of the same shape."""
    _need_cuda(gate, up)
    o = out if out is not None else torch.empty(gate.shape, dtype=torch.bfloat16, device=gate.device)
    check(lib.miori_silu_mul(gate.data_ptr(), up.data_ptr(), o.data_ptr(), gate.numel(), flags, _stream()))
    return o


def embed8(q, s, b, tokens, group=32, flags=0, out=None):
    """Rows tokens[t] of the 8-bit table q [rows][K/4] dequantized to bf16 [T][K]."""
    _need_cuda(q, s, b, tokens)
    rows, K = q.shape[0], q.shape[1] * 4
    T = tokens.numel()
    o = out if out is not None else torch.empty((T, K), dtype=torch.bfloat16, device=q.device)
    check(lib.miori_embed8(q.data_ptr(), s.data_ptr(), b.data_ptr(), tokens.data_ptr(), o.data_ptr(), T, rows,
                           K, group, flags, _stream()))
    return o


def argmax(v, flags=0):
    """(index, value) tensors of the largest element of a 1-D fp32 or bf16 vector; ties: lowest index."""
    _need_cuda(v)
    f = flags | (OUT_BF16 if v.dtype == torch.bfloat16 else 0)
    idx = torch.empty(1, dtype=torch.int32, device=v.device)
    val = torch.empty(1, dtype=torch.float32, device=v.device)
    check(lib.miori_argmax(v.data_ptr(), v.numel(), f, idx.data_ptr(), val.data_ptr(), _stream()))
    return idx, val


def _gemv_rmsnorm(fn, per_word, q, s, b, x, gamma, eps, group, flags, out):
    _need_cuda(q, s, b, x, gamma)
    if x.dtype != torch.float32:
        raise TypeError("the fused norm takes fp32 activations")
    if x.dim() == 1:
        x = x.unsqueeze(0)
    M, K = x.shape
    N = q.shape[0]
    dt = torch.bfloat16 if flags & OUT_BF16 else torch.float32
    y = out if out is not None else torch.empty((M, N), dtype=dt, device=x.device)
    check(fn(q.data_ptr(), s.data_ptr(), b.data_ptr(), x.data_ptr(), gamma.data_ptr(), float(eps), y.data_ptr(),
             N, K, M, group, flags, _stream()))
    return y


def gemv4_rmsnorm(q, s, b, x, gamma, eps, group=32, flags=0, out=None):
    """gemv4 over bf16(rmsnorm(x) * gamma) with the norm fused into the kernel's activation staging."""
    return _gemv_rmsnorm(lib.miori_gemv4_rmsnorm, 8, q, s, b, x, gamma, eps, group, flags, out)


def gemv8_rmsnorm(q, s, b, x, gamma, eps, group=32, flags=0, out=None):
    return _gemv_rmsnorm(lib.miori_gemv8_rmsnorm, 4, q, s, b, x, gamma, eps, group, flags, out)


def gemv4_silu(q, s, b, x, group=32, flags=0, out=None):
    """bf16(silu(gate) * up) [M][N/2] for the fused gate + up weights q [N][K/8] (gate rows first):
    gemv4 with silu_mul as its epilogue."""
    _need_cuda(q, s, b, x)
    if x.dim() == 1:
        x = x.unsqueeze(0)
    M, K = x.shape
    N = q.shape[0]
    if q.shape[1] * 8 != K:
        raise ValueError(f"q has {q.shape[1]} words per row, expected {K // 8}")
    y = out if out is not None else torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    check(lib.miori_gemv4_silu(q.data_ptr(), s.data_ptr(), b.data_ptr(), x.data_ptr(), y.data_ptr(), N, K, M,
                               group, flags, _stream()))
    return y


def gemv4_post_norm_add(q, s, b, x, residual, gamma, eps, counter, group=32, flags=0, out=None):
    """residual + v * rsqrt(mean(v^2) + eps) * gamma for v = gemv4(x), fp32 [M][N], M <= 4: gemv4 with
    post_norm_add as its epilogue.  `counter`: a zeroed int32 tensor of one element, left zero."""
    _need_cuda(q, s, b, x, residual, gamma, counter)
    if x.dim() == 1:
        x = x.unsqueeze(0)
    M, K = x.shape
    N = q.shape[0]
    if q.shape[1] * 8 != K:
        raise ValueError(f"q has {q.shape[1]} words per row, expected {K // 8}")
    if residual.dtype != torch.float32 or residual.numel() != M * N:
        raise ValueError("residual: fp32 [M][N] expected")
    o = out if out is not None else torch.empty((M, N), dtype=torch.float32, device=x.device)
    check(lib.miori_gemv4_post_norm_add(q.data_ptr(), s.data_ptr(), b.data_ptr(), x.data_ptr(), residual.data_ptr(),
                                        gamma.data_ptr(), float(eps), counter.data_ptr(), o.data_ptr(), N, K, M,
                                        group, flags, _stream()))
    return o


def gemv4_rmsnorm_silu(q, s, b, x, gamma, eps, group=32, flags=0, out=None):
    """bf16(silu(gate) * up) [M][N/2] of the fused gate + up weights applied to bf16(rmsnorm(x) * gamma),
    x fp32 [M][K], M <= 4: one launch for the norm, both projections and the activation."""
    _need_cuda(q, s, b, x, gamma)
    if x.dtype != torch.float32:
        raise TypeError("the fused norm takes fp32 activations")
    if x.dim() == 1:
        x = x.unsqueeze(0)
    M, K = x.shape
    N = q.shape[0]
    y = out if out is not None else torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    check(lib.miori_gemv4_rmsnorm_silu(q.data_ptr(), s.data_ptr(), b.data_ptr(), x.data_ptr(), gamma.data_ptr(),
                                       float(eps), y.data_ptr(), N, K, M, group, flags, _stream()))
    return y
