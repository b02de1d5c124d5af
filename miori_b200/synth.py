"""Seeded synthetic inputs for the quantized-matmul path (input generation only).

The reference has no quantizer (its weights arrive pre-quantized), so this is the
workload generator: fp32 W ~ N(0, 0.02^2) is affine-quantized per group along K in the
MLX format the kernels consume; activations are bf16 ~ N(0, 1).  Runs on CPU or GPU
tensors alike; both the CUDA path and the CPU oracle are fed the same outputs.
"""
from __future__ import annotations

import torch


def quantize_affine(W: torch.Tensor, bits: int, group: int):
    """Return (q int32 [N][K*bits/32], s bf16 [N][K/group], b bf16 [N][K/group]).

    scale=(max-min)/qmax and bias=min are stored as bf16 (round-to-nearest-even);
    q=round((w-bias)/scale) clamped to [0,qmax] against the stored values; codes are packed
    low nibble / low byte first.
    """
    assert bits in (4, 8) and W.dim() == 2
    N, K = W.shape
    assert K % group == 0
    per = 32 // bits
    qmax = float((1 << bits) - 1)
    Wg = W.float().reshape(N, K // group, group)
    mn = Wg.amin(dim=-1)
    mx = Wg.amax(dim=-1)
    sc = (mx - mn) / qmax
    sc = torch.where(sc > 0, sc, torch.ones_like(sc))
    s = sc.to(torch.bfloat16)
    b = mn.to(torch.bfloat16)
    codes = torch.round((Wg - b.float().unsqueeze(-1)) / s.float().unsqueeze(-1))
    codes = codes.clamp_(0, qmax).to(torch.int64).reshape(N, K // per, per)
    shifts = (torch.arange(per, device=W.device, dtype=torch.int64) * bits)
    packed = (codes << shifts).sum(dim=-1)
    packed = torch.where(packed >= 2**31, packed - 2**32, packed).to(torch.int32)
    return packed.contiguous(), s.contiguous(), b.contiguous()


def make_weight(N: int, K: int, bits: int, group: int, seed: int, device="cpu", std=0.02,
                chunk_rows: int = 16384):
    """Quantized W[N][K] ~ N(0, std^2) with a per-tensor seed, generated in row chunks."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    qs, ss, bs = [], [], []
    for r0 in range(0, N, chunk_rows):
        rows = min(chunk_rows, N - r0)
        W = torch.randn((rows, K), generator=gen, device=device, dtype=torch.float32) * std
        q, s, b = quantize_affine(W, bits, group)
        qs.append(q), ss.append(s), bs.append(b)
    return torch.cat(qs), torch.cat(ss), torch.cat(bs)


def make_activation(M: int, K: int, seed: int, device="cpu"):
    """bf16 x[M][K] ~ N(0,1)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    return torch.randn((M, K), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)


def ramp_activation(M: int, K: int, device="cpu"):
    """The reference test's deterministic ramp, src/main.cpp:28: ((k*37)%101-50)/50."""
    k = torch.arange(M * K, dtype=torch.int64, device=device)
    return ((((k * 37) % 101).float() - 50.0) / 50.0).to(torch.bfloat16).reshape(M, K)
