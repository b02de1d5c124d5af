"""GPU parity of the prefill GEMM (tcgen05) against the CPU oracle, through the C ABI.

The reference has no GEMM-vs-CPU test (its GEMM is a closed library call); the contract is
max|d| <= 1e-2*max|ref| and cosine >= 0.9999 against an exact product over the bit-exact
bf16 cache, plus the reference's own tile-shape invariance (src/main.cpp:1403-1443).
"""
import numpy as np
import pytest
import torch

import miori_b200
from miori_b200 import ops, synth
from conftest import assert_close, u16, u32

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
WIDE, NARROW, PAIR, NOPAIR = 0x200, 0x100, 0x4000, 0x8000  # kernel-shape overrides (tuning flags)


def _weights(N, K, group, seed):
    q, s, b = synth.make_weight(N, K, 4, group, seed=seed, device=DEV)
    cache = miori_b200.dequant4_cache(q, s, b, group=group)
    return q, s, b, cache


@pytest.mark.parametrize("flags", [0, WIDE, NARROW, PAIR])
@pytest.mark.parametrize("M,N,K", [(192, 512, 2048), (64, 256, 64), (1, 8, 64), (128, 128, 128),
                                   (300, 1000, 448), (33, 16, 2048), (257, 6144, 512)])
def test_gemm_matches_oracle(port, M, N, K, flags):
    q, s, b, cache = _weights(N, K, 32, seed=M + N + K)
    A = synth.make_activation(M, K, seed=3, device=DEV)
    Cm = miori_b200.gemm_bf16_cache(A, cache, N, flags=flags)
    torch.cuda.synchronize()
    Bc = port.dequant_rowmajor(4, u32(q), u16(s), u16(b), 32)
    want = port.gemm_bf16(u16(A), Bc)
    assert_close(Cm.cpu().numpy(), want, rel_max=1e-4, what=f"gemm {M}x{N}x{K} flags={flags:#x}")
    assert miori_b200.lib.miori_device_error_poll() == 0


@pytest.mark.parametrize("N,K", [(3072, 2048), (2048, 2048), (16384, 2048), (2048, 8192)])
def test_prefill_shapes_sampled(port, N, K):
    """M=1024 prefill over the four projection shapes: 4096 sampled entries vs the oracle."""
    M = 1024
    q, s, b, cache = _weights(N, K, 64, seed=N + K)
    A = synth.make_activation(M, K, seed=5, device=DEV)
    Cm = miori_b200.gemm_bf16_cache(A, cache, N).cpu().numpy()
    rng = np.random.default_rng(N + K)
    ms, ns = rng.integers(0, M, 4096), rng.integers(0, N, 4096)
    rows = np.unique(ns)
    Bc = port.dequant_rowmajor(4, u32(q[rows]), u16(s[rows]), u16(b[rows]), 64)
    where = {int(n): i for i, n in enumerate(rows)}
    An = u16(A)
    want = np.array([port.gemm_entry(An, Bc, int(m), where[int(n)]) for m, n in zip(ms, ns)])
    got = Cm[ms, ns]
    assert_close(got, want, rel_max=1e-4, what=f"prefill N={N} K={K}")
    assert np.isfinite(Cm).all()
    # packed prefill (32 prompts x 32 tokens) is the same product: rows are independent
    Cp = torch.cat([miori_b200.gemm_bf16_cache(A[i:i + 32].contiguous(), cache, N)
                    for i in range(0, 128, 32)]).cpu().numpy()
    assert np.array_equal(Cp, Cm[:128])


def test_rows_do_not_depend_on_m_tiling():
    """The reference's test-mpp-tile: 23 rows through three launch shapes, 0 differences."""
    N, K = 6144, 2048
    _, _, _, cache = _weights(N, K, 32, seed=8)
    A = synth.ramp_activation(64, K).to(DEV)
    c23 = miori_b200.gemm_bf16_cache(A[:23].contiguous(), cache, N)
    c64 = miori_b200.gemm_bf16_cache(A, cache, N)
    c23w = miori_b200.gemm_bf16_cache(A[:23].contiguous(), cache, N, flags=WIDE)
    c64p = miori_b200.gemm_bf16_cache(A, cache, N, flags=PAIR)
    assert torch.equal(c23, c64[:23])
    assert torch.equal(c23, c23w)
    assert torch.equal(c64p, c64)


def test_bf16_output_and_guard_bands():
    M, N, K = 200, 1032, 256
    _, _, _, cache = _weights(N, K, 32, seed=9)
    A = synth.make_activation(M, K, seed=10, device=DEV)
    c32 = miori_b200.gemm_bf16_cache(A, cache, N)
    c16 = miori_b200.gemm_bf16_cache(A, cache, N, flags=miori_b200.OUT_BF16)
    assert torch.equal(c16, c32.to(torch.bfloat16))
    buf = torch.full((M * N + 2048,), 777.0, device=DEV)
    out = buf[1024:1024 + M * N].view(M, N)
    miori_b200.gemm_bf16_cache(A, cache, N, out=out)
    torch.cuda.synchronize()
    assert (buf[:1024] == 777.0).all() and (buf[1024 + M * N:] == 777.0).all()
    assert torch.equal(out, c32)


def test_linearity_at_full_size():
    """Size-independent property at M=8192: C(A1+A2) = C(A1)+C(A2) when the sum is exact in
    bf16 (A2 = A1 gives 2*A1), and C is reproducible run to run."""
    M, N, K = 8192, 2048, 2048
    _, _, _, cache = _weights(N, K, 64, seed=12)
    A = synth.make_activation(M, K, seed=13, device=DEV)
    c1 = miori_b200.gemm_bf16_cache(A, cache, N)
    c2 = miori_b200.gemm_bf16_cache((A.float() * 2).to(torch.bfloat16), cache, N)
    assert torch.equal(c2, c1 * 2)
    assert torch.equal(miori_b200.gemm_bf16_cache(A, cache, N), c1)
    ref = A[:64].float() @ ops.cache_to_rowmajor(cache, N, K).float().T  # torch fp32 spot check
    assert torch.allclose(c1[:64], ref, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("M,N,K", [(32, 2048, 2048), (16, 3072, 2048), (32, 2048, 8192), (9, 512, 1024),
                                   (200, 256, 4096)])
def test_split_k_with_workspace_matches_oracle(port, M, N, K):
    """Few output tiles: K is split across SMs through a caller-provided workspace and summed
    in a fixed order."""
    q, s, b, cache = _weights(N, K, 64, seed=M * 3 + N + K)
    A = synth.make_activation(M, K, seed=21, device=DEV)
    ws = miori_b200.gemm_workspace(M, N, K, DEV)
    assert ws is not None, "expected this shape to split"
    c_split = miori_b200.gemm_bf16_cache(A, cache, N, workspace=ws)
    c_plain = miori_b200.gemm_bf16_cache(A, cache, N)
    torch.cuda.synchronize()
    want = port.gemm_bf16(u16(A), port.dequant_rowmajor(4, u32(q), u16(s), u16(b), 64))
    assert_close(c_split.cpu().numpy(), want, rel_max=1e-4, what=f"split-K {M}x{N}x{K}")
    assert_close(c_plain.cpu().numpy(), want, rel_max=1e-4, what=f"plain {M}x{N}x{K}")
    # reproducible, independent of M, bf16 epilogue is the rounded fp32 result
    assert torch.equal(miori_b200.gemm_bf16_cache(A, cache, N, workspace=ws), c_split)
    half = miori_b200.gemm_bf16_cache(A[:M // 2 + 1].contiguous(), cache, N, workspace=ws)
    assert torch.equal(half, c_split[:M // 2 + 1])
    c16 = miori_b200.gemm_bf16_cache(A, cache, N, flags=miori_b200.OUT_BF16, workspace=ws)
    assert torch.equal(c16, c_split.to(torch.bfloat16))
    assert miori_b200.lib.miori_device_error_poll() == 0


@pytest.mark.parametrize("N,K", [(3072, 2048), (2048, 8192), (6144, 2048)])
@pytest.mark.parametrize("M", [1, 4, 5, 8, 9, 16, 17, 32])
def test_linear_dispatch(port, M, N, K):
    """miori_linear4 keeps up to four rows on the packed weights (the reference's cut-over,
    src/batch.cpp:223-230) and sends wider batches to the bf16 cache -- the narrow-batch kernel or
    the tensor-core GEMM by shape -- unless no cache is given; miori_linear4_route says which, and
    the result is that entry's own."""
    q, s, b, cache = _weights(N, K, 64, seed=31)
    x = synth.make_activation(M, K, seed=32, device=DEV)
    ws = miori_b200.gemm_workspace(max(M, 9), N, K, DEV)
    y = miori_b200.linear4(q, s, b, cache, x, group=64, workspace=ws)
    y_nocache = miori_b200.linear4(q, s, b, None, x, group=64)
    torch.cuda.synchronize()
    want = port.gemv(4, u32(q), u16(s), u16(b), u16(x), 64)
    assert_close(y.cpu().numpy(), want, what=f"linear4 M={M}")
    assert_close(y_nocache.cpu().numpy(), want, what=f"linear4 (no cache) M={M}")
    r = miori_b200.lib.miori_linear4_route(M, N, K, 1)
    assert miori_b200.lib.miori_linear4_route(M, N, K, 0) == 0
    assert (r == 0) == (M <= 4 or (N == 6144 and M <= 8))
    if r == 0:
        assert torch.equal(y, miori_b200.gemv4(q, s, b, x, group=64))
    elif r == 1:
        assert torch.equal(y, miori_b200.gemv_bf16_cache(x, cache, N))
    else:
        assert torch.equal(y, miori_b200.gemm_bf16_cache(x, cache, N, workspace=ws))
    assert torch.equal(y_nocache, miori_b200.gemv4(q, s, b, x, group=64))


@pytest.mark.parametrize("M,N,K", [(32, 2048, 2048), (16, 3072, 2048), (5, 1000, 512), (1, 16, 64), (9, 17, 1096),
                                   (16, 2048, 4096), (24, 640, 2048), (32, 16384, 2048), (31, 100, 2048),
                                   (8, 512, 8192), (32, 256, 1536), (16, 2048, 8192), (32, 2048, 8192),
                                   (32, 100, 4096), (24, 700, 6144), (9, 4000, 8192)])
def test_narrow_batch_cache_kernel(port, M, N, K):
    """miori_gemv_bf16_cache against the oracle's exact product over the bit-exact cache, with the
    GEMM's tolerance; a row's value does not depend on M within a class of batch sizes (1..8,
    9..16, 17..32: the classes split k over the warps differently); bf16 output is the rounded fp32
    one; a K that is not a multiple of the 512-wide slab is zero-filled, not read past."""
    Kq = (K + 63) // 64 * 64
    q, s, b, cache = _weights(N, Kq, 64, seed=M + N + K)
    rm = ops.cache_to_rowmajor(cache, N, Kq)[:, :K].contiguous()
    x = synth.make_activation(M, K, seed=7, device=DEV)
    y = miori_b200.gemv_bf16_cache(x, rm.reshape(-1), N)
    torch.cuda.synchronize()
    want = port.gemm_bf16(u16(x), u16(rm))
    assert_close(y.cpu().numpy(), want, rel_max=1e-4, what=f"narrow batch {M}x{N}x{K}")
    h = max(1, M // 2) if M <= 8 else 9 if M <= 16 else 17   # the smallest batch of M's class
    assert torch.equal(miori_b200.gemv_bf16_cache(x[:h].contiguous(), rm.reshape(-1), N), y[:h])
    assert torch.equal(miori_b200.gemv_bf16_cache(x, rm.reshape(-1), N, flags=miori_b200.OUT_BF16), y.to(torch.bfloat16))
    assert miori_b200.lib.miori_device_error_poll() == 0


def test_narrow_batch_cache_kernel_random_shapes():
    """Sixty seeded random shapes -- N from 1 (ragged tiles, fewer tiles than SMs) to a few thousand,
    K any multiple of 8 up to 8192 (ragged last slab, K shorter than one MMA step's 32, rows whose
    fragments are resident in registers and rows that are streamed), every batch class -- against a plain fp32 product of the same bf16 operands."""
    g = torch.Generator().manual_seed(1234)
    for case in range(60):
        M = int(torch.randint(1, 33, (1,), generator=g))
        kmax = 8192
        K = 8 * int(torch.randint(1, kmax // 8 + 1, (1,), generator=g))
        N = int(torch.randint(1, 3000, (1,), generator=g)) if case % 3 else int(torch.randint(1, 40, (1,), generator=g))
        W = (torch.randn((N, K), generator=g) * 0.05).to(torch.bfloat16).to(DEV)
        x = torch.randn((M, K), generator=g).to(torch.bfloat16).to(DEV)
        y = miori_b200.gemv_bf16_cache(x, W.reshape(-1), N)
        want = x.float() @ W.float().T
        err = float((y - want).abs().max() / want.abs().max().clamp_min(1e-30))
        assert err <= 1e-4, f"case {case}: M={M} N={N} K={K} rel={err:.2e}"
    assert miori_b200.lib.miori_device_error_poll() == 0


def test_narrow_batch_cache_kernel_refuses_what_it_cannot_hold():
    _, _, _, cache = _weights(64, 8192 + 512, 64, seed=3)
    x = synth.make_activation(16, 8192 + 512, seed=4, device=DEV)
    with pytest.raises(miori_b200.MioriError, match="8192"):
        miori_b200.gemv_bf16_cache(x, cache, 64)
    with pytest.raises(miori_b200.MioriError):
        miori_b200.gemv_bf16_cache(synth.make_activation(33, 64, seed=1, device=DEV), cache[:64 * 64], 64)


# ---- strided bf16 GEMM (the reference's gemm_naive, shaders/ops.metal:199-251) ---------------

def _bf16_randn(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).to(torch.bfloat16).to(DEV)


@pytest.mark.parametrize("M,N,K,lda,ldb,ldc,why", [
    (64, 16, 2048, 2048, 2048, 16, "gate projection: N=16 against the bf16 weights"),
    (23, 16, 2048, 4096, 2048, 16, "gate on a slice of a wider activation buffer"),
    (32, 4096, 2048, 2048, 2048, 4096, "wide-batch head against a bf16 table"),
    (200, 130, 128, 2048, 128, 136, "attention scores: K=128, ragged M and N, padded C rows"),
    (130, 128, 200, 200, 4096, 2048, "probabilities x V: K not a multiple of 64"),
    (300, 72, 96, 104, 96, 72, "small everything, K below one block"),
])
def test_strided_gemm_tma_path(port, M, N, K, lda, ldb, ldc, why):
    """Row pitches that are multiples of 16 bytes run on the tcgen05 kernels; compared with the
    oracle GEMM on dense copies, and the padding of C must stay untouched."""
    Abig, Bbig = _bf16_randn((M, lda), 1 + M), _bf16_randn((N, ldb), 2 + N)
    A, B = Abig[:, :K], Bbig[:, :K]
    Cbig = torch.full((M, ldc), -7.0, device=DEV)
    miori_b200.gemm_bf16_strided(A, B, out=Cbig[:, :N])
    torch.cuda.synchronize()
    want = port.gemm_bf16(u16(A.contiguous()), u16(B.contiguous()))
    assert_close(Cbig[:, :N].cpu().numpy(), want, rel_max=1e-4, what=why)
    assert bool((Cbig[:, N:] == -7.0).all())
    assert miori_b200.lib.miori_device_error_poll() == 0


@pytest.mark.parametrize("M,N,K,lda,ldb,ldc", [(37, 50, 70, 77, 71, 53), (5, 3, 129, 131, 133, 3)])
def test_strided_gemm_odd_pitches(port, M, N, K, lda, ldb, ldc):
    """Pitches and sizes TMA cannot describe take the plain kernel; same contract."""
    Abig, Bbig = _bf16_randn((M, lda), 3), _bf16_randn((N, ldb), 4)
    A, B = Abig[:, :K], Bbig[:, :K]
    Cbig = torch.full((M, ldc), 9.0, device=DEV)
    miori_b200.gemm_bf16_strided(A, B, out=Cbig[:, :N])
    c16 = miori_b200.gemm_bf16_strided(A, B, flags=miori_b200.OUT_BF16)
    torch.cuda.synchronize()
    want = port.gemm_bf16(u16(A.contiguous()), u16(B.contiguous()))
    assert_close(Cbig[:, :N].cpu().numpy(), want, rel_max=1e-4, what="odd pitches")
    assert bool((Cbig[:, N:] == 9.0).all())
    assert torch.equal(c16, Cbig[:, :N].to(torch.bfloat16))


def test_strided_gemm_equals_cache_gemm_and_rejects_bad_pitch():
    """On a dense cache the strided entry is the cache GEMM, bit for bit."""
    N, K = 3072, 2048
    _, _, _, cache = _weights(N, K, 64, seed=77)
    A = synth.make_activation(48, K, seed=9, device=DEV)
    got = miori_b200.gemm_bf16_strided(A, cache.view(N, K))
    assert torch.equal(got, miori_b200.gemm_bf16_cache(A, cache, N))
    with pytest.raises(miori_b200.MioriError):
        check = miori_b200.check
        check(miori_b200.lib.miori_gemm_bf16_strided(A.data_ptr(), K - 8, cache.data_ptr(), K,
                                                     got.data_ptr(), N, 48, N, K, 0, None))


def test_full_size_packed_prefill_rows_are_independent():
    """M = 131072 token rows (64 prompts x 2048 tokens) against a 2048 x 2048 projection: every
    1024-row block of the big product must equal the M = 1024 product of the same rows bit for
    bit (rows are independent), checked on blocks spread over the whole range, ragged tail
    included; the values themselves are pinned by the M = 1024 tests against the oracle."""
    N, K, M = 2048, 2048, 131072 + 40
    _, _, _, cache = _weights(N, K, 64, seed=55)
    g = torch.Generator(device=DEV).manual_seed(5)
    A = torch.randn((M, K), generator=g, device=DEV).to(torch.bfloat16)
    big = miori_b200.gemm_bf16_cache(A, cache, N, flags=miori_b200.OUT_BF16)
    torch.cuda.synchronize()
    assert bool(torch.isfinite(big.float()).all())
    for r0 in (0, 1024 * 37, 1024 * 64 + 128, 131072 - 1024, 131072 - 984):
        rows = slice(r0, min(r0 + 1024, M))
        small = miori_b200.gemm_bf16_cache(A[rows].contiguous(), cache, N, flags=miori_b200.OUT_BF16)
        assert torch.equal(small, big[rows]), f"rows {r0}.. differ"
    assert miori_b200.lib.miori_device_error_poll() == 0
