"""The steps either side of a projection (RMSNorm, SiLU x up, post-norm + residual), the 8-bit
embedding gather, the arg-max, and the GEMVs that take those steps in (the RMSNorm in the activation
staging, SiLU x up and the post-norm as epilogues), against the CPU restatements of the reference's
shaders (oracle/miori_oracle.c)."""
import numpy as np
import pytest
import torch

import miori_b200
from miori_b200 import synth
from conftest import TOL_EXACT_PATH, assert_close, u16, u32

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def bf16_ulps(a_bits, b_bits):
    """Distance in bf16 steps between two arrays of bf16 bit patterns (same-sign finite values)."""
    def key(v):
        v = v.astype(np.int32)
        return np.where(v & 0x8000, 0x8000 - (v & 0x7FFF), v + 0x8000)
    return np.abs(key(a_bits) - key(b_bits))


@pytest.mark.parametrize("rows,n", [(1, 2048), (4, 2048), (3, 7680), (32, 1000)])
def test_rmsnorm(port, rows, n):
    g = torch.Generator().manual_seed(rows + n)
    x = torch.randn((rows, n), generator=g) * 3.0
    w = (torch.randn(n, generator=g) * 0.2 + 1.0).to(torch.bfloat16)
    y = miori_b200.rmsnorm(x.to(DEV), w.to(DEV), 1e-5)
    want = port.rmsnorm(x.numpy(), u16(w), 1e-5)
    d = bf16_ulps(u16(y), want)
    assert d.max() <= 1, f"rmsnorm differs by {d.max()} bf16 steps"
    assert (d != 0).mean() < 0.02   # only where fp32 rounding of the sum of squares tips a rounding


def test_silu_mul(port):
    g = torch.Generator().manual_seed(3)
    gate, up = torch.randn(7680 * 3, generator=g) * 4.0, torch.randn(7680 * 3, generator=g)
    gate[:4] = torch.tensor([0.0, -100.0, 100.0, -0.0])
    out = miori_b200.silu_mul(gate.to(DEV), up.to(DEV))
    d = bf16_ulps(u16(out), port.silu_mul(gate.numpy(), up.numpy()))
    assert d.max() <= 1 and (d != 0).mean() < 0.01


@pytest.mark.parametrize("rows,n", [(1, 2048), (5, 2048)])
def test_post_norm_add(port, rows, n):
    g = torch.Generator().manual_seed(rows)
    x, src = torch.randn((rows, n), generator=g), torch.randn((rows, n), generator=g) * 2.0
    w = (torch.randn(n, generator=g) * 0.1 + 1.0).to(torch.bfloat16)
    out = miori_b200.post_norm_add(x.to(DEV), src.to(DEV), w.to(DEV), 1e-5)
    want = port.post_norm_add(x.numpy(), src.numpy(), u16(w), 1e-5)
    assert_close(out.cpu().numpy(), want, rel_max=1e-6, what="post_norm_add")


@pytest.mark.parametrize("group", [32, 64])
def test_embed8_bit_exact(port, group):
    rows, K = 1000, 2048
    q, s, b = synth.make_weight(rows, K, 8, group, seed=41)
    tokens = torch.tensor([0, 999, 17, 17, 512, 3], dtype=torch.int32)
    out = miori_b200.embed8(q.to(DEV), s.to(DEV), b.to(DEV), tokens.to(DEV), group=group)
    want = port.embed8(u32(q), u16(s), u16(b), tokens.numpy().astype(np.uint32), group)
    assert np.array_equal(u16(out), want)
    # the same rows as the cache build produces them
    full = miori_b200.dequant8_rowmajor(q.to(DEV), s.to(DEV), b.to(DEV), group=group)
    assert torch.equal(out, full[tokens.long().to(DEV)])
    # an id outside the table leaves its row as it was
    guard = torch.full((2, K), 7.0, dtype=torch.bfloat16, device=DEV)
    miori_b200.embed8(q.to(DEV), s.to(DEV), b.to(DEV), torch.tensor([5, 1000], dtype=torch.int32, device=DEV),
                      group=group, out=guard)
    assert (guard[1] == 7.0).all() and torch.equal(guard[0], full[5])


def test_argmax_ties_go_to_the_lowest_index():
    g = torch.Generator().manual_seed(9)
    v = torch.randn(131072, generator=g)
    idx, val = miori_b200.argmax(v.to(DEV))
    assert int(idx.item()) == int(np.argmax(v.numpy())) and float(val.item()) == float(v.max())
    v[1000] = v[77777] = v.max() + 1.0
    idx, _ = miori_b200.argmax(v.to(DEV))
    assert int(idx.item()) == 1000
    vb = v.to(torch.bfloat16)
    idx, val = miori_b200.argmax(vb.to(DEV))
    assert int(idx.item()) == int(np.argmax(vb.float().numpy())) and float(val.item()) == float(vb.float().max())


@pytest.mark.parametrize("n", [1, 7, 33, 8191, 8192, 8200, 20001, 65536, 131077])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_argmax_sizes_and_alignment(n, dtype):
    """Every cluster size (1, 2, 4, 8 CTAs), ragged tails, a maximum in the last element, and a
    vector that does not start on a 16-byte boundary (scalar loads then)."""
    g = torch.Generator().manual_seed(n)
    v = torch.randn(n + 3, generator=g).to(dtype)
    for shift in (0, 1):   # 1: the view starts 2 or 4 bytes into the allocation
        w = v[shift:shift + n].clone()
        for spot in (None, n - 1, 0, n // 2):
            if spot is not None:
                w[spot] = 50.0 + (spot % 7)
            dv = v.to(DEV)
            dv[shift:shift + n] = w.to(DEV)
            idx, val = miori_b200.argmax(dv[shift:shift + n])
            want = int(np.argmax(w.float().numpy()))
            assert int(idx.item()) == want and float(val.item()) == float(w.float()[want]), (n, dtype, shift, spot)


@pytest.mark.parametrize("bits,N,K,M,group", [(4, 2048, 2048, 1, 64), (4, 3072, 2048, 4, 32), (4, 640, 2048, 8, 64),
                                              (8, 1024, 2048, 2, 64), (4, 2048, 8192, 1, 64), (4, 1536, 2048, 32, 64),
                                              (4, 16384, 2048, 2, 64), (4, 1000, 4096, 3, 64), (4, 48, 512, 3, 32)])
@pytest.mark.parametrize("force", [0, 0x100000, 0x1000], ids=["default", "tcgen05", "mma.sync"])
def test_gemv_with_fused_rmsnorm(port, bits, N, K, M, group, force):
    """y = W * bf16(rmsnorm(x)): the fused kernels (by default the TMA + mma.sync one for 4-bit weights,
    up to four rows and K <= 2048, the tcgen05 one otherwise; either when forced, where it applies)
    against the oracle's norm followed by its GEMV, and against this library's own unfused pair."""
    q, s, b = synth.make_weight(N, K, bits, group, seed=N + K + M)
    g = torch.Generator().manual_seed(M)
    x = torch.randn((M, K), generator=g) * 2.5
    w = (torch.randn(K, generator=g) * 0.2 + 1.0).to(torch.bfloat16)
    fused = (miori_b200.gemv4_rmsnorm if bits == 4 else miori_b200.gemv8_rmsnorm)(
        q.to(DEV), s.to(DEV), b.to(DEV), x.to(DEV), w.to(DEV), 1e-5, group=group, flags=force).cpu().numpy()
    xn = port.rmsnorm(x.numpy(), u16(w), 1e-5)
    want = port.gemv(bits, u32(q), u16(s), u16(b), xn, group)
    # a bf16 rounding of a normalised activation may tip differently than in the oracle (fp32 order
    # of the sum of squares): each such flip moves one term by 2^-8 of its size
    assert_close(fused, want, rel_max=1e-3, what=f"fused norm gemv{bits} M={M}")
    xn_dev = miori_b200.rmsnorm(x.to(DEV), w.to(DEV), 1e-5)
    unfused = (miori_b200.gemv4 if bits == 4 else miori_b200.gemv8)(
        q.to(DEV), s.to(DEV), b.to(DEV), xn_dev, group=group, flags=0x100000).cpu().numpy()
    assert_close(fused, unfused, rel_max=1e-3, what="fused vs unfused")


TILED = 0x2000    # tuning flag: tiled TMA even where one slab of K fits the linear copies
MMASYNC = 0x1000  # tuning flag: keep the unfused GEMV on the kernel the fused entry runs on


@pytest.mark.parametrize("N,K,M,group,flags", [
    (16384, 2048, 1, 64, 0), (16384, 2048, 2, 64, 0), (12288, 2048, 3, 64, 0), (4096, 2048, 4, 32, 0),
    (2048, 2048, 8, 64, 0), (3072, 2048, 16, 64, 0), (1024, 1024, 16, 32, 0), (4096, 4096, 1, 64, 0),
    (512, 8192, 2, 64, 0), (2048, 2048, 1, 64, TILED), (1024, 2048, 6, 32, TILED), (4096, 1024, 5, 32, 0),
    (32, 2048, 1, 64, 0), (16, 512, 7, 64, 0), (6000 * 2, 1536, 4, 64, 0)])
def test_gemv_with_silu_epilogue(port, N, K, M, group, flags):
    """bf16(silu(gate) * up) out of the fused gate + up projection: bit for bit the unfused pair of
    this library, and the oracle's GEMV followed by its silu_mul within one bf16 step (M <= 4, the
    fp32-dequantization kernels) resp. the batched GEMV's tolerance."""
    q, s, b = synth.make_weight(N, K, 4, group, seed=N + K + M)
    x = synth.make_activation(M, K, seed=M)
    dq, ds, db, dx = q.to(DEV), s.to(DEV), b.to(DEV), x.to(DEV)
    fused = miori_b200.gemv4_silu(dq, ds, db, dx, group=group, flags=flags)
    assert fused.shape == (M, N // 2) and fused.dtype == torch.bfloat16
    y = miori_b200.gemv4(dq, ds, db, dx, group=group, flags=flags | MMASYNC)
    h = N // 2
    unfused = miori_b200.silu_mul(y[:, :h].contiguous(), y[:, h:].contiguous())
    assert torch.equal(fused.view(torch.int16), unfused.view(torch.int16)), "fused and unfused differ"
    want_y = port.gemv(4, u32(q), u16(s), u16(b), u16(x), group)
    want = port.silu_mul(np.ascontiguousarray(want_y[:, :h]), np.ascontiguousarray(want_y[:, h:]))
    got = fused.float().cpu().numpy()
    ref = (want.astype(np.uint32) << 16).view(np.float32).reshape(got.shape)
    if M <= 4:
        # one bf16 step plus what the GEMV's fp32 sums (within 2e-5 of the largest output) may move a
        # small product by; nearly all outputs equal bit for bit
        assert (np.abs(got - ref) <= np.abs(ref) * 2.0 ** -7 + 1e-3).all()
        assert (u16(fused).reshape(-1) != want.reshape(-1)).mean() < 0.01
    else:
        assert_close(got, ref, rel_max=2e-2, what=f"gated gemv4 M={M}")
    assert miori_b200.lib.miori_device_error_poll() == 0


def test_gemv_with_silu_epilogue_refuses_what_it_cannot_take():
    q, s, b = synth.make_weight(48, 2048, 4, 64, seed=1)
    x = synth.make_activation(1, 2048, seed=1).to(DEV)
    with pytest.raises(miori_b200.MioriError, match="multiple of 16"):
        miori_b200.gemv4_silu(q[:40].contiguous().to(DEV), s[:40].contiguous().to(DEV), b[:40].contiguous().to(DEV), x,
                              group=64)
    # scale rows of 96 / 32 = 3 groups have no 16-byte pitch: outside the TMA kernel's range
    q2, s2, b2 = synth.make_weight(32, 96, 4, 32, seed=2)
    x2 = synth.make_activation(1, 96, seed=2).to(DEV)
    with pytest.raises(miori_b200.MioriError, match="outside the fused kernel's range"):
        miori_b200.gemv4_silu(q2.to(DEV), s2.to(DEV), b2.to(DEV), x2, group=32)
    # more than 16 activation rows do not fit the kernel's staging area
    x3 = synth.make_activation(17, 2048, seed=3).to(DEV)
    with pytest.raises(miori_b200.MioriError, match="outside 1..16"):
        miori_b200.gemv4_silu(q.to(DEV), s.to(DEV), b.to(DEV), x3, group=64)


@pytest.mark.parametrize("N,K,M,group,flags", [
    (2048, 2048, 1, 64, 0), (2048, 8192, 1, 64, 0), (2048, 2048, 2, 32, 0), (2048, 2048, 3, 64, 0),
    (2048, 8192, 4, 64, 0), (1000, 2048, 4, 32, 0), (2048, 2048, 1, 64, TILED), (16, 512, 2, 64, 0),
    (5120, 4096, 1, 64, 0)])
def test_gemv_with_post_norm_add_epilogue(port, N, K, M, group, flags):
    """residual + v * rsqrt(mean(v^2) + eps) * gamma with v the GEMV's output row: bit for bit the
    unfused pair of this library, close to the oracle's pair, repeatable, and the arrival counter is
    left at zero."""
    q, s, b = synth.make_weight(N, K, 4, group, seed=N + K + M)
    x = synth.make_activation(M, K, seed=M)
    g = torch.Generator().manual_seed(N + M)
    res = torch.randn((M, N), generator=g)
    w = (torch.randn(N, generator=g) * 0.1 + 1.0).to(torch.bfloat16)
    dq, ds, db, dx, dres, dw = q.to(DEV), s.to(DEV), b.to(DEV), x.to(DEV), res.to(DEV), w.to(DEV)
    counter = torch.zeros(1, dtype=torch.int32, device=DEV)
    fused = miori_b200.gemv4_post_norm_add(dq, ds, db, dx, dres, dw, 1e-5, counter, group=group, flags=flags)
    again = miori_b200.gemv4_post_norm_add(dq, ds, db, dx, dres, dw, 1e-5, counter, group=group, flags=flags)
    assert int(counter.item()) == 0
    v = miori_b200.gemv4(dq, ds, db, dx, group=group, flags=flags | MMASYNC)
    unfused = miori_b200.post_norm_add(dres, v, dw, 1e-5)
    assert torch.equal(fused, unfused), "fused and unfused differ"
    assert torch.equal(fused, again), "second launch differs"
    want_v = port.gemv(4, u32(q), u16(s), u16(b), u16(x), group)
    want = port.post_norm_add(res.numpy(), want_v.astype(np.float32), u16(w), 1e-5)
    assert_close(fused.cpu().numpy(), want, rel_max=1e-4, what=f"post-norm gemv4 M={M}")
    assert miori_b200.lib.miori_device_error_poll() == 0


def test_gemv_with_post_norm_add_epilogue_refuses_what_it_cannot_take():
    q, s, b = synth.make_weight(64, 2048, 4, 64, seed=1)
    x = synth.make_activation(5, 2048, seed=1).to(DEV)
    res = torch.zeros((5, 64), device=DEV)
    w = torch.ones(64, dtype=torch.bfloat16, device=DEV)
    counter = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(miori_b200.MioriError, match="outside 1..4"):
        miori_b200.gemv4_post_norm_add(q.to(DEV), s.to(DEV), b.to(DEV), x, res, w, 1e-5, counter, group=64)
    with pytest.raises(miori_b200.MioriError, match="must not be the residual"):
        miori_b200.gemv4_post_norm_add(q.to(DEV), s.to(DEV), b.to(DEV), x[:1].contiguous(), res[:1], w, 1e-5,
                                       counter, group=64, out=res[:1])


@pytest.mark.parametrize("N,K,M,group,flags", [(16384, 2048, 1, 64, 0), (4096, 2048, 2, 32, 0), (12288, 2048, 3, 64, 0),
                                               (2048, 4096, 4, 64, 0), (1024, 2048, 1, 64, TILED), (32, 512, 4, 64, 0)])
def test_gate_up_projection_with_both_neighbours(port, N, K, M, group, flags):
    """rmsnorm, w1, w3 and silu_mul in one launch, against this library's own chain (norm kernel, then
    the gated GEMV) and against the oracle's."""
    q, s, b = synth.make_weight(N, K, 4, group, seed=N + K + M)
    g = torch.Generator().manual_seed(M + 11)
    x = torch.randn((M, K), generator=g) * 1.5
    w = (torch.randn(K, generator=g) * 0.2 + 1.0).to(torch.bfloat16)
    dq, ds, db, dx, dw = q.to(DEV), s.to(DEV), b.to(DEV), x.to(DEV), w.to(DEV)
    fused = miori_b200.gemv4_rmsnorm_silu(dq, ds, db, dx, dw, 1e-5, group=group, flags=flags)
    assert fused.shape == (M, N // 2) and fused.dtype == torch.bfloat16
    chain = miori_b200.gemv4_silu(dq, ds, db, miori_b200.rmsnorm(dx, dw, 1e-5), group=group, flags=flags)
    got = fused.float().cpu().numpy()
    # a bf16 rounding of a normalised activation may tip differently (fp32 order of the sum of squares)
    assert_close(got, chain.float().cpu().numpy(), rel_max=1e-2, what="one launch vs norm kernel + gated GEMV")
    xn = port.rmsnorm(x.numpy(), u16(w), 1e-5)
    want_y = port.gemv(4, u32(q), u16(s), u16(b), xn, group)
    h = N // 2
    want = port.silu_mul(np.ascontiguousarray(want_y[:, :h]), np.ascontiguousarray(want_y[:, h:]))
    ref = (want.astype(np.uint32) << 16).view(np.float32).reshape(got.shape)
    assert_close(got, ref, rel_max=1e-2, what=f"norm + gated gemv4 M={M}")
    assert miori_b200.lib.miori_device_error_poll() == 0
