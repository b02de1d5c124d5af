"""GPU parity of the GEMV family against the CPU oracle, through the C ABI.

Mirrors the reference's test-gemv4 / test-gemv8 procedure (src/main.cpp:44-87): the
device result is compared with a double-precision dot of dequant*_elem and the bf16
activations.  Tolerances are the ones in conftest.py.
"""
import numpy as np
import pytest
import torch

import miori_b200
from miori_b200 import synth
from conftest import (GOLDEN, TOL_EXACT_PATH, assert_close, closeness, u16, u32)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

OPS = {4: miori_b200.gemv4, 8: miori_b200.gemv8}


def _case(bits, N, K, M, group, seed, kind="randn"):
    q, s, b = synth.make_weight(N, K, bits, group, seed=seed)
    x = synth.ramp_activation(M, K) if kind == "ramp" else synth.make_activation(M, K, seed + 1)
    return q, s, b, x


def _run(bits, q, s, b, x, group, flags=0):
    y = OPS[bits](q.to(DEV), s.to(DEV), b.to(DEV), x.to(DEV), group=group, flags=flags)
    torch.cuda.synchronize()
    return y.float().cpu().numpy()


@pytest.mark.parametrize("path", ["gemv4_n48_k256_m1_ramp", "gemv4_n33_k512_m4_randn",
                                  "gemv8_n40_k256_m1_ramp", "gemv8_n17_k128_m3_randn"])
def test_golden_fixture(path):
    import os
    g = np.load(os.path.join(GOLDEN, path + ".npz"))
    bits = int(g["bits"])
    q = torch.from_numpy(g["q"].view(np.int32))
    s = torch.from_numpy(g["s"].view(np.int16)).view(torch.bfloat16)
    b = torch.from_numpy(g["b"].view(np.int16)).view(torch.bfloat16)
    x = torch.from_numpy(g["x"].view(np.int16)).view(torch.bfloat16)
    y = _run(bits, q, s, b, x, 32)
    assert_close(y, g["y"], rel_max=TOL_EXACT_PATH, what=path)


# the reference model's projection shapes (config/m6.h) and the benchmark's synthetic ones
SHAPES4 = [(2048, 2048), (512, 2048), (16, 2048), (6144, 2048), (7680, 2048), (2048, 7680),
           (8192, 2048), (3072, 2048), (2048, 8192), (1, 32), (17, 64), (130, 96)]


@pytest.mark.parametrize("group", [32, 64])
@pytest.mark.parametrize("N,K", SHAPES4)
def test_gemv4_m1_matches_oracle(port, N, K, group):
    if K % group:
        pytest.skip("K not a multiple of the group")
    q, s, b, x = _case(4, N, K, 1, group, seed=N * 7 + K)
    want = port.gemv(4, u32(q), u16(s), u16(b), u16(x), group)
    got = _run(4, q, s, b, x, group)
    assert_close(got, want, rel_max=TOL_EXACT_PATH, what=f"gemv4 N={N} K={K} g={group}")


@pytest.mark.parametrize("group", [32, 64])
@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8, 16, 31, 32])
def test_gemv4_batched_matches_oracle(port, M, group):
    N, K = 1536, 2048
    q, s, b, x = _case(4, N, K, M, group, seed=100 + M)
    want = port.gemv(4, u32(q), u16(s), u16(b), u16(x), group)
    got = _run(4, q, s, b, x, group)
    tol = TOL_EXACT_PATH if M <= 4 else 1e-2
    assert_close(got, want, rel_max=tol, what=f"gemv4 M={M} g={group}")
    got_exact = _run(4, q, s, b, x, group, flags=miori_b200.GEMV_EXACT)
    assert_close(got_exact, want, rel_max=TOL_EXACT_PATH, what=f"gemv4 exact M={M} g={group}")


@pytest.mark.parametrize("M", [2, 4, 8, 32])
def test_gemv4_batched_long_k(port, M):
    N, K = 256, 8192
    q, s, b, x = _case(4, N, K, M, 64, seed=300 + M)
    want = port.gemv(4, u32(q), u16(s), u16(b), u16(x), 64)
    got = _run(4, q, s, b, x, 64)
    assert_close(got, want, what=f"gemv4 K=8192 M={M}")


def test_rows_do_not_depend_on_m():
    """The reference's gemv4_b gives each row the same value as gemv4 (batch.metal:142-144)."""
    N, K = 512, 2048
    q, s, b, x = _case(4, N, K, 4, 32, seed=77)
    y4 = _run(4, q, s, b, x, 32)
    for m in range(4):
        y1 = _run(4, q, s, b, x[m:m + 1].contiguous(), 32)
        assert np.array_equal(y1[0], y4[m]), f"row {m} differs between M=1 and M=4"
    x8 = synth.make_activation(8, K, seed=78)
    y8 = _run(4, q, s, b, x8, 32)
    y5 = _run(4, q, s, b, x8[:5].contiguous(), 32)
    assert np.array_equal(y5, y8[:5]), "rows differ between M=5 and M=8"


def test_rows_at_group_64_agree_across_m(port):
    """Group 64: M = 1, 2 share one arithmetic order and M = 3, 4 another (chunk-pair columns);
    inside each pair rows are bit-identical, across them they agree to fp32 rounding."""
    N, K = 528, 2048
    q, s, b, x = _case(4, N, K, 4, 64, seed=91)
    y4 = _run(4, q, s, b, x, 64)
    y3 = _run(4, q, s, b, x[:3].contiguous(), 64)
    y2 = _run(4, q, s, b, x[:2].contiguous(), 64)
    y1 = _run(4, q, s, b, x[:1].contiguous(), 64)
    assert np.array_equal(y3, y4[:3])
    assert np.array_equal(y1, y2[:1])
    assert closeness(y2, y4[:2])[0] < TOL_EXACT_PATH
    want = port.gemv(4, u32(q), u16(s), u16(b), u16(x), 64)
    assert_close(y4, want, rel_max=TOL_EXACT_PATH, what="pair columns M=4")
    assert_close(y3, want[:3], rel_max=TOL_EXACT_PATH, what="pair columns M=3")


@pytest.mark.parametrize("flags", [0x400, 0x800])
@pytest.mark.parametrize("bits,M", [(4, 1), (4, 3), (4, 8), (4, 32), (8, 2)])
def test_every_kernel_family_matches_oracle(port, bits, M, flags):
    """The shape-agnostic SIMT kernel (0x400) and the register-streaming tensor-core kernel
    (0x800) are held to the same oracle as the default bulk-copy kernel."""
    N, K = 528, 2048
    q, s, b, x = _case(bits, N, K, M, 64, seed=500 + M)
    want = port.gemv(bits, u32(q), u16(s), u16(b), u16(x), 64)
    got = _run(bits, q, s, b, x, 64, flags=flags)
    tol = TOL_EXACT_PATH if (M <= 4 or flags == 0x400) else 1e-2
    assert_close(got, want, rel_max=tol, what=f"gemv{bits} M={M} flags={flags:#x}")


@pytest.mark.parametrize("group", [32, 64])
@pytest.mark.parametrize("N,K,M", [(4096, 2048, 1), (1000, 2048, 1), (129, 256, 4), (640, 2048, 8),
                                   (512, 2048, 32)])
def test_gemv8_matches_oracle(port, N, K, M, group):
    q, s, b, x = _case(8, N, K, M, group, seed=N + K + M)
    want = port.gemv(8, u32(q), u16(s), u16(b), u16(x), group)
    got = _run(8, q, s, b, x, group)
    tol = TOL_EXACT_PATH if M <= 4 else 1e-2
    assert_close(got, want, rel_max=tol, what=f"gemv8 N={N} K={K} M={M} g={group}")


def test_gemv8_lm_head_sampled_rows(port):
    """The reference checks every 997th row of the 128000-row head (src/main.cpp:73)."""
    N, K = 128000, 2048
    q, s, b = synth.make_weight(N, K, 8, 32, seed=5, device=DEV)
    x = synth.ramp_activation(1, K)
    y = OPS[8](q, s, b, x.to(DEV), group=32).cpu().numpy()
    rows = np.arange(0, N, 997)
    qn, sn, bn = u32(q[rows]), u16(s[rows]), u16(b[rows])
    want = port.gemv(8, qn, sn, bn, u16(x), 32)
    assert_close(y[:, rows], want, rel_max=TOL_EXACT_PATH, what="gemv8 head")
    err = np.abs(y[0, rows] - want[0])
    max_rel = (err / (np.abs(want[0]) + 1e-6)).max()
    print(f"gemv8 head: checked {len(rows)} rows max_abs={err.max():.3g} max_rel={max_rel:.3g}")


def test_bf16_output_is_rounded_fp32_output():
    N, K = 1024, 2048
    q, s, b, x = _case(4, N, K, 2, 64, seed=9)
    y32 = OPS[4](q.to(DEV), s.to(DEV), b.to(DEV), x.to(DEV), group=64)
    y16 = OPS[4](q.to(DEV), s.to(DEV), b.to(DEV), x.to(DEV), group=64, flags=miori_b200.OUT_BF16)
    assert y16.dtype == torch.bfloat16
    assert torch.equal(y16, y32.to(torch.bfloat16))


def test_pdl_launch_gives_same_result():
    N, K = 2048, 2048
    q, s, b, x = _case(4, N, K, 1, 64, seed=10)
    args = (q.to(DEV), s.to(DEV), b.to(DEV), x.to(DEV))
    y0 = OPS[4](*args, group=64)
    ys = [OPS[4](*args, group=64, flags=miori_b200.LAUNCH_PDL) for _ in range(4)]
    torch.cuda.synchronize()
    for y in ys:
        assert torch.equal(y, y0)


def test_output_guard_bands_untouched():
    """Nothing is written outside y[M][N] (odd N, M not a multiple of the row tile)."""
    N, K, M = 1037, 2048, 3
    q, s, b, x = _case(4, N, K, M, 32, seed=12)
    buf = torch.full((M * N + 512,), 12345.0, device=DEV)
    y = buf[256:256 + M * N].view(M, N)
    OPS[4](q.to(DEV), s.to(DEV), b.to(DEV), x.to(DEV), group=32, out=y)
    torch.cuda.synchronize()
    assert (buf[:256] == 12345.0).all() and (buf[256 + M * N:] == 12345.0).all()
    assert not (y == 12345.0).any()


def test_runtime_buffers_and_copies(port):
    """The device runtime path a C++ host uses: shared buffers, begin/submit, copies."""
    import ctypes as C
    from miori_b200._lib import check, lib
    N, K = 256, 512
    q, s, b, x = _case(4, N, K, 1, 32, seed=13)
    dev = C.c_void_p()
    check(lib.miori_device_open(0, C.byref(dev)))
    bufs = []
    try:
        def shared(arr):
            h = C.c_void_p()
            check(lib.miori_buffer_alloc(dev, arr.nbytes, 1, C.byref(h)))
            bufs.append(h)
            assert lib.miori_buffer_length(h) == arr.nbytes
            C.memmove(lib.miori_buffer_contents(h), arr.ctypes.data, arr.nbytes)
            return h
        hq, hs, hb, hx = shared(u32(q)), shared(u16(s)), shared(u16(b)), shared(u16(x))
        hy = C.c_void_p()
        check(lib.miori_buffer_alloc(dev, N * 4, 1, C.byref(hy)))
        bufs.append(hy)
        priv = C.c_void_p()
        check(lib.miori_buffer_alloc(dev, 4096, 0, C.byref(priv)))
        bufs.append(priv)
        assert lib.miori_buffer_contents(priv) is None
        check(lib.miori_begin(dev))
        p = lib.miori_buffer_device_ptr
        check(lib.miori_gemv4(p(hq), p(hs), p(hb), p(hx), p(hy), N, K, 1, 32, 0,
                              lib.miori_device_stream(dev)))
        check(lib.miori_submit(dev, 1))
        y = np.ctypeslib.as_array(C.cast(lib.miori_buffer_contents(hy), C.POINTER(C.c_float)), (N,))
        want = port.gemv(4, u32(q), u16(s), u16(b), u16(x), 32)
        assert_close(y, want[0], rel_max=TOL_EXACT_PATH, what="runtime path")
        assert lib.miori_device_error_poll() == 0
    finally:
        for h in bufs:
            lib.miori_buffer_free(h)
        lib.miori_device_close(dev)


def test_gemv8_activation_range(port):
    """8-bit codes meet x as fp16 scaled by a power of two taken from the largest |x|: scaling x
    by a power of two must scale y exactly, an outlier must not cost the other terms their
    precision, rows keep their own scale, and zeros must stay zeros."""
    N, K = 1024, 2048
    q, s, b, x = _case(8, N, K, 2, 64, seed=808)
    y = _run(8, q, s, b, x, 64)
    for k in (20, -30, 100):
        xs = (x.float() * 2.0 ** k).to(torch.bfloat16)
        ys = _run(8, q, s, b, xs, 64)
        assert np.array_equal(ys, y * np.float32(2.0 ** k)), f"x * 2^{k}"
    xo = x.clone()
    xo[0, 7] = 3.0e4   # one huge activation in row 0
    xo[1, :] = (xo[1, :].float() * 2.0 ** -40).to(torch.bfloat16)  # a very quiet row beside it
    want = port.gemv(8, u32(q), u16(s), u16(b), u16(xo), 64)
    got = _run(8, q, s, b, xo, 64)
    assert_close(got[0], want[0], rel_max=TOL_EXACT_PATH, what="row with an outlier")
    assert_close(got[1], want[1], rel_max=TOL_EXACT_PATH, what="quiet row next to the outlier")
    alone = _run(8, q, s, b, xo[1:2].contiguous(), 64)
    assert np.array_equal(alone[0], got[1]), "a row's value depends on its neighbour"
    assert not _run(8, q, s, b, torch.zeros_like(x), 64).any()


# ---- the tcgen05 kernel (integer tensor cores), forced with the private tuning flag ----------
UMMA = 0x100000          # MIORI_TUNE_GEMV_UMMA (csrc/tune.h)
SPLIT_SHIFT = 16         # MIORI_TUNE_UMMA_SPLIT_SHIFT


@pytest.mark.parametrize("group", [32, 64])
@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("bits", [4, 8])
def test_tcgen05_gemv_matches_oracle_every_m(port, bits, M, group):
    """fp32 dequantization with an exact integer inner sum: the tight tolerance holds for every M."""
    N, K = 1537, 2048   # not a multiple of the 128-row tile
    q, s, b, x = _case(bits, N, K, M, group, seed=700 + M + bits)
    want = port.gemv(bits, u32(q), u16(s), u16(b), u16(x), group)
    got = _run(bits, q, s, b, x, group, flags=UMMA)
    assert_close(got, want, rel_max=TOL_EXACT_PATH, what=f"tcgen05 gemv{bits} M={M} g={group}")


@pytest.mark.parametrize("N,K,group", [(2048, 2048, 64), (16, 2048, 32), (512, 2048, 32), (6144, 2048, 32),
                                       (2048, 7680, 32), (2048, 7680, 64), (3072, 2048, 64), (2048, 8192, 64),
                                       (130, 256, 32), (8192, 2048, 64)])
def test_tcgen05_gemv4_shapes(port, N, K, group):
    """The reference model's projection shapes (config/m6.h) and the synthetic stack's, M = 1 and 4."""
    q, s, b, x = _case(4, N, K, 4, group, seed=N + K)
    want = port.gemv(4, u32(q), u16(s), u16(b), u16(x), group)
    got4 = _run(4, q, s, b, x, group, flags=UMMA)
    got1 = _run(4, q, s, b, x[:1].contiguous(), group, flags=UMMA)
    assert_close(got4, want, rel_max=TOL_EXACT_PATH, what=f"tcgen05 gemv4 N={N} K={K} g={group} M=4")
    assert np.array_equal(got1[0], got4[0]), "row 0 differs between M=1 and M=4"


@pytest.mark.parametrize("split", [1, 2, 4, 8])
@pytest.mark.parametrize("bits,M", [(4, 1), (4, 8), (8, 3), (4, 32)])
def test_tcgen05_gemv_k_split_over_a_cluster(port, bits, M, split):
    """K split over the CTAs of a cluster (partials meet through distributed shared memory)."""
    N, K = 640, 2048
    q, s, b, x = _case(bits, N, K, M, 64, seed=900 + split + M)
    want = port.gemv(bits, u32(q), u16(s), u16(b), u16(x), 64)
    got = _run(bits, q, s, b, x, 64, flags=UMMA | (split << SPLIT_SHIFT))
    assert_close(got, want, rel_max=TOL_EXACT_PATH, what=f"tcgen05 gemv{bits} M={M} split={split}")
    again = _run(bits, q, s, b, x, 64, flags=UMMA | (split << SPLIT_SHIFT))
    assert np.array_equal(got, again), "the split sum is not reproducible"


def test_tcgen05_rows_do_not_depend_on_m():
    """Inside a class of M (<= 8, <= 16, <= 32) a row's value is bit-identical whatever the batch."""
    N, K = 1024, 2048
    q, s, b = synth.make_weight(N, K, 4, 64, seed=31)
    x = synth.make_activation(32, K, seed=32)
    for lo, hi in ((1, 8), (9, 16), (17, 32)):
        full = _run(4, q, s, b, x[:hi].contiguous(), 64, flags=UMMA)
        part = _run(4, q, s, b, x[:lo].contiguous(), 64, flags=UMMA)
        assert np.array_equal(part, full[:lo]), f"rows differ between M={lo} and M={hi}"


def test_tcgen05_activation_range(port):
    """x is rounded to fixed point against its row's largest magnitude: a power-of-two factor on x
    scales y exactly, an outlier in one row costs neither that row nor its neighbour the tight
    tolerance, and zeros stay zeros."""
    N, K = 1024, 2048
    q, s, b, x = _case(4, N, K, 2, 64, seed=808)
    y = _run(4, q, s, b, x, 64, flags=UMMA)
    for k in (20, -30, 90):
        xs = (x.float() * 2.0 ** k).to(torch.bfloat16)
        ys = _run(4, q, s, b, xs, 64, flags=UMMA)
        assert np.array_equal(ys, y * np.float32(2.0 ** k)), f"x * 2^{k}"
    xo = x.clone()
    xo[0, 7] = 3.0e4
    xo[1, :] = (xo[1, :].float() * 2.0 ** -40).to(torch.bfloat16)
    want = port.gemv(4, u32(q), u16(s), u16(b), u16(xo), 64)
    got = _run(4, q, s, b, xo, 64, flags=UMMA)
    assert_close(got[0], want[0], rel_max=TOL_EXACT_PATH, what="row with an outlier")
    assert_close(got[1], want[1], rel_max=TOL_EXACT_PATH, what="quiet row next to the outlier")
    assert not _run(4, q, s, b, torch.zeros_like(x), 64, flags=UMMA).any()


def test_gemv8_batched_default_path_is_exact(port):
    """Three rows and more of 8-bit weights run on the tcgen05 kernel by default (the reference's
    gemv8_b and the four-row head of packed prefill, src/batch.cpp:596-600): tight tolerance."""
    N, K = 4096, 2048
    for M in (3, 4, 8, 32):
        q, s, b, x = _case(8, N, K, M, 32, seed=60 + M)
        want = port.gemv(8, u32(q), u16(s), u16(b), u16(x), 32)
        assert_close(_run(8, q, s, b, x, 32), want, rel_max=TOL_EXACT_PATH, what=f"gemv8 M={M}")


@pytest.mark.parametrize("flags", [0, UMMA])
def test_config1_head_exact_shape(port, flags):
    """The 8-bit head at its benchmark shape: N = 131072, K = 2048, group 64, every 997th row."""
    N, K = 131072, 2048
    q, s, b = synth.make_weight(N, K, 8, 64, seed=15, device=DEV)
    x = synth.make_activation(1, K, seed=16)
    y = OPS[8](q, s, b, x.to(DEV), group=64, flags=flags).cpu().numpy()
    rows = np.arange(0, N, 997)
    want = port.gemv(8, u32(q[rows]), u16(s[rows]), u16(b[rows]), u16(x), 64)
    assert_close(y[:, rows], want, rel_max=TOL_EXACT_PATH, what="config 1 head")


@pytest.mark.parametrize("M", [1, 2, 4, 8, 16, 32])
@pytest.mark.parametrize("N,K", [(3072, 2048), (2048, 2048), (16384, 2048), (2048, 8192)])
def test_config2_grid_default_dispatch(port, N, K, M):
    """Every projection shape of the synthetic decode stack at every M of the sweep, group 64,
    through the default dispatch (whichever kernel it selects), on every 61st row."""
    q, s, b = synth.make_weight(N, K, 4, 64, seed=N + K + M, device=DEV)
    x = synth.make_activation(M, K, seed=M)
    y = OPS[4](q, s, b, x.to(DEV), group=64).cpu().numpy()
    rows = np.arange(0, N, 61)
    want = port.gemv(4, u32(q[rows]), u16(s[rows]), u16(b[rows]), u16(x), 64)
    tol = TOL_EXACT_PATH if M <= 4 else 1e-2
    assert_close(y[:, rows], want, rel_max=tol, what=f"config 2 N={N} K={K} M={M}")


@pytest.mark.parametrize("M", [1, 4])
def test_long_stream_gemv4_default_dispatch(port, M):
    """A 151 MB matrix of 4-bit weights (N = 131072): the default dispatch takes the tcgen05 kernel
    with two CTAs per SM there; every 997th row against the oracle, tight tolerance."""
    N, K = 131072, 2048
    q, s, b = synth.make_weight(N, K, 4, 64, seed=21, device=DEV)
    x = synth.make_activation(M, K, seed=22)
    y = OPS[4](q, s, b, x.to(DEV), group=64).cpu().numpy()
    again = OPS[4](q, s, b, x.to(DEV), group=64).cpu().numpy()
    rows = np.arange(0, N, 997)
    want = port.gemv(4, u32(q[rows]), u16(s[rows]), u16(b[rows]), u16(x), 64)
    assert_close(y[:, rows], want, rel_max=TOL_EXACT_PATH, what=f"long stream M={M}")
    assert np.array_equal(y, again)
