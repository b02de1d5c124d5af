"""The C++ operator shim (miori::Metal, miori::Weights, miori::gemv4 ... gemm_mpp32 with the
reference's signatures) driven like the reference's own test commands, checked against the
CPU oracle.  Group size is the reference's 32, so oracle/_ref (the reference header itself)
is the checker when it was built."""
import ctypes as C
import os

import numpy as np
import pytest

from miori_b200 import synth
from conftest import TOL_EXACT_PATH, assert_close, u16, u32

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
SHIM = os.path.join(HERE, "..", "miori_b200", "libmiori_shim.so")


@pytest.fixture(scope="module")
def shim():
    lib = C.CDLL(SHIM)
    lib.miori_shim_last_error.restype = C.c_char_p
    p, u = C.c_void_p, C.c_uint32
    lib.miori_shim_test_gemv.argtypes = [C.c_int, p, p, p, p, p, u, u, u]
    lib.miori_shim_test_prefill.argtypes = [p, p, p, p, p, p, u, u, u]
    lib.miori_shim_test_naive.argtypes = [p, p, p, u, u, u, u, u, u]
    return lib


@pytest.mark.parametrize("bits,N,K,B", [(4, 2048, 2048, 1), (4, 512, 2048, 4), (4, 16, 2048, 1),
                                        (4, 2048, 7680, 2), (8, 4000, 2048, 1), (8, 1024, 2048, 4),
                                        (4, 1024, 2048, 32)])
def test_gemv_through_operator_api(shim, port, ref, bits, N, K, B):
    q, s, b = synth.make_weight(N, K, bits, 32, seed=bits * 1000 + N + B)
    x = synth.ramp_activation(B, K)  # the reference test's x (src/main.cpp:28)
    qn, sn, bn, xn = u32(q), u16(s), u16(b), u16(x)
    y = np.zeros((B, N), np.float32)
    rc = shim.miori_shim_test_gemv(bits, qn.ctypes.data, sn.ctypes.data, bn.ctypes.data,
                                   xn.ctypes.data, y.ctypes.data, N, K, B)
    assert rc == 0, shim.miori_shim_last_error()
    want = ref.gemv(bits, qn, sn, bn, xn) if ref is not None else port.gemv(bits, qn, sn, bn, xn, 32)
    assert_close(y, want, rel_max=TOL_EXACT_PATH if B <= 4 else 1e-2, what=f"shim gemv{bits} B={B}")
    # the reference's own report format (src/main.cpp:80-86)
    err = np.abs(y - want)
    print(f"gemv{bits} N={N} K={K} B={B}: max_abs={err.max():.3g} "
          f"max_rel={(err / (np.abs(want) + 1e-6)).max():.3g}")


def test_prefill_through_operator_api(shim, port):
    """dequant_tile at a cache offset, then gemm_mpp32 and gemm_mpp on 23 rows: both equal the
    oracle product and each other bit for bit (the reference's test-mpp-tile)."""
    M, N, K = 23, 6144, 2048
    q, s, b = synth.make_weight(N, K, 4, 32, seed=77)
    A = synth.ramp_activation(M, K)
    qn, sn, bn, An = u32(q), u16(s), u16(b), u16(A)
    c32, c64 = np.zeros((M, N), np.float32), np.zeros((M, N), np.float32)
    rc = shim.miori_shim_test_prefill(qn.ctypes.data, sn.ctypes.data, bn.ctypes.data, An.ctypes.data,
                                      c32.ctypes.data, c64.ctypes.data, M, N, K)
    assert rc == 0, shim.miori_shim_last_error()
    assert np.array_equal(c32, c64)
    want = port.gemm_bf16(An, port.dequant_rowmajor(4, qn, sn, bn, 32))
    assert_close(c64, want, rel_max=1e-4, what="shim prefill")


@pytest.mark.parametrize("M,N,K,lda,ldb,ldc", [(40, 16, 2048, 2048, 2048, 16), (130, 128, 200, 208, 4096, 2048),
                                               (37, 50, 70, 77, 71, 53)])
def test_gemm_naive_through_operator_api(shim, port, M, N, K, lda, ldb, ldc):
    """gemm_naive with row pitches and byte offsets (the gate projection, the probabilities x V
    product, and a shape with odd pitches that takes the plain kernel)."""
    import torch
    g = torch.Generator().manual_seed(M + N)
    A = torch.randn((M, lda), generator=g).to(torch.bfloat16)
    B = torch.randn((N, ldb), generator=g).to(torch.bfloat16)
    An, Bn = u16(A), u16(B)
    Cn = np.zeros((M, ldc), np.float32)
    rc = shim.miori_shim_test_naive(An.ctypes.data, Bn.ctypes.data, Cn.ctypes.data, M, N, K, lda, ldb, ldc)
    assert rc == 0, shim.miori_shim_last_error()
    want = port.gemm_bf16(np.ascontiguousarray(An[:, :K]), np.ascontiguousarray(Bn[:, :K]))
    assert_close(Cn[:, :N], want, rel_max=1e-4, what="shim gemm_naive")
    assert not Cn[:, N:].any()


def test_errors_surface_as_messages(shim):
    y = np.zeros((1, 16), np.float32)
    z = np.zeros(4096, np.uint32)
    # K not a multiple of the group: the operator throws, the entry reports it
    rc = shim.miori_shim_test_gemv(4, z.ctypes.data, z.ctypes.data, z.ctypes.data, z.ctypes.data,
                                   y.ctypes.data, 16, 48, 1)
    assert rc != 0 and b"multiple" in shim.miori_shim_last_error()


def test_neighbors_through_operator_api(shim, port):
    """embed8, rmsnorm and silu_mul with the reference's signatures (src/ops.h:16-24, 35-37), one
    command buffer, against the oracle's restatements of the shaders: the embedding bit for bit,
    the two float ops within one bf16 ulp."""
    rows8, K, T, rows, n_act = 300, 2048, 5, 3, 4096
    q, s, b = synth.make_weight(rows8, K, 8, 32, seed=41)
    tokens = np.array([0, 299, 7, 7, 123], np.int32)
    g = np.random.default_rng(3)
    x = g.standard_normal((rows, K)).astype(np.float32) * 3.0
    gamma = u16(synth.make_activation(1, K, seed=5)).reshape(-1)
    gate = g.standard_normal(n_act).astype(np.float32) * 4.0
    up = g.standard_normal(n_act).astype(np.float32)
    qn, sn, bn = u32(q), u16(s), u16(b)
    emb = np.zeros((T, K), np.uint16)
    norm = np.zeros((rows, K), np.uint16)
    act = np.zeros(n_act, np.uint16)
    p, u, f = C.c_void_p, C.c_uint32, C.c_float
    shim.miori_shim_test_neighbors.argtypes = [p, p, p, u, p, u, p, p, p, p, u, u, f, p, p, p, u]
    rc = shim.miori_shim_test_neighbors(qn.ctypes.data, sn.ctypes.data, bn.ctypes.data, rows8, tokens.ctypes.data, T,
                                        emb.ctypes.data, x.ctypes.data, gamma.ctypes.data, norm.ctypes.data, rows, K,
                                        1e-5, gate.ctypes.data, up.ctypes.data, act.ctypes.data, n_act)
    assert rc == 0, shim.miori_shim_last_error()
    assert np.array_equal(emb, port.embed8(qn, sn, bn, tokens, 32))

    def ulps(a, w):  # distance in bf16 steps between two arrays of bf16 bit patterns of equal sign
        return np.abs(a.astype(np.int32) - w.astype(np.int32)).max()
    assert ulps(norm, port.rmsnorm(x, gamma, 1e-5)) <= 1
    assert ulps(act, port.silu_mul(gate, up)) <= 1


def test_ffn_block_through_operator_api(shim, port):
    """The feed-forward block of a decode step (src/engine.cpp:388-399) encoded with the reference's
    six operators, with the gate + up GEMV that carries the activation, and with the norm in front of
    it too: the first two agree bit for bit, the third to the rounding of the normalised activations,
    and all follow the oracle's chain."""
    F, H = 1536, 2048
    q13, s13, b13 = synth.make_weight(2 * F, H, 4, 32, seed=51)
    q2, s2, b2 = synth.make_weight(H, F, 4, 32, seed=52)
    g = np.random.default_rng(9)
    x = g.standard_normal(H).astype(np.float32) * 2.0
    gi = u16(synth.make_activation(1, H, seed=6)).reshape(-1)
    gp = u16(synth.make_activation(1, H, seed=7)).reshape(-1)
    arrs = [u32(q13), u16(s13), u16(b13), u32(q2), u16(s2), u16(b2)]
    outs = [np.zeros(H, np.float32) for _ in range(3)]
    p, u, f = C.c_void_p, C.c_uint32, C.c_float
    shim.miori_shim_test_ffn.argtypes = [p] * 9 + [u, u, f, p, p, p]
    rc = shim.miori_shim_test_ffn(*[a.ctypes.data for a in arrs], gi.ctypes.data, gp.ctypes.data, x.ctypes.data,
                                  F, H, 1e-5, *[o.ctypes.data for o in outs])
    assert rc == 0, shim.miori_shim_last_error()
    six, gated, normed_gated = outs
    assert np.array_equal(six, gated), "the gated GEMV changes the block's result"
    h = port.rmsnorm(x[None, :], gi, 1e-5)
    y13 = port.gemv(4, arrs[0], arrs[1], arrs[2], h, 32)
    act = port.silu_mul(np.ascontiguousarray(y13[:, :F]), np.ascontiguousarray(y13[:, F:]))
    down = port.gemv(4, arrs[3], arrs[4], arrs[5], act, 32).astype(np.float32)
    want = port.post_norm_add(x[None, :], down, gp, 1e-5)[0]
    for name, got in (("six operators", six), ("norm + gated GEMV", normed_gated)):
        rel = np.abs(got - want).max() / np.abs(want).max()
        assert rel < 2e-3, f"{name}: max|d|/max|ref| = {rel:.2e}"
