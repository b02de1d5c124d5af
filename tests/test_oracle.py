"""CPU tests of the oracle itself: known answers, the golden vectors made by the
reference's own header, and agreement with that header when it is compiled here."""
import glob
import os

import numpy as np
import pytest

from conftest import GOLDEN


def _golden(pattern):
    files = sorted(glob.glob(os.path.join(GOLDEN, pattern)))
    assert files, f"no golden fixtures match {pattern}"
    return files


def test_known_answer_nibbles(port):
    # word 0x76543210, scale 0.5, bias -1: codes 0..7 -> -1, -0.5, ..., 2.5
    q = np.array([[0x76543210, 0xFEDCBA98, 0, 0xFFFFFFFF]], np.uint32)
    s = port.float_to_bf16(np.array([[0.5]], np.float32))
    b = port.float_to_bf16(np.array([[-1.0]], np.float32))
    got = [port.dequant_elem(4, q, s, b, 0, k, 32, 32) for k in range(32)]
    want = [c * 0.5 - 1.0 for c in list(range(16)) + [0] * 8 + [15] * 8]
    assert got == want


def test_known_answer_bytes(port):
    q = np.array([[0x03020100, 0xFF808001] + [0] * 6], np.uint32)
    s = port.float_to_bf16(np.array([[0.25]], np.float32))
    b = port.float_to_bf16(np.array([[2.0]], np.float32))
    got = [port.dequant_elem(8, q, s, b, 0, k, 32, 32) for k in range(8)]
    assert got == [2.0, 2.25, 2.5, 2.75, 2.25, 34.0, 34.0, 65.75]


def test_bf16_rounding_known_answers(port):
    f2b = port.lib.mo_float_to_bf16
    assert f2b(3.14159) == 0x4049
    assert f2b(1.0) == 0x3F80
    # ties to even: 1 + 2^-8 is halfway between 0x3F80 and 0x3F81
    assert f2b(1.0 + 2.0**-8) == 0x3F80
    assert f2b(1.0 + 3 * 2.0**-8) == 0x3F82
    assert port.lib.mo_bf16_to_float(0xC000) == -2.0


@pytest.mark.parametrize("path", _golden("gemv*.npz"))
def test_port_matches_golden_gemv(port, path):
    g = np.load(path)
    bits, K = int(g["bits"]), g["x"].shape[1]
    N = g["q"].shape[0]
    w = np.array([[port.dequant_elem(bits, g["q"], g["s"], g["b"], n, k, K, 32) for k in range(K)]
                  for n in range(N)], np.float32)
    assert np.array_equal(w.view(np.uint32), g["w"].view(np.uint32))
    assert np.array_equal(port.dequant_rowmajor(bits, g["q"], g["s"], g["b"], 32), g["cache"])
    y = port.gemv(bits, g["q"], g["s"], g["b"], g["x"], 32)
    assert np.array_equal(y, g["y"])  # same double-precision summation order


@pytest.mark.parametrize("path", _golden("dequant*_bitpatterns.npz"))
def test_port_matches_golden_bitpatterns(port, path):
    g = np.load(path)
    bits = int(g["bits"])
    assert np.array_equal(port.dequant_rowmajor(bits, g["q"], g["s"], g["b"], 32), g["cache"])


@pytest.mark.parametrize("bits", [4, 8])
def test_port_equals_compiled_reference(port, ref, bits):
    if ref is None:
        pytest.skip("oracle/_ref not built (reference sources not mounted)")
    import torch
    from miori_b200 import synth
    from conftest import u16, u32
    q, s, b = synth.make_weight(96, 1024, bits, 32, seed=11 + bits)
    x = synth.make_activation(3, 1024, seed=5)
    qn, sn, bn, xn = u32(q), u16(s), u16(b), u16(x)
    assert np.array_equal(port.gemv(bits, qn, sn, bn, xn, 32), ref.gemv(bits, qn, sn, bn, xn))
    assert np.array_equal(port.dequant_rowmajor(bits, qn, sn, bn, 32),
                          ref.dequant_rowmajor(bits, qn, sn, bn))


@pytest.mark.parametrize("bits", [4, 8])
def test_group64_equals_group32_with_repeated_scales(port, ref, bits):
    """A group-64 tensor is a group-32 tensor whose scales repeat in pairs, so the group-64
    restatement can be checked by the group-32 reference header."""
    from miori_b200 import synth
    from conftest import u16, u32
    q, s, b = synth.make_weight(40, 512, bits, 64, seed=21 + bits)
    x = synth.make_activation(2, 512, seed=6)
    qn, sn, bn, xn = u32(q), u16(s), u16(b), u16(x)
    s32, b32 = np.repeat(sn, 2, axis=1), np.repeat(bn, 2, axis=1)
    assert np.array_equal(port.gemv(bits, qn, sn, bn, xn, 64), port.gemv(bits, qn, s32, b32, xn, 32))
    assert np.array_equal(port.dequant_rowmajor(bits, qn, sn, bn, 64),
                          port.dequant_rowmajor(bits, qn, s32, b32, 32))
    if ref is not None:
        assert np.array_equal(port.gemv(bits, qn, sn, bn, xn, 64), ref.gemv(bits, qn, s32, b32, xn))


def test_tile_layout_is_a_permutation_of_rowmajor(port):
    from miori_b200 import synth
    from conftest import u16, u32
    q, s, b = synth.make_weight(128, 256, 4, 32, seed=31)
    row = port.dequant_rowmajor(4, u32(q), u16(s), u16(b), 32)
    tile = port.dequant_tile(u32(q), u16(s), u16(b), 32)  # [N/64][K][64]
    assert np.array_equal(tile.transpose(0, 2, 1).reshape(128, 256), row)


def test_gemm_oracle_small(port):
    rng = np.random.default_rng(3)
    A = port.float_to_bf16(rng.standard_normal((5, 64)).astype(np.float32))
    B = port.float_to_bf16(rng.standard_normal((7, 64)).astype(np.float32))
    want = port.bf16_to_float(A).astype(np.float64) @ port.bf16_to_float(B).astype(np.float64).T
    got = port.gemm_bf16(A, B)
    assert np.allclose(got, want, rtol=1e-12, atol=1e-12)
    assert got[2, 3] == port.gemm_entry(A, B, 2, 3)


def test_quantizer_matches_torch_generator(port):
    import torch
    from miori_b200 import synth
    from conftest import u16, u32
    W = torch.randn(32, 256, generator=torch.Generator().manual_seed(9)) * 0.02
    W[3, 64:128] = 0.0125  # a constant group
    for bits, group in [(4, 32), (4, 64), (8, 32), (8, 64)]:
        qa, sa, ba = synth.quantize_affine(W, bits, group)
        qb, sb, bb = port.quantize(bits, W.numpy(), group)
        assert np.array_equal(u32(qa), qb) and np.array_equal(u16(sa), sb) and np.array_equal(u16(ba), bb)
        # reconstruction error is at most half a step (plus the bf16 rounding of scale/bias)
        w = port.bf16_to_float(port.dequant_rowmajor(bits, qb, sb, bb, group))
        step = port.bf16_to_float(sb).repeat(group, axis=1)
        assert (np.abs(w - W.numpy()) <= 0.75 * step + 1e-3).all()


def test_known_answers_of_the_projection_neighbours(port):
    """rmsnorm, silu_mul, post_norm_add and embed8 (shaders/ops.metal:86-115, 129-139, 605-631, 170-197)
    on inputs whose results can be written down by hand."""
    bf = lambda *v: port.float_to_bf16(np.array(v, np.float32))
    # rmsnorm: mean(x^2) = 4, eps = 0 -> inv = 1/2; y = x * 0.5 * w
    y = port.rmsnorm(np.array([[2.0, -2.0, 2.0, -2.0]], np.float32), bf(1.0, 1.0, 0.5, 3.0), 0.0)
    assert y.tolist() == [[0x3F80, 0xBF80, 0x3F00, 0xC040]]           # 1, -1, 0.5, -3
    # eps alone under the root: x = 0 stays 0; x = 1 with eps = 3 -> 1/sqrt(1 + 3) = 0.5
    assert port.rmsnorm(np.zeros((1, 4), np.float32), bf(1, 1, 1, 1), 1e-5).tolist() == [[0, 0, 0, 0]]
    assert port.rmsnorm(np.ones((1, 2), np.float32), bf(1.0, 2.0), 3.0).tolist() == [[0x3F00, 0x3F80]]
    # silu_mul: silu(0) = 0; silu(ln 3) = 0.75 ln 3 = 0.82396 -> bf16 0x3F53 (0.82422; 0x3F52 is 0.82031);
    # a large gate passes through (silu(100) = 100 in fp32), a large negative one gives -0 * up = -0 or 0
    g = np.array([0.0, np.log(3.0), 100.0, 100.0], np.float32)
    u = np.array([5.0, 1.0, 1.0, -0.5], np.float32)
    assert port.silu_mul(g, u).tolist() == [0x0000, 0x3F53, 0x42C8, 0xC248]   # 0, 0.824, 100, -50
    assert port.silu_mul(np.array([-100.0], np.float32), np.array([1.0], np.float32))[0] & 0x7FFF == 0
    # post_norm_add: src = (2, -2): mean square 4, inv = 0.5 -> x + src * 0.5 * w
    out = port.post_norm_add(np.array([[1.0, 2.0]], np.float32), np.array([[2.0, -2.0]], np.float32), bf(1.0, 0.5), 0.0)
    assert out.tolist() == [[2.0, 1.5]]
    # embed8: row 1 of a two-row table, codes 0, 1, 2, 3 and 255 with scale 0.5, bias -1
    q = np.zeros((2, 8), np.uint32)
    q[1, 0], q[1, 1] = 0x03020100, 0x000000FF
    s, b = np.tile(bf(0.5), (2, 1)), np.tile(bf(-1.0), (2, 1))
    e = port.embed8(q, s, b, np.array([1, 0], np.uint32), 32)
    assert e.shape == (2, 32)
    assert e[0, :5].tolist() == [0xBF80, 0xBF00, 0x0000, 0x3F00, 0x42FD]     # -1, -0.5, 0, 0.5, 126.5
    assert (e[1] == 0xBF80).all()                                            # row 0: all codes 0 -> -1
