"""GPU bit-exactness of the int4/int8 -> bf16 cache build against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

import miori_b200
from miori_b200 import ops, synth
from conftest import GOLDEN, u16, u32

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("name", ["dequant4_bitpatterns", "dequant8_bitpatterns",
                                  "gemv4_n48_k256_m1_ramp", "gemv8_n40_k256_m1_ramp"])
def test_golden_cache_bits(name):
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    bits = int(g["bits"])
    q = torch.from_numpy(g["q"].view(np.int32)).to(DEV)
    s = torch.from_numpy(g["s"].view(np.int16)).view(torch.bfloat16).to(DEV)
    b = torch.from_numpy(g["b"].view(np.int16)).view(torch.bfloat16).to(DEV)
    fn = miori_b200.dequant4_rowmajor if bits == 4 else miori_b200.dequant8_rowmajor
    out = fn(q, s, b, group=32)
    assert np.array_equal(u16(out), g["cache"])


@pytest.mark.parametrize("group", [32, 64])
@pytest.mark.parametrize("bits,N,K", [(4, 2048, 2048), (4, 16, 2048), (4, 3072, 2048), (4, 2048, 8192),
                                      (4, 1000, 7680), (8, 4000, 2048), (8, 33, 128), (4, 1, 64)])
def test_rowmajor_bit_exact(port, bits, N, K, group):
    q, s, b = synth.make_weight(N, K, bits, group, seed=N + K + bits)
    fn = miori_b200.dequant4_rowmajor if bits == 4 else miori_b200.dequant8_rowmajor
    out = fn(q.to(DEV), s.to(DEV), b.to(DEV), group=group)
    want = port.dequant_rowmajor(bits, u32(q), u16(s), u16(b), group)
    assert np.array_equal(u16(out), want)


@pytest.mark.parametrize("group", [32, 64])
def test_cache_roundtrips_to_rowmajor(port, group):
    """The GEMM's private cache layout, undone, equals the row-major cache bit for bit."""
    N, K = 3072, 2048
    q, s, b = synth.make_weight(N, K, 4, group, seed=41)
    cache = miori_b200.dequant4_cache(q.to(DEV), s.to(DEV), b.to(DEV), group=group)
    assert cache.numel() * 2 == miori_b200.lib.miori_cache_bytes(N, K)
    row = ops.cache_to_rowmajor(cache, N, K)
    assert np.array_equal(u16(row), port.dequant_rowmajor(4, u32(q), u16(s), u16(b), group))


def test_full_size_cache_checksum(port):
    """gate+up projection (16384 x 2048): sampled rows bit-exact, and the whole tensor agrees
    with a dequantization done row-shard by row-shard (layout independent of launch shape)."""
    N, K = 16384, 2048
    q, s, b = synth.make_weight(N, K, 4, 64, seed=43, device=DEV)
    out = miori_b200.dequant4_rowmajor(q, s, b, group=64)
    rows = np.arange(0, N, 257)
    want = port.dequant_rowmajor(4, u32(q[rows]), u16(s[rows]), u16(b[rows]), 64)
    assert np.array_equal(u16(out[rows]), want)
    parts = [miori_b200.dequant4_rowmajor(q[i:i + 4096].contiguous(), s[i:i + 4096].contiguous(),
                                          b[i:i + 4096].contiguous(), group=64)
             for i in range(0, N, 4096)]
    assert torch.equal(torch.cat(parts), out)
