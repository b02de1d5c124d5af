"""Generate tests/golden/*.npz from the reference's own CPU checker.

Run in a container where the reference sources are mounted (oracle/Makefile compiles the
reference's src/cpu_ref.h, unmodified, into oracle/_ref/libmiori_cpuref.so):

    python tests/golden/make_golden.py

Each fixture stores the inputs (packed codes, bf16 scales/biases, bf16 activations) and the
outputs computed by that compiled reference header: per-element dequantized weights
(dequant4_elem / dequant8_elem), their bf16 rounding (float_to_bf16), and the double
-precision GEMV that the reference's test procedure defines (src/main.cpp:67-86).  Group
size is 32, the only one the reference header supports.  The reference repository holds no
golden vectors of its own for this path; these stand in for them.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from miori_b200 import synth  # noqa: E402
from oracle import oracle  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def bits16(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main():
    oracle.build()
    ref = oracle.ref()
    if ref is None:
        raise SystemExit("oracle/_ref was not built: reference sources are not mounted")
    cases = [
        # name, bits, N, K, M, x kind
        ("gemv4_n48_k256_m1_ramp", 4, 48, 256, 1, "ramp"),
        ("gemv4_n33_k512_m4_randn", 4, 33, 512, 4, "randn"),
        ("gemv8_n40_k256_m1_ramp", 8, 40, 256, 1, "ramp"),
        ("gemv8_n17_k128_m3_randn", 8, 17, 128, 3, "randn"),
    ]
    for i, (name, bits, N, K, M, kind) in enumerate(cases):
        q, s, b = synth.make_weight(N, K, bits, 32, seed=1000 + i)
        x = synth.ramp_activation(M, K) if kind == "ramp" else synth.make_activation(M, K, 2000 + i)
        qn, sn, bn, xn = q.numpy().view(np.uint32), bits16(s), bits16(b), bits16(x)
        w = np.array([[ref.dequant_elem(bits, qn, sn, bn, n, k, K) for k in range(K)]
                      for n in range(N)], np.float32)
        cache = ref.dequant_rowmajor(bits, qn, sn, bn)
        y = ref.gemv(bits, qn, sn, bn, xn)
        np.savez_compressed(os.path.join(OUT, name + ".npz"), bits=bits, group=32, q=qn, s=sn, b=bn,
                            x=xn, w=w, cache=cache, y=y)
        print(name, "y[0,:3] =", y[0, :3])
    # adversarial scale/bias bit patterns (denormals, large magnitudes, negative scales)
    rng = np.random.default_rng(7)
    N, K = 24, 128
    for bits in (4, 8):
        qn = rng.integers(0, 2**32, size=(N, K * bits // 32), dtype=np.uint64).astype(np.uint32)
        sn = rng.integers(0, 2**16, size=(N, K // 32), dtype=np.uint32).astype(np.uint16)
        bn = rng.integers(0, 2**16, size=(N, K // 32), dtype=np.uint32).astype(np.uint16)
        # keep exponents finite (no Inf/NaN: the reference's rounding has no special case)
        sn[(sn & 0x7F80) == 0x7F80] &= 0xBFFF
        bn[(bn & 0x7F80) == 0x7F80] &= 0xBFFF
        w = np.array([[ref.dequant_elem(bits, qn, sn, bn, n, k, K) for k in range(K)]
                      for n in range(N)], np.float32)
        cache = ref.dequant_rowmajor(bits, qn, sn, bn)
        np.savez_compressed(os.path.join(OUT, f"dequant{bits}_bitpatterns.npz"), bits=bits, group=32,
                            q=qn, s=sn, b=bn, w=w, cache=cache)
        print(f"dequant{bits}_bitpatterns", cache[0, :4])


if __name__ == "__main__":
    main()
