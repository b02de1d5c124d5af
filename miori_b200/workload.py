"""Run one operator of the library on synthetic data, for timing or profiling a single kernel.

    python -m miori_b200.workload gemv --bits 4 --n 131072 --k 2048 --m 1 --group 64 --reps 7
    python -m miori_b200.workload gemm --m 1024 --n 16384 --k 2048 --pool 3 --reps 2

Prints the CUDA-event time per launch.  Weights are drawn from a pool of `--pool` distinct tensors
so that a working set larger than L2 can be requested.
"""
from __future__ import annotations

import argparse

import torch

import miori_b200
from miori_b200 import synth


def _time(fn, reps):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("op", choices=["gemv", "gemm", "dequant"])
    ap.add_argument("--bits", type=int, default=4, choices=[4, 8])
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--group", type=int, default=64, choices=[32, 64])
    ap.add_argument("--pool", type=int, default=1)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--flags", type=lambda v: int(v, 0), default=0)
    a = ap.parse_args()
    dev = "cuda:0"
    bits = 4 if a.op != "gemv" else a.bits
    pool = [synth.make_weight(a.n, a.k, bits, a.group, seed=i, device=dev) for i in range(a.pool)]
    x = synth.make_activation(a.m, a.k, seed=99, device=dev)
    wbytes = a.n * a.k * bits // 8 + a.n * (a.k // a.group) * 4
    if a.op == "gemv":
        fn = miori_b200.gemv4 if a.bits == 4 else miori_b200.gemv8
        y = torch.empty((a.m, a.n), device=dev)
        ms = _time(lambda: [fn(q, s, b, x, group=a.group, flags=a.flags, out=y) for q, s, b in pool], a.reps)
        ms /= a.pool
        print(f"gemv{a.bits} N={a.n} K={a.k} M={a.m} g={a.group}: {ms * 1e3:.2f} us/launch "
              f"{wbytes / ms / 1e6:.0f} GB/s")
    elif a.op == "dequant":
        out = torch.empty((a.n, a.k), dtype=torch.bfloat16, device=dev)
        ms = _time(lambda: [miori_b200.dequant4_rowmajor(q, s, b, group=a.group, out=out) for q, s, b in pool],
                   a.reps) / a.pool
        print(f"dequant4 N={a.n} K={a.k}: {ms * 1e3:.2f} us/launch {(wbytes + 2 * a.n * a.k) / ms / 1e6:.0f} GB/s")
    else:
        caches = [miori_b200.dequant4_cache(q, s, b, group=a.group) for q, s, b in pool]
        del pool
        ws = miori_b200.gemm_workspace(a.m, a.n, a.k, dev)
        Cm = torch.empty((a.m, a.n), device=dev)
        ms = _time(lambda: [miori_b200.gemm_bf16_cache(x, c, a.n, flags=a.flags, out=Cm, workspace=ws)
                            for c in caches], a.reps) / a.pool
        print(f"gemm M={a.m} N={a.n} K={a.k}: {ms * 1e3:.2f} us/launch "
              f"{2.0 * a.m * a.n * a.k / ms / 1e9:.0f} TFLOP/s")


if __name__ == "__main__":
    main()
