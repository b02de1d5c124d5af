"""Times every (tile shape, K split) candidate of the cache GEMM on the benchmark's shapes and writes
tests/golden/gemm_candidates.json, the table tests/test_gemm_plan_cpu.py checks the planner against.
Needs one B200:  python tests/golden/make_gemm_candidates.py
"""
import sys, os, json
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import ctypes as C
import torch
import miori_b200
from miori_b200 import synth
from miori_b200._lib import lib
dev = "cuda:0"
PDL = miori_b200.LAUNCH_PDL
NARROW, WIDE, PAIR, NOPAIR = 0x100, 0x200, 0x4000, 0x8000
G = 64
def timed(fn, n=10):
    fn(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n): fn()
    e1.record(); torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n
out = []
for (N, K) in [(3072, 2048), (2048, 2048), (16384, 2048), (2048, 8192)]:
    npool = min(24, max(2, (300 << 20) // (N * K * 2)))
    pool = []
    for i in range(npool):
        q, s, b = synth.make_weight(N, K, 4, G, seed=N + K + i, device=dev)
        pool.append(miori_b200.dequant4_cache(q, s, b, group=G)); del q, s, b
    for M in (16, 32, 1024):
        A = synth.make_activation(M, K, seed=3, device=dev)
        obf = M >= 128
        Cm = torch.empty((M, N), device=dev, dtype=torch.bfloat16 if obf else torch.float32)
        ws = torch.empty(16 * M * N, dtype=torch.float32, device=dev)
        t, c, sp = C.c_uint32(), C.c_uint32(), C.c_uint32()
        lib.miori_gemm_plan(M, N, K, ws.numel() * 4, C.byref(t), C.byref(c), C.byref(sp))
        row = {"M": M, "N": N, "K": K, "pick": [t.value, c.value, sp.value], "us": {}}
        for name, tf in (("128x128", NARROW), ("128x256", WIDE), ("256x256 pair", PAIR)):
            if tf == PAIR and M <= 128: continue
            for s_ in (1, 2, 3, 4, 6, 8, 12):   # the forced count travels in four flag bits
                if s_ > max(1, K // 64 // 4): continue
                fl = PDL | tf | (s_ << 16) | (miori_b200.OUT_BF16 if obf else 0)
                def run():
                    for cch in pool:
                        miori_b200.gemm_bf16_cache(A, cch, N, flags=fl, out=Cm, workspace=ws)
                run(); torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g): run()
                us = 1e3 * timed(g.replay) / npool
                row["us"][f"{name} x{s_}"] = round(us, 2)
                del g
        # the default (planner's pick) through the same chain
        fl = PDL | (miori_b200.OUT_BF16 if obf else 0)
        def run():
            for cch in pool:
                miori_b200.gemm_bf16_cache(A, cch, N, flags=fl, out=Cm, workspace=ws)
        run(); torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g): run()
        row["default_us"] = round(1e3 * timed(g.replay) / npool, 2)
        best = min(row["us"], key=row["us"].get)
        print(f"M={M} N={N} K={K}: pick {row['pick']} default {row['default_us']} us; best {best} {row['us'][best]} us; all {row['us']}", flush=True)
        out.append(row)
    del pool
json.dump({"how": "python tests/golden/make_gemm_candidates.py on one B200: CUDA-event time per launch in a CUDA graph of "
                  "dependent launches over a pool of bf16 caches larger than L2; every tile shape and K split forced "
                  "through the private tuning flags", "rows": out},
          open(os.path.join(HERE, "gemm_candidates.json"), "w"), indent=1)
print("deverr", lib.miori_device_error_poll())
