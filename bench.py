#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path on B200.

Headline workload: a synthetic 24-layer int4 stack, four
projections per layer (2048->3072, 2048->2048, 2048->16384, 8192->2048), group-64 affine
4-bit weights, evaluated at M in {1,2,4,8,16,32} activation rows.  One "step" is one pass of
the GEMV path over the whole stack at each of the six M values (576 GEMV launches, six
CUDA graphs with programmatic dependent launch).  `value` is effective HBM GB/s over the
packed weight bytes streamed per step, inputs resident in HBM.  `e2e` is the same metric
with host buffers: every pass copies its activations from pinned host memory and reads the
last layer's outputs back, all through the C ABI.

`--impl reference` times the reference's CPU arithmetic (its own header compiled into
oracle/_ref when present, else the C port in oracle/) on the host cores on a bounded sample, at
every M of the sweep.

With torchrun (N>1) the total work is fixed (strong scaling).  A projection is split by output
rows over the ranks, its y gathered by peer stores from the GEMV's own epilogue (or by
ncclAllGather with --allgather nccl), only when its weights are large enough for the split to
pay; the others are computed by every rank.  By default (--shard auto) both choices are replayed
for every M before the timed region and the faster one is kept.  Outside the timed
region every rank checks one forced-sharded pass against the single-GPU kernels.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS = 24
SHAPES = [(3072, 2048), (2048, 2048), (16384, 2048), (2048, 8192)]  # (N, K)
M_SWEEP = [1, 2, 4, 8, 16, 32]
GEMM_SHAPES = [(3072, 2048), (2048, 2048), (16384, 2048), (2048, 8192)]


def packed_bytes(N, K, bits, group):
    return N * K * bits // 8 + N * (K // group) * 4


class ClockSampler:
    """SM clock and throttle reasons sampled (NVML, every few milliseconds) while the measurements run."""

    def __init__(self, index):
        self.index, self.samples, self.reasons, self.stop_flag, self.t = index, [], set(), False, None
        self.max_mhz, self.err = None, None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # no NVML: report that instead of clocks
            self.err = f"NVML unavailable: {e}"
            return
        self.t = threading.Thread(target=self._pump, daemon=True)
        self.t.start()

    def _pump(self):
        nv = self.nv
        names = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown,
                 "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                 "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
        while not self.stop_flag:
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for nm, bit in names.items():
                    if bits & bit:
                        self.reasons.add(nm)
            except Exception as e:
                self.err = str(e)
                return
            time.sleep(0.004)

    def clear(self):
        self.samples, self.reasons = [], set()

    def stop(self):
        self.stop_flag = True
        if self.t is not None:
            self.t.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "samples": 0,
                    "reasons": [self.err or "no samples"]}
        sm = sorted(self.samples)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": self.max_mhz, "samples": len(sm),
                "reasons": sorted(self.reasons)}


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p, "measured"
    except (OSError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# --------------------------------------------------------------------------- CPU arm

def cpu_decode_sample(group, seconds=12.0):
    """Time the reference's CPU arithmetic on one layer of the stack at every M of the sweep.

    The reference's own header (oracle/_ref, src/cpu_ref.h compiled unmodified) does the work when
    it was built; it hard-codes group 32, so a group-64 tensor is handed to it as the identical
    group-32 tensor with every scale and bias repeated twice.  Each M gets an equal share of
    `seconds` on a row prefix of every projection sized to fit that share (the loop's time is
    proportional to rows x M), and the throughput is combined over the sweep exactly as the GPU
    arm combines its passes: total weight bytes of six passes / total time of six passes."""
    import numpy as np
    import torch
    from miori_b200 import synth
    from oracle import oracle

    ref = oracle.ref()
    port = oracle.port()
    kind = "reference" if ref is not None else "port"
    cores = (ref or port).threads()

    def u16(t):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)

    layer = []
    for i, (N, K) in enumerate(SHAPES):
        q, s, b = synth.make_weight(N, K, 4, group, seed=100 + i)
        sn, bn = u16(s), u16(b)
        if ref is not None and group == 64:
            sn, bn = np.repeat(sn, 2, axis=1), np.repeat(bn, 2, axis=1)
        layer.append((N, K, q.numpy().view(np.uint32), np.ascontiguousarray(sn), np.ascontiguousarray(bn)))
    xs = {M: [u16(synth.make_activation(M, K, seed=7 + M)) for _, K in SHAPES] for M in M_SWEEP}

    def run(M, frac):
        """One pass over the first `frac` of every projection's rows; returns (seconds, bytes)."""
        nbytes, t0 = 0, time.perf_counter()
        for (N, K, q, s, b), x in zip(layer, xs[M]):
            rows = max(16, int(N * frac)) if frac < 1.0 else N
            if ref is not None:
                ref.gemv(4, q, s, b, x, rows=(0, rows))
            else:
                port.gemv(4, q, s, b, x, group, rows=(0, rows))
            nbytes += packed_bytes(rows, K, 4, group)
        return time.perf_counter() - t0, nbytes

    run(1, 1.0)
    t1, _ = run(1, 1.0)              # one full layer at M = 1
    share = seconds / len(M_SWEEP)
    per_m, inv_rate_sum, used = {}, 0.0, 0.0
    for M in M_SWEEP:
        frac = min(1.0, share / (t1 * M))
        reps = max(1, int(share / max(t1 * M * frac, 1e-6)))
        reps = min(reps, 200)
        t, by = 0.0, 0
        for _ in range(reps):
            dt, nb = run(M, frac)
            t += dt
            by += nb
        rate = by / t / 1e9          # weight GB/s at this M
        per_m[str(M)] = {"gbs": rate, "row_fraction": round(frac, 4), "passes": reps}
        inv_rate_sum += 1.0 / rate
        used += t
    gbs = len(M_SWEEP) / inv_rate_sum
    return {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"one layer (4 projections, group {group}) at each M of {M_SWEEP}, a row prefix of "
                      f"every projection sized for {share:.1f} s per M; double-precision dot of "
                      f"dequant4_elem as src/main.cpp:67-86"
                      + ("; group-64 scales handed to the group-32 header repeated twice" if ref is not None and group == 64 else ""),
            "per_m": per_m, "seconds": used}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, t_all, vals = max(1, args.steps), 0.0, []
    per_step = max(6.0, min(24.0, 120.0 / (steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_decode_sample(args.group, seconds=per_step / 3)
    base = None
    for _ in range(steps):
        base = cpu_decode_sample(args.group, seconds=per_step)
        vals.append(base["value"])
        t_all += base["seconds"]
    value = sum(vals) / len(vals)
    base["value"] = value
    out = {
        "impl": "reference", "metric": METRIC, "value": value,
        "unit": "GB/s", "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * t_all / steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f64 accumulate over f32 dequant", "data": "synthetic",
        "config": workload_config(args), "cpu_baseline": base,
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out))


METRIC = "int4 GEMV effective HBM GB/s (M=1-32)"


def run_one(a):
    """`--one`: a single operator on synthetic data, `--reps` timed launches per weight tensor after
    one untimed pass; prints the CUDA-event time per launch.  The weights come from a pool of
    `--pool` distinct tensors so that a working set larger than L2 can be asked for."""
    import torch
    import miori_b200
    from miori_b200 import synth

    dev = "cuda:0"
    G = a.group
    bits = a.bits if a.one.startswith("gemv") else 4
    pool = [synth.make_weight(a.n, a.k, bits, G, seed=i, device=dev) for i in range(a.pool)]
    x = synth.make_activation(a.m, a.k, seed=99, device=dev)
    wbytes = packed_bytes(a.n, a.k, bits, G)

    def time_ms(fn):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / a.reps / a.pool

    if a.one == "gemv":
        fn = miori_b200.gemv4 if bits == 4 else miori_b200.gemv8
        y = torch.empty((a.m, a.n), device=dev)
        ms = time_ms(lambda: [fn(q, s, b, x, group=G, flags=a.flags, out=y) for q, s, b in pool])
        print(f"gemv{bits} N={a.n} K={a.k} M={a.m} g={G} flags={a.flags:#x}: {ms * 1e3:.2f} us/launch "
              f"{wbytes / ms / 1e6:.0f} GB/s")
    elif a.one == "gemv_rmsnorm":
        fn = miori_b200.gemv4_rmsnorm if bits == 4 else miori_b200.gemv8_rmsnorm
        xf = x.float()
        gamma = synth.make_activation(1, a.k, seed=98, device=dev).float().reshape(-1)
        y = torch.empty((a.m, a.n), device=dev)
        ms = time_ms(lambda: [fn(q, s, b, xf, gamma, 1e-5, group=G, flags=a.flags, out=y) for q, s, b in pool])
        print(f"gemv{bits}_rmsnorm N={a.n} K={a.k} M={a.m} g={G}: {ms * 1e3:.2f} us/launch "
              f"{wbytes / ms / 1e6:.0f} GB/s")
    elif a.one == "gemv_silu":
        act = torch.empty((a.m, a.n // 2), dtype=torch.bfloat16, device=dev)
        ms = time_ms(lambda: [miori_b200.gemv4_silu(q, s, b, x, group=G, flags=a.flags, out=act) for q, s, b in pool])
        print(f"gemv4_silu N={a.n} K={a.k} M={a.m} g={G}: {ms * 1e3:.2f} us/launch {wbytes / ms / 1e6:.0f} GB/s")
    elif a.one == "dequant":
        out = torch.empty((a.n, a.k), dtype=torch.bfloat16, device=dev)
        ms = time_ms(lambda: [miori_b200.dequant4_rowmajor(q, s, b, group=G, out=out) for q, s, b in pool])
        print(f"dequant4 N={a.n} K={a.k}: {ms * 1e3:.2f} us/launch {(wbytes + 2 * a.n * a.k) / ms / 1e6:.0f} GB/s")
    elif a.one == "gemv_cache":
        caches = [miori_b200.dequant4_cache(q, s, b, group=G) for q, s, b in pool]
        del pool
        y = torch.empty((a.m, a.n), device=dev)
        ms = time_ms(lambda: [miori_b200.gemv_bf16_cache(x, c, a.n, flags=a.flags, out=y) for c in caches])
        print(f"gemv_bf16_cache N={a.n} K={a.k} M={a.m}: {ms * 1e3:.2f} us/launch "
              f"{2.0 * a.n * a.k / ms / 1e6:.0f} GB/s of cache")
    else:
        caches = [miori_b200.dequant4_cache(q, s, b, group=G) for q, s, b in pool]
        del pool
        ws = miori_b200.gemm_workspace(a.m, a.n, a.k, dev)
        Cm = torch.empty((a.m, a.n), device=dev)
        ms = time_ms(lambda: [miori_b200.gemm_bf16_cache(x, c, a.n, flags=a.flags, out=Cm, workspace=ws)
                              for c in caches])
        print(f"gemm M={a.m} N={a.n} K={a.k}: {ms * 1e3:.2f} us/launch "
              f"{2.0 * a.m * a.n * a.k / ms / 1e9:.0f} TFLOP/s")


def workload_config(args):
    """The workload both arms print (identical dicts: the driver compares them)."""
    return {"workload": "decode_stack_int4: 24 layers x {2048->3072, 2048->2048, 2048->16384, "
                        "8192->2048}, M in {1,2,4,8,16,32}", "group": args.group, "bits": 4,
            "layers": args.layers, "m_sweep": M_SWEEP, "out": "f32", "n_gpus": args.gpus,
            "l2": "inputs larger than L2 (821 MB of weights per pass)"}


# --------------------------------------------------------------------------- GPU arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--group", type=int, default=64, choices=[32, 64])
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary measurements")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--allgather", default="peer", choices=["peer", "nccl"],
                    help="N > 1: gather y by peer stores from the GEMV epilogue (default) or with "
                         "ncclAllGather after each launch")
    ap.add_argument("--shard", default="auto", choices=["auto", "policy", "all", "none"],
                    help="N > 1: which projections are split by rows over the ranks: those whose packed "
                         "weights reach --shard-bytes (policy), all of them, none, or per batch size "
                         "whichever of policy / none replays faster (auto)")
    ap.add_argument("--shard-bytes", type=int, default=16 << 20,
                    help="policy: a projection is split when its packed weights reach this many bytes")
    ap.add_argument("--eager", action="store_true",
                    help="launch the passes directly instead of replaying CUDA graphs (for a "
                         "profiler's launch list; timings then include host launch overhead)")
    ap.add_argument("--layers", type=int, default=LAYERS, help="stack depth (24 is the benchmark)")
    ap.add_argument("--verbose", action="store_true", help="progress on stderr")
    one = ap.add_argument_group("one operator on one GPU (--one): a small case to time or to profile")
    one.add_argument("--one", choices=["gemv", "gemv_rmsnorm", "gemv_silu", "gemm", "gemv_cache", "dequant"])
    one.add_argument("--bits", type=int, default=4, choices=[4, 8])
    one.add_argument("--n", type=int, default=8192)
    one.add_argument("--k", type=int, default=2048)
    one.add_argument("--m", type=int, default=1)
    one.add_argument("--pool", type=int, default=1, help="distinct weight tensors visited in turn")
    one.add_argument("--reps", type=int, default=5)
    one.add_argument("--flags", type=lambda v: int(v, 0), default=0)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.one:
        run_one(args)
        return

    import torch
    import torch.distributed as dist
    import miori_b200
    from miori_b200 import synth
    from miori_b200._lib import check, lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    layers = args.layers

    def say(msg):
        if args.verbose:
            print(f"[bench rank {rank}] {msg}", file=sys.stderr, flush=True)

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    G = args.group
    pdl = 0 if args.no_pdl else miori_b200.LAUNCH_PDL

    # ---- which projections are split by rows over the ranks.  Every rank holds the whole stack
    # (0.7 GB); a split projection reads only its own rows of q / s / b (rows are contiguous, so a
    # shard is a view), which lets the split be decided per projection and per batch size.
    from miori_b200 import shard as shard_plan
    wbytes = [packed_bytes(N, K, 4, G) for N, K in SHAPES]
    no_split = [False] * len(SHAPES)
    if args.shard == "auto":
        candidates = [no_split, shard_plan.split_plan(wbytes, world, args.shard_bytes, "policy")]
    else:
        candidates = [shard_plan.split_plan(wbytes, world, args.shard_bytes, args.shard)]
    candidates = [c for n, c in enumerate(candidates) if c not in candidates[:n]]
    split = {M: candidates[-1] for M in M_SWEEP}   # per M; settled by measurement below when "auto"

    def my_rows(t, N):
        rows = N // world
        return t[rank * rows:(rank + 1) * rows]

    def my_cache_rows(cache, N, K):
        # the bf16 cache is flat; rows are stored one after the other (a promise of the header)
        rows = N // world
        lo, hi = lib.miori_cache_bytes(rank * rows, K) // 2, lib.miori_cache_bytes((rank + 1) * rows, K) // 2
        return cache[lo:hi]

    stack = []
    for l in range(layers):
        projs = []
        for i, (N, K) in enumerate(SHAPES):
            assert N % (16 * world) == 0
            projs.append(synth.make_weight(N, K, 4, G, seed=1234 + l * 4 + i, device=dev))
        stack.append(projs)
    bytes_pass = layers * sum(packed_bytes(N, K, 4, G) for N, K in SHAPES)  # whole job
    say("weights ready")
    # the four activations of a pass live in one device buffer, so the end-to-end leg moves each
    # pass's inputs with one copy
    def carve(flat, shapes):
        out, at = [], 0
        for shp in shapes:
            n = shp[0] * shp[1]
            n_al = (n + 127) // 128 * 128  # keep every view 256-byte aligned
            out.append(flat[at:at + n].view(shp))
            at += n_al
        return out

    def flat_len(shapes):
        return sum((a * b + 127) // 128 * 128 for a, b in shapes)

    x_flat, x_dev, y_loc, y_part = {}, {}, {}, {}
    for M in M_SWEEP:
        xs = [(M, K) for _, K in SHAPES]
        x_flat[M] = torch.empty(flat_len(xs), dtype=torch.bfloat16, device=dev)
        x_dev[M] = carve(x_flat[M], xs)
        # outputs of unsplit projections, and this rank's rows of a split one on the cache-GEMM path
        y_loc[M] = [torch.empty((M, N), device=dev) for N, _ in SHAPES]
        y_part[M] = [torch.empty((M, N // world), device=dev) for N, _ in SHAPES] if world > 1 else None
        for v, (_, K) in zip(x_dev[M], SHAPES):
            v.copy_(synth.make_activation(M, K, seed=50 + M, device=dev))
    # N > 1: the gathered outputs of split projections.  "peer": y[M][N] at the same offset of every
    # rank's arena, written by all ranks' GEMV epilogues over NVLink; "nccl": rank-major blocks
    grp, gather = None, "none"
    if world > 1 and args.allgather == "peer":
        from miori_b200.peers import PeerGroup
        try:
            grp = PeerGroup(rank, world, 32 << 20, dev)
            gather = "peer stores fused in the GEMV epilogue"
        except RuntimeError as e:
            say(f"peer mapping unavailable ({e}); using ncclAllGather")
    if world > 1 and grp is None:
        gather = "ncclAllGather after each launch"
    y_off = {M: [grp.alloc(M * N * 4) if grp is not None else None for N, _ in SHAPES] for M in M_SWEEP}

    def gathered(M, i):
        """Where the whole y of projection i ends up on this rank."""
        N = SHAPES[i][0]
        if not split[M][i]:
            return y_loc[M][i]
        if grp is not None:
            return grp.tensor(y_off[M][i], (M, N))
        return y_nccl[M][i]
    y_nccl = {M: [torch.empty((world * M, N // world), device=dev) if world > 1 and grp is None else None
                  for N, _ in SHAPES] for M in M_SWEEP}

    # bf16 caches for the wide-batch path (M > 8 goes through the cache GEMM, the reference's
    # own policy for wide batches) and one split-K workspace shared by the in-order launches
    caches = [[miori_b200.dequant4_cache(q, s, b, group=G) for (q, s, b) in projs] for projs in stack]
    ws_bytes = max(lib.miori_gemm_workspace_bytes(M, rows, K)
                   for M in M_SWEEP for N, K in SHAPES for rows in (N, N // world))
    ws = torch.empty(max(ws_bytes // 4, 4), dtype=torch.float32, device=dev)

    def packed_path(M, K):  # the packed-weight GEMV has a fast form (and a fused exchange) here
        return M <= 8 or (M <= 16 and K <= 2048)

    def route(M, rows, K):  # miori_linear4's own rule: 0 packed GEMV, 1 narrow-batch cache kernel, 2 GEMM
        return lib.miori_linear4_route(M, rows, K, 1)

    def run_proj(M, i, w, cache, x, do_split):
        """One projection: on this rank's rows with the result gathered everywhere (split), or whole."""
        N, K = SHAPES[i]
        q, s, b = w
        if not do_split:
            miori_b200.linear4(q, s, b, cache, x, group=G, flags=pdl, out=y_loc[M][i], workspace=ws)
            return
        q, s, b, cache = my_rows(q, N), my_rows(s, N), my_rows(b, N), my_cache_rows(cache, N, K)
        if grp is not None and packed_path(M, K):
            grp.gemv_allgather(4, q, s, b, x, y_off[M][i], rank * (N // world), N, group=G, flags=pdl)
            return
        y = y_part[M][i]
        miori_b200.linear4(q, s, b, cache, x, group=G, flags=pdl, out=y, workspace=ws)
        if grp is not None:
            grp.allgather(y, y_off[M][i], rank * (N // world), N, flags=pdl)
        else:
            dist.all_gather_into_tensor(y_nccl[M][i], y)

    def one_pass(M, plan=None):
        plan = split[M] if plan is None else plan
        for projs, cs in zip(stack, caches):
            for i, (w, c, x) in enumerate(zip(projs, cs, x_dev[M])):
                run_proj(M, i, w, c, x, plan[i])

    # ---- parity of the split path (N > 1, outside every timed region): the last layer's four
    # projections, forced through the row split at M = 1 and M = 32, against the same kernels on
    # the unsplit weights.  The packed-weight GEMV must agree bit for bit; the cache GEMM picks its
    # K split by shape, so its rows agree to fp32 rounding.
    parity = None
    if world > 1:
        cases, worst_gemm, bad = 0, 0.0, []
        for M in (1, 32):
            tmp_off = [grp.alloc(M * N * 4) if grp is not None else None for N, _ in SHAPES]
            for i, (N, K) in enumerate(SHAPES):
                full = stack[-1][i]
                part = tuple(my_rows(t, N) for t in full)
                x = x_dev[M][i]
                want = miori_b200.linear4(*full, caches[-1][i], x, group=G, workspace=ws)
                c_part = my_cache_rows(caches[-1][i], N, K)
                rows = N // world
                if grp is not None and packed_path(M, K):
                    grp.gemv_allgather(4, *part, x, tmp_off[i], rank * rows, N, group=G, flags=pdl)
                    torch.cuda.synchronize()
                    got = grp.tensor(tmp_off[i], (M, N))
                else:
                    yp = miori_b200.linear4(*part, c_part, x, group=G, workspace=ws)
                    if grp is not None:
                        grp.allgather(yp, tmp_off[i], rank * rows, N, flags=pdl)
                        torch.cuda.synchronize()
                        got = grp.tensor(tmp_off[i], (M, N))
                    else:
                        buf = torch.empty((world * M, rows), device=dev)
                        dist.all_gather_into_tensor(buf, yp)
                        got = buf.view(world, M, rows).permute(1, 0, 2).reshape(M, N)
                torch.cuda.synchronize()
                cases += 1
                if M <= 4:  # packed weights on both sides: bit for bit
                    if not torch.equal(got, want):
                        bad.append(f"M={M} N={N} K={K}")
                else:
                    rel = float((got - want).abs().max() / want.abs().max())
                    worst_gemm = max(worst_gemm, rel)
                    if not rel <= 1e-5:
                        bad.append(f"M={M} N={N} K={K} rel={rel:.2e}")
        flag = torch.tensor([len(bad)], device=dev)
        dist.all_reduce(flag)
        parity = {"sharded_vs_single": "bit-exact" if int(flag.item()) == 0 else "MISMATCH",
                  "cases": cases, "gemm_path_max_rel": worst_gemm, "failed": bad}
        if int(flag.item()) != 0:
            print(f"[bench rank {rank}] sharded path differs from the single-GPU kernels: {bad}",
                  file=sys.stderr, flush=True)
        say(f"parity: {parity}")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # ---- one CUDA graph per M.  With --shard auto (N > 1) every candidate split is captured and
    # replayed a few times, and the faster one is kept: the time is the maximum over the ranks, so
    # all ranks keep the same one.  Replicating a projection costs HBM time, splitting it costs an
    # exchange over NVLink; which is cheaper depends on the rows a rank keeps and on M.
    class Eager:
        def __init__(self, M, plan):
            self.M, self.plan = M, plan

        def replay(self):
            one_pass(self.M, self.plan)

    def capture(M, plan):
        one_pass(M, plan)
        torch.cuda.synchronize()
        if args.eager:
            return Eager(M, plan)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            one_pass(M, plan)
        return g

    graphs, tuning = {}, {}
    for M in M_SWEEP:
        best = None
        for plan in candidates:
            g = capture(M, plan)
            if len(candidates) == 1:
                best = (0.0, plan, g)
                break
            # every rank has instantiated this graph before anyone replays it: the kernels' waits for
            # a peer are bounded, and a rank still capturing would look like a missing one
            barrier()
            timed(g.replay, 3)
            ms = timed(g.replay, 10) / 10
            tuning.setdefault(str(M), {})["+".join(f"{K}->{N}" for (N, K), sp in zip(SHAPES, plan) if sp)
                                           or "none"] = ms * 1e3
            if best is None or ms < best[0]:
                best = (ms, plan, g)
        graphs[M], split[M] = best[2], best[1]
    launches_pass = layers * len(SHAPES)
    barrier()

    def kernels_in_pass(M):  # this library's kernel launches in one pass at M rows, on one rank
        n = 0
        for i, (N, K) in enumerate(SHAPES):
            if split[M][i] and grp is not None and packed_path(M, K):
                n += 1                                                    # GEMV with the exchange in its epilogue
                continue
            rows = N // world if split[M][i] else N
            if route(M, rows, K) == 2:
                n += 2 if lib.miori_gemm_workspace_bytes(M, rows, K) else 1   # GEMM (+ K-split sum)
            else:
                n += 1
            n += 1 if (grp is not None and split[M][i]) else 0            # peer all-gather
        return layers * n
    say("graphs captured")

    def step():
        for M in M_SWEEP:
            graphs[M].replay()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(3, args.warmup)):
        step()
    if rank == 0:
        sampler.clear()  # keep only samples taken under load: the timed region and all that follows
    ms_total = timed(step, args.steps)
    ms_step = ms_total / args.steps
    say(f"timed region done: {ms_step:.3f} ms/step")
    value = len(M_SWEEP) * bytes_pass / (ms_step * 1e-3) / 1e9

    # ---- per-M breakdown (each M timed alone, same graphs)
    per_m = {}
    for M in M_SWEEP:
        ms = timed(graphs[M].replay, max(3, args.steps // 2)) / max(3, args.steps // 2)
        per_m[str(M)] = {"ms_per_pass": ms, "gbs": bytes_pass / (ms * 1e-3) / 1e9,
                         "us_per_launch": 1e3 * ms / launches_pass,
                         "path": {f"{K}->{N}": ("packed int4 GEMV", "narrow-batch kernel on the bf16 cache",
                                                "tcgen05 GEMM on the bf16 cache")[route(M, N, K)]
                                  for N, K in SHAPES}}

    # ---- the same M=1 pass with the four projections of a layer on four concurrent streams
    # (no dependency between them): separates kernel throughput from launch-chain latency
    if world == 1 and not args.eager:
        side = [torch.cuda.Stream(device=dev) for _ in SHAPES]
        y_ind = [torch.empty((1, N), device=dev) for N, _ in SHAPES]

        def independent_pass():
            cur = torch.cuda.current_stream()
            for st in side:
                st.wait_stream(cur)
            for projs in stack:
                for (q, s, b), x, y, st in zip(projs, x_dev[1], y_ind, side):
                    with torch.cuda.stream(st):
                        miori_b200.gemv4(q, s, b, x, group=G, flags=pdl, out=y)
            for st in side:
                cur.wait_stream(st)
        independent_pass()
        torch.cuda.synchronize()
        gi = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gi):
            independent_pass()
        ms = timed(gi.replay, max(3, args.steps // 2)) / max(3, args.steps // 2)
        per_m["1"]["four_streams_gbs"] = bytes_pass / (ms * 1e-3) / 1e9
        per_m["1"]["four_streams_note"] = ("same 96 launches, each projection type on its own stream: "
                                           "four independent PDL chains run concurrently")
        say("independent-stream pass done")

    # ---- e2e: host buffers through the C ABI, copies inside the timed region
    stream = torch.cuda.current_stream().cuda_stream
    h2d = d2h = 0
    host_x, host_y, dev_y = {}, {}, {}
    for M in M_SWEEP:
        host_x[M] = x_flat[M].cpu().pin_memory()
        dev_y[M] = [gathered(M, i) for i in range(len(SHAPES))]   # the whole y of every projection
        host_y[M] = [torch.empty(t.shape).pin_memory() for t in dev_y[M]]
        d2h += sum(t.numel() * 4 for t in dev_y[M])
        h2d += host_x[M].numel() * 2

    # a pass's results travel back on a second stream while the next pass runs: the host waits for
    # pass i only after it has enqueued pass i + 1 (what a decode loop with two batches in flight does)
    back = torch.cuda.Stream(device=dev)
    computed = {M: torch.cuda.Event() for M in M_SWEEP}
    landed = {M: torch.cuda.Event() for M in M_SWEEP}

    def e2e_step():
        prev = None
        for M in M_SWEEP:
            check(lib.miori_memcpy_h2d(x_flat[M].data_ptr(), host_x[M].data_ptr(),
                                       host_x[M].numel() * 2, stream))
            graphs[M].replay()
            computed[M].record()
            back.wait_event(computed[M])
            for hy, dy in zip(host_y[M], dev_y[M]):
                check(lib.miori_memcpy_d2h(hy.data_ptr(), dy.data_ptr(), hy.numel() * 4, back.cuda_stream))
            landed[M].record(back)
            if prev is not None:
                landed[prev].synchronize()  # the host consumes the previous pass's result
            prev = M
        landed[prev].synchronize()

    say("per-M breakdown done")
    e2e_step()
    ms_e2e = timed(e2e_step, args.steps) / args.steps
    e2e_val = len(M_SWEEP) * bytes_pass / (ms_e2e * 1e-3) / 1e9

    peaks, peak_kind = measured_peaks()
    m1 = per_m["1"]
    # DRAM bytes (read + write) per algorithmic byte of gemv_tma_kernel, from an ncu capture of
    # the N=8192, K=2048, M=1 launch over a pool larger than L2 (9.465 MB read, nothing written --
    # the 32 KB of y stay in L2 -- for 9.437 MB of weights); traffic grows in proportion to the
    # weights a launch streams
    DRAM_PER_ALGO_BYTE = 1.003
    roofline = {
        "kernel": "gemv_tma_kernel<4,exact,1> (M=1 pass of the stack, 96 launches per pass)",
        "bound": "hbm", "achieved": m1["gbs"] / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
        "frac": m1["gbs"] / world / peaks["hbm_gbs"], "peak_kind": peak_kind,
        "bytes_per_launch": bytes_pass / launches_pass / world,
        "us_per_launch": m1["us_per_launch"],
        "traffic": DRAM_PER_ALGO_BYTE * bytes_pass / launches_pass / world,
    }
    out = {
        "metric": METRIC, "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(args), "collective": gather,
        "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e},
        "gpu_launches": args.steps * sum(kernels_in_pass(M) for M in M_SWEEP),
        "per_m": per_m, "roofline": roofline,
        "sharding": {"mode": args.shard if world > 1 else "single GPU", "threshold_bytes": args.shard_bytes,
                     "weights": "replicated; a split projection reads only its own rows",
                     "split_per_m": {str(M): [f"{K}->{N}" for (N, K), sp in zip(SHAPES, split[M]) if sp]
                                     for M in M_SWEEP},
                     "candidates_us_per_pass": tuning},
    }
    if parity is not None:
        out["parity"] = parity

    if rank == 0 and not args.no_extras and world == 1:
        out["extras"] = extras(torch, miori_b200, synth, dev, G, peaks, timed)
    if not args.no_extras and grp is not None:
        c1 = config1_sharded(torch, miori_b200, synth, dev, G, peaks, timed, rank, world, grp)
        if rank == 0:
            out.setdefault("extras", {})["config1_gemv8_sharded"] = c1
    if not args.no_extras:
        # every rank takes part: the large prefill GEMM is sharded by token rows, no collective
        c4 = config4_prefill(torch, miori_b200, synth, dev, G, peaks, timed, rank, world)
        if rank == 0:
            out.setdefault("extras", {})["config4_prefill_gemm_m131072"] = c4
    if rank == 0:
        # the sampler ran through the timed region, the per-M passes, the end-to-end leg and the extras
        out["clocks"] = sampler.stop()
    if rank == 0 and not args.no_cpu:
        out["cpu_baseline"] = cpu_decode_sample(G, seconds=12.0)
        out["cpu_baseline"].pop("seconds", None)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if parity is not None and parity["sharded_vs_single"] != "bit-exact":
        sys.stdout.flush()
        os._exit(3)
    if world > 1:
        # Captured graphs hold NCCL work and tearing the communicator down under them can block;
        # every rank has finished the same work here, so leave without the teardown.
        torch.cuda.synchronize()
        if grp is not None:
            try:
                grp.status()
            except Exception as e:
                print(f"[bench rank {rank}] {e}", file=sys.stderr, flush=True)
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def config1_sharded(torch, miori_b200, synth, dev, G, peaks, timed, rank, world, grp):
    """The 8-bit head (N=131072, K=2048, M=1, bf16 logits) with its rows split over the ranks.
    Three ways to finish: the logits gathered on every rank by the GEMV's own epilogue; or -- for
    greedy sampling -- only each rank's best (value, index) exchanged (two 8-byte packets per rank),
    by a second kernel after the GEMV or by the GEMV's own epilogue.  Every rank cycles through a
    pool of distinct shards larger than L2; GB/s counts the whole matrix."""
    import torch.distributed as dist
    N, K = 131072, 2048
    rows = N // world
    shard_bytes = packed_bytes(rows, K, 8, G)
    npool = max(2, -(-(300 << 20) // shard_bytes))
    pool = []
    for i in range(npool):  # same seeds on every rank: shard `rank` of matrix i
        g = torch.Generator(device=dev).manual_seed(4000 + i * 64 + rank)
        q = torch.randint(-2**31, 2**31 - 1, (rows, K // 4), generator=g, device=dev, dtype=torch.int64).to(torch.int32)
        sc = (torch.rand((rows, K // G), generator=g, device=dev) * 1e-3 + 1e-4).to(torch.bfloat16)
        bi = (torch.rand((rows, K // G), generator=g, device=dev) * -0.1).to(torch.bfloat16)
        pool.append((q, sc, bi))
    x = synth.make_activation(1, K, seed=9, device=dev)
    off = grp.alloc(N * 2)
    off_best = grp.alloc(256)
    off_own, off_pick = grp.alloc(N * 2), grp.alloc(256)
    y_local = torch.empty((1, rows), dtype=torch.bfloat16, device=dev)
    flags = miori_b200.LAUNCH_PDL | miori_b200.OUT_BF16
    by = packed_bytes(N, K, 8, G)

    def run_gather():
        for q, sc, bi in pool:
            grp.gemv_allgather(8, q, sc, bi, x, off, rank * rows, N, group=G, flags=flags)

    def run_argmax():
        for q, sc, bi in pool:
            miori_b200.gemv8(q, sc, bi, x, group=G, flags=flags, out=y_local)
            grp.argmax_allreduce(y_local.view(-1), rank * rows, off_best, flags=miori_b200.LAUNCH_PDL)

    def run_fused():
        for q, sc, bi in pool:
            grp.gemv_argmax(8, q, sc, bi, x, off_own, off_pick, rank * rows, N, group=G, flags=flags)

    out = {"n_gpus": world, "rows_per_gpu": rows, "pool": npool, "out": "bf16"}
    for name, run in (("gather_logits", run_gather), ("exchange_argmax", run_argmax),
                      ("argmax_in_the_gemv_epilogue", run_fused)):
        run()
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            run()
        torch.cuda.synchronize()
        dist.barrier()
        ms = timed(g.replay, 10) / 10 / npool
        out[name] = {"us": 1e3 * ms, "gbs": by / (ms * 1e-3) / 1e9,
                     "frac_of_hbm_peak": by / (ms * 1e-3) / 1e9 / (world * peaks["hbm_gbs"])}
    # the exchanged winner must be the arg-max of the gathered logits of the last matrix (ties: lowest index)
    torch.cuda.synchronize()
    logits = grp.tensor(off, (N,), torch.bfloat16).float()
    want = int(torch.argmax((logits == logits.max()).to(torch.int8)).item())
    got_i, got_v = grp.argmax_result(off_best)
    out["argmax_matches_gathered_logits"] = bool(got_i == want and got_v == float(logits.max()) and
                                                 grp.gemv_argmax_result(off_pick) == (got_i, got_v))
    out["us"], out["gbs"], out["frac_of_hbm_peak"] = (out["gather_logits"][k] for k in ("us", "gbs", "frac_of_hbm_peak"))
    out["how"] = ("CUDA graph of dependent launches over a pool of distinct shards (> L2 per rank); "
                  "gather_logits ends with the whole logits vector on every rank, exchange_argmax (GEMV, then "
                  "a second kernel) and argmax_in_the_gemv_epilogue (one launch) with the winning (value, index) "
                  "pair on every rank")
    return out


def config4_prefill(torch, miori_b200, synth, dev, G, peaks, timed, rank, world):
    """Prefill configuration: 64 prompts x 2048 tokens = 131072 rows through the four projection
    shapes, token rows split evenly over the ranks, bf16 cache replicated, no collective.
    `timed` brackets with barriers and takes the max over ranks; TFLOP/s is the whole job's."""
    M_total = 131072
    M = M_total // world
    flags = miori_b200.LAUNCH_PDL | miori_b200.OUT_BF16
    per, tot_flop, tot_ms = {}, 0.0, 0.0
    for N, K in GEMM_SHAPES:
        q, s, b = synth.make_weight(N, K, 4, G, seed=900 + N + K, device=dev)
        cache = miori_b200.dequant4_cache(q, s, b, group=G)
        del q, s, b
        # this rank's token rows: seeded per rank, standard normal like every activation here
        g = torch.Generator(device=dev).manual_seed(7000 + rank)
        A = torch.randn((M, K), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        Cm = torch.empty((M, N), device=dev, dtype=torch.bfloat16)

        def run():
            miori_b200.gemm_bf16_cache(A, cache, N, flags=flags, out=Cm)
        run()
        ms = timed(run, 5) / 5
        fl = 2.0 * M_total * N * K
        per[f"N{N}_K{K}"] = {"ms": ms, "tflops": fl / (ms * 1e-3) / 1e12}
        tot_flop += fl
        tot_ms += ms
        del A, Cm, cache
    tf = tot_flop / (tot_ms * 1e-3) / 1e12
    return {"tflops": tf, "frac_of_bf16_peak": tf / (world * peaks["bf16_tflops"]),
            "frac_of_bf16_sustained": tf / (world * peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])),
            "peak_used": "n_gpus x the measured burst / sustained cuBLAS bf16 figures (kernels of "
                         "milliseconds run under the power cap, so the sustained one applies)",
            "rows_per_gpu": M, "n_gpus": world, "per_shape": per, "out": "bf16",
            "how": "each rank multiplies its M/n_gpus rows by the replicated cache; CUDA events, "
                   "max over ranks; A (0.5-2.1 GB) and C (up to 4.3 GB) are far larger than L2"}


def extras(torch, miori_b200, synth, dev, G, peaks, timed):
    """Secondary measurements on one GPU: config 0 (rotating pool), config 1 (int8 head),
    config 3 (prefill GEMM M=1024) and the cache build."""
    ex = {}
    flags = miori_b200.LAUNCH_PDL
    # config 0: gemv4 M=1 K=2048 N=8192 over a rotating pool of 32 distinct matrices (302 MB > L2)
    N, K = 8192, 2048
    pool = [synth.make_weight(N, K, 4, G, seed=900 + i, device=dev) for i in range(32)]
    x = synth.make_activation(1, K, seed=1, device=dev)
    y = torch.empty((1, N), device=dev)
    for q, s, b in pool:
        miori_b200.gemv4(q, s, b, x, group=G, flags=flags, out=y)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for q, s, b in pool:
            miori_b200.gemv4(q, s, b, x, group=G, flags=flags, out=y)
    ms = timed(g.replay, 20) / 20
    by = packed_bytes(N, K, 4, G)
    ex["config0_gemv4_m1_n8192_k2048"] = {
        "us_per_launch": 1e3 * ms / len(pool), "gbs": by * len(pool) / (ms * 1e-3) / 1e9,
        "frac_of_hbm_peak": by * len(pool) / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
        "how": "CUDA graph of 32 PDL launches over 32 distinct weight matrices (302 MB)"}
    del pool
    # config 1: gemv8 M=1 K=2048 N=131072
    N, K = 131072, 2048
    q, s, b = synth.make_weight(N, K, 8, G, seed=77, device=dev)
    y = torch.empty((1, N), device=dev)
    ms = timed(lambda: miori_b200.gemv8(q, s, b, x, group=G, out=y), 20) / 20
    by = packed_bytes(N, K, 8, G)
    ex["config1_gemv8_m1_n131072_k2048"] = {"us": 1e3 * ms, "gbs": by / (ms * 1e-3) / 1e9,
                                            "frac_of_hbm_peak": by / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    # the same head followed by the greedy pick: two launches (gemv8, then arg-max) against one
    # (the arg-max in the GEMV's epilogue), bf16 logits, both as replayed graphs of dependent launches
    from miori_b200.peers import PeerGroup
    grp1 = PeerGroup(0, 1, 1 << 20, dev)
    off_y, off_b = grp1.alloc(N * 2), grp1.alloc(256)
    yb = torch.empty((1, N), dtype=torch.bfloat16, device=dev)
    hf = flags | miori_b200.OUT_BF16

    def two_launches():
        miori_b200.gemv8(q, s, b, x, group=G, flags=hf, out=yb)
        return miori_b200.argmax(yb.view(-1), flags=flags)

    def one_launch():
        grp1.gemv_argmax(8, q, s, b, x, off_y, off_b, 0, N, group=G, flags=hf)
    pick = {}
    for name, fn in (("gemv8_then_argmax", two_launches), ("argmax_in_the_gemv_epilogue", one_launch)):
        res = fn()
        torch.cuda.synchronize()
        gg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gg):
            for _ in range(4):
                fn()
        pick[name + "_us"] = 1e3 * timed(gg.replay, 10) / 10 / 4
        if res is not None:
            pick["index"] = int(res[0].item())
    torch.cuda.synchronize()
    pick["same_token"] = grp1.gemv_argmax_result(off_b)[0] == pick.pop("index")
    ex["config1_gemv8_m1_n131072_k2048"]["greedy_pick"] = pick
    grp1.close()
    del q, s, b
    # long stream of 4-bit weights: M=1 over two distinct 151 MB matrices (N=131072, K=2048) -- the
    # kernel's rate once the fixed cost of a launch is amortised
    N, K = 131072, 2048
    big = [synth.make_weight(N, K, 4, G, seed=300 + i, device=dev) for i in range(2)]
    y = torch.empty((1, N), device=dev)

    def run_stream():
        for q, s, b in big:
            miori_b200.gemv4(q, s, b, x, group=G, flags=flags, out=y)
    run_stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run_stream()
    ms = timed(g.replay, 10) / 10 / len(big)
    by = packed_bytes(N, K, 4, G)
    ex["stream_gemv4_m1_n131072_k2048"] = {"us": 1e3 * ms, "gbs": by / (ms * 1e-3) / 1e9,
                                           "frac_of_hbm_peak": by / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                           "kernel": "gemv_umma_kernel<4,1> (tcgen05.mma.kind::i8), two CTAs per SM"}
    del big
    # RMSNorm in front of a projection: norm kernel + GEMV against the GEMV with the norm fused into
    # its activation staging, M=1, one layer's four shapes over pools of distinct weights (> L2)
    fused = {}
    for N, K in SHAPES:
        npool = max(2, min(24, (300 << 20) // packed_bytes(N, K, 4, G)))
        pool = [synth.make_weight(N, K, 4, G, seed=700 + i, device=dev) for i in range(npool)]
        xf = torch.randn((1, K), device=dev)
        gam = torch.ones(K, dtype=torch.bfloat16, device=dev)
        xn = torch.empty((1, K), dtype=torch.bfloat16, device=dev)
        y = torch.empty((1, N), device=dev)

        def two_kernels():
            for q, s, b in pool:
                miori_b200.rmsnorm(xf, gam, 1e-5, flags=flags, out=xn)
                miori_b200.gemv4(q, s, b, xn, group=G, flags=flags, out=y)

        def one_kernel():
            for q, s, b in pool:
                miori_b200.gemv4_rmsnorm(q, s, b, xf, gam, 1e-5, group=G, flags=flags, out=y)

        def one_kernel_tcgen05():
            for q, s, b in pool:
                miori_b200.gemv4_rmsnorm(q, s, b, xf, gam, 1e-5, group=G, flags=flags | 0x100000, out=y)
        res = {}
        for name, fn in (("norm_then_gemv_us", two_kernels), ("fused_us", one_kernel),
                         ("fused_tcgen05_us", one_kernel_tcgen05)):
            fn()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            res[name] = 1e3 * timed(g.replay, 10) / 10 / npool
        fused[f"N{N}_K{K}"] = res
        del pool
    ex["rmsnorm_fusion_m1"] = {"per_projection": fused,
                               "layer_norm_then_gemv_us": sum(v["norm_then_gemv_us"] for v in fused.values()),
                               "layer_fused_us": sum(v["fused_us"] for v in fused.values()),
                               "how": "CUDA graphs of PDL launches; the unfused pair is the default GEMV after "
                                      "miori_rmsnorm, the fused one miori_gemv4_rmsnorm (by default the TMA + mma.sync "
                                      "kernel with the norm in its staging pass; the tcgen05 kernel when forced)"}
    # SiLU x up behind the fused gate + up projection (2048 -> 2 x 8192): GEMV + activation kernel
    # against the GEMV with the activation as its epilogue, over a pool of distinct weights (> L2)
    N, K = 16384, 2048
    pool = [synth.make_weight(N, K, 4, G, seed=800 + i, device=dev) for i in range(24)]
    gated = {}
    for M in (1, 4, 8, 16):
        xg = synth.make_activation(M, K, seed=5, device=dev)
        yf = torch.empty((M, N), device=dev)
        act = torch.empty((M, N // 2), dtype=torch.bfloat16, device=dev)

        g1 = torch.empty((M, N // 2), device=dev)
        u1 = torch.empty((M, N // 2), device=dev)

        def three_launches():  # the reference's structure: w1, w3, then the activation (src/engine.cpp)
            for q, s, b in pool:
                miori_b200.gemv4(q[:N // 2], s[:N // 2], b[:N // 2], xg, group=G, flags=flags, out=g1)
                miori_b200.gemv4(q[N // 2:], s[N // 2:], b[N // 2:], xg, group=G, flags=flags, out=u1)
                miori_b200.silu_mul(g1, u1, flags=flags, out=act)

        def two_launches():  # one row only: gate and up are the two halves of the fused projection's row
            for q, s, b in pool:
                miori_b200.gemv4(q, s, b, xg, group=G, flags=flags, out=yf)
                miori_b200.silu_mul(yf[0, :N // 2], yf[0, N // 2:], flags=flags, out=act[0])

        def gated_gemv():
            for q, s, b in pool:
                miori_b200.gemv4_silu(q, s, b, xg, group=G, flags=flags, out=act)
        res = {}
        for name, fn in (("w1_w3_silu_mul_us", three_launches), ("gate_up_silu_mul_us", two_launches),
                         ("fused_us", gated_gemv)):
            if fn is two_launches and M > 1:
                continue
            fn()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            res[name] = 1e3 * timed(g.replay, 10) / 10 / len(pool)
        gated[f"M{M}"] = res
    del pool
    ex["silu_fusion_gate_up"] = {"per_m": gated,
                                 "how": "CUDA graphs of PDL launches; miori_gemv4 on w1 and on w3 then miori_silu_mul (three "
                                        "launches), miori_gemv4 on the fused weights then miori_silu_mul (two, one row), "
                                        "and miori_gemv4_silu (TMA + mma.sync kernel, gated epilogue)"}
    # post_norm_add behind the o and w2 projections (M = 1): GEMV + norm kernel against the GEMV with the
    # norm as its epilogue, over pools of distinct weights (> L2)
    post = {}
    for N, K in ((2048, 2048), (2048, 8192)):
        npool = max(2, min(24, (300 << 20) // packed_bytes(N, K, 4, G)))
        pool = [synth.make_weight(N, K, 4, G, seed=850 + i, device=dev) for i in range(npool)]
        xg = synth.make_activation(1, K, seed=6, device=dev)
        resid = torch.randn((1, N), device=dev)
        gam = torch.ones(N, dtype=torch.bfloat16, device=dev)
        v = torch.empty((1, N), device=dev)
        o = torch.empty((1, N), device=dev)
        counter = torch.zeros(1, dtype=torch.int32, device=dev)

        def gemv_then_norm():
            for q, s, b in pool:
                miori_b200.gemv4(q, s, b, xg, group=G, flags=flags, out=v)
                miori_b200.post_norm_add(resid, v, gam, 1e-5, flags=flags, out=o)

        def norm_in_epilogue():
            for q, s, b in pool:
                miori_b200.gemv4_post_norm_add(q, s, b, xg, resid, gam, 1e-5, counter, group=G, flags=flags, out=o)
        res = {}
        for name, fn in (("gemv_then_post_norm_add_us", gemv_then_norm), ("fused_us", norm_in_epilogue)):
            fn()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            res[name] = 1e3 * timed(g.replay, 10) / 10 / npool
        post[f"N{N}_K{K}"] = res
        del pool
    ex["post_norm_add_fusion_m1"] = {"per_projection": post,
                                     "how": "CUDA graphs of PDL launches; miori_gemv4 then miori_post_norm_add against "
                                            "miori_gemv4_post_norm_add (the last CTA to finish normalises the rows)"}
    # One decode layer at M = 1 with its neighbours (attention left out: o reads a fixed vector), 24
    # layers of distinct weights in one graph: the reference's ten launches per layer, eight with SiLU x up
    # in the gate + up GEMV, seven with qkv's norm in its GEMV's staging, six with the other input norm in
    # front of the gated GEMV too (the post-norms stay kernels: fused they measured slower)
    H, QKV, FF = 2048, 3072, 8192
    layers = [[synth.make_weight(n, k, 4, G, seed=9000 + 4 * i + j, device=dev)
               for j, (n, k) in enumerate(((QKV, H), (H, H), (2 * FF, H), (H, FF)))] for i in range(24)]
    hid = torch.randn((1, H), device=dev)
    gam = torch.ones(H, dtype=torch.bfloat16, device=dev)
    xn = torch.empty((1, H), dtype=torch.bfloat16, device=dev)
    attn = synth.make_activation(1, H, seed=8, device=dev)
    qkv = torch.empty((1, QKV), device=dev)
    proj = torch.empty((1, H), device=dev)
    h2 = torch.empty((1, H), device=dev)
    h3 = torch.empty((1, H), device=dev)
    gate = torch.empty((1, FF), device=dev)
    up = torch.empty((1, FF), device=dev)
    act = torch.empty((1, FF), dtype=torch.bfloat16, device=dev)

    def layer(wq, wo, wgu, wd, fuse):
        if fuse >= 2:
            miori_b200.gemv4_rmsnorm(*wq, hid, gam, 1e-5, group=G, flags=flags, out=qkv)
        else:
            miori_b200.rmsnorm(hid, gam, 1e-5, flags=flags, out=xn)
            miori_b200.gemv4(*wq, xn, group=G, flags=flags, out=qkv)
        miori_b200.gemv4(*wo, attn, group=G, flags=flags, out=proj)
        miori_b200.post_norm_add(hid, proj, gam, 1e-5, flags=flags, out=h2)
        if fuse == 3:
            miori_b200.gemv4_rmsnorm_silu(*wgu, h2, gam, 1e-5, group=G, flags=flags, out=act)
        else:
            miori_b200.rmsnorm(h2, gam, 1e-5, flags=flags, out=xn)
        if fuse == 3:
            pass
        elif fuse:
            miori_b200.gemv4_silu(*wgu, xn, group=G, flags=flags, out=act)
        else:
            q, s, b = wgu
            miori_b200.gemv4(q[:FF], s[:FF], b[:FF], xn, group=G, flags=flags, out=gate)
            miori_b200.gemv4(q[FF:], s[FF:], b[FF:], xn, group=G, flags=flags, out=up)
            miori_b200.silu_mul(gate, up, flags=flags, out=act)
        miori_b200.gemv4(*wd, act, group=G, flags=flags, out=proj)
        miori_b200.post_norm_add(h2, proj, gam, 1e-5, flags=flags, out=h3)
    res = {}
    for name, fuse in (("ten_launches_us", 0), ("eight_launches_us", 1), ("seven_launches_us", 2), ("six_launches_us", 3)):
        def run():
            for ws in layers:
                layer(*ws, fuse)
        run()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            run()
        res[name] = 1e3 * timed(g.replay, 10) / 10 / len(layers)
    del layers
    ex["decode_layer_m1_with_neighbours"] = dict(res, how="us per layer; rmsnorm, qkv, o, post_norm_add, rmsnorm, w1, w3, "
                                                 "silu_mul, w2, post_norm_add; with miori_gemv4_silu in place of w1, w3, "
                                                 "silu_mul (eight); with miori_gemv4_rmsnorm for qkv as well (seven); with "
                                                 "miori_gemv4_rmsnorm_silu for the gate + up projection too (six); "
                                                 "CUDA graph of PDL launches")
    # config 3: prefill GEMM M=1024 on the bf16 cache + cache build.  Each shape runs over a
    # pool of distinct caches larger than L2 (weights come from HBM, as in a real prefill where
    # consecutive layers evict each other), one CUDA graph of PDL launches per shape.
    M = 1024
    tot_flop, tot_ms, per = 0.0, 0.0, {}
    A_by_k = {}
    for N, K in GEMM_SHAPES:
        npool = max(2, (300 << 20) // (N * K * 2))
        pool = []
        ms_c = 0.0
        for i in range(npool):
            q, s, b = synth.make_weight(N, K, 4, G, seed=N + K + i, device=dev)
            cache = miori_b200.dequant4_cache(q, s, b, group=G)
            if i == 0:
                ms_c = timed(lambda: miori_b200.dequant4_cache(q, s, b, group=G, out=cache), 10) / 10
            pool.append(cache)
            del q, s, b
        A = A_by_k.setdefault(K, synth.make_activation(M, K, seed=3, device=dev))
        Cm = torch.empty((M, N), device=dev, dtype=torch.bfloat16)  # fp32 accumulation, bf16 out
        ws = miori_b200.gemm_workspace(M, N, K, dev)

        def run():
            for c in pool:
                miori_b200.gemm_bf16_cache(A, c, N, flags=flags | miori_b200.OUT_BF16, out=Cm,
                                           workspace=ws)
        run()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            run()
        ms = timed(g.replay, 10) / 10 / npool
        fl = 2.0 * M * N * K
        per[f"N{N}_K{K}"] = {"us": 1e3 * ms, "tflops": fl / (ms * 1e-3) / 1e12, "pool": npool,
                             "cache_build_gbs": (packed_bytes(N, K, 4, G) + 2 * N * K) / (ms_c * 1e-3) / 1e9}
        tot_flop += fl
        tot_ms += ms
        del pool, Cm, g
    ex["config3_prefill_gemm_m1024"] = {
        "tflops": tot_flop / (tot_ms * 1e-3) / 1e12,
        "frac_of_bf16_peak": tot_flop / (tot_ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
        "per_shape": per, "out": "bf16",
        "how": "per shape a CUDA graph over a pool of distinct bf16 caches (> L2), A L2-resident"}
    return ex


if __name__ == "__main__":
    main()
