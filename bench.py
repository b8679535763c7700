"""Benchmark of the EXL3 quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (`config.workload`): the dense 27B-shape decode layer set at K = 3 bpw, 3INST codebook, batch 1 --
64 layers x (q|k|v 5120->7168, o 5120->5120, gate|up 5120->34816, down 17408->5120) = 7.93 GB of packed
trellis, uniform-random bits, random +-1 suh/svh, fp16 N(0,1) activations.  One step = every linear of the stack
once (the linear work of one decoded token).  The weights are distinct per layer and far larger than L2, so no
L2 flush is needed between steps.

Printed metric: achieved HBM GB/s on packed-weight bytes, whole job (all ranks), plus tokens/s.  With N > 1 the
stack is tensor-parallel (column-parallel q/k/v/gate/up, row-parallel o/down with an all-reduce), total work
fixed: "strong" scaling.

`--impl reference` times the CPU implementation of the same path (the oracle port of the reference decoder,
multi-threaded C) on a bounded sample: the seven matrices of one layer.

The timed region is repeated in BLOCKS of `--steps` steps (each block bracketed by a barrier and a synchronise); the
median block gives `ms_per_step`, and the clock sampler sees seconds of load instead of a tenth of one.
Secondary workloads: `--workload c1` (one 4096x4096 K=4 3INST linear at batch 1 over a ring of distinct matrices larger
than L2), `--workload prefill`, `--workload moe`.  The default line also carries `sweep` (batch 4 / 16 of the same step,
and K = 2..8 on the 17408x5120 shape), measured outside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "exl3_gemv_hbm_gbs_packed_bytes_batch1_27b_k3"
UNIT = "GB/s"
WORKLOAD = "27B-shape decode layer set, K=3 3INST, batch 1, 64 layers x (qkv, o, gate_up, down), inputs > L2 (no flush)"


def measured_peak_hbm() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.first = index, [], None, 0

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            deadline = time.time() + 5.0                 # nvidia-smi needs a moment before its first row
            while not self.rows and time.time() < deadline:
                time.sleep(0.02)
            self.first = len(self.rows)
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        self.rows = self.rows[max(self.first - 1, 0):]   # keep the rows sampled while the timed region ran
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def cpu_sample(K: int, codebook: int, min_seconds: float = 8.0, max_reps: int = 4, threads: int | None = None) -> dict:
    """Oracle forward (decode + multiply fused, OpenMP) on the seven matrices of one 27B-shape layer, batch 1."""
    import numpy as np
    from oracle import exl3_oracle as orc
    # All usable host cores, whatever OMP_NUM_THREADS says (torchrun sets it to 1 for its workers).
    orc.set_threads(threads or len(os.sched_getaffinity(0)))
    shapes = [(5120, 5120), (5120, 1024), (5120, 1024), (5120, 5120), (5120, 17408), (5120, 17408), (17408, 5120)]
    rng = np.random.default_rng(100)
    mats = []
    for k, n in shapes:
        tr = rng.integers(0, 65536, size=(k // 16, n // 16, 16 * K), dtype=np.uint16)
        suh = (rng.integers(0, 2, size=k) * 2 - 1).astype(np.float16)
        svh = (rng.integers(0, 2, size=n) * 2 - 1).astype(np.float16)
        x = rng.standard_normal((1, k)).astype(np.float16)
        mats.append((x, tr, suh, svh))
    nbytes = sum(k * n * K // 8 for k, n in shapes)
    orc.c_linear_forward(*mats[1], K, codebook)                      # warm the thread pool
    times = []
    t_all = time.perf_counter()
    while len(times) < max_reps and (time.perf_counter() - t_all < min_seconds or not times):
        t0 = time.perf_counter()
        for m in mats:
            orc.c_linear_forward(*m, K, codebook)
        times.append(time.perf_counter() - t0)
    best = min(times)
    return {"value": nbytes / best / 1e9, "unit": UNIT, "cores": orc.num_threads(), "kind": "port",
            "sample": f"one 27B-shape layer (7 matrices, {nbytes / 1e6:.2f} MB packed, K={K}, batch 1), best of {len(times)} passes, "
                      f"{best:.3f} s per pass; multi-threaded C port of the reference decoder (the reference itself is Python)",
            "seconds_per_layer": best, "tok_s": 1.0 / (best * 64)}


BLOCKS = 10          # timed blocks of `--steps` steps; the median block is reported


def workload_config(args, world: int, total_bytes: float) -> dict:
    """The `config` object: identical in the repo's arm and the reference arm for the same command line."""
    return {"workload": WORKLOAD, "layers": args.layers, "bits": args.bits, "codebook": "3inst", "rows": args.rows,
            "parallelism": f"tp{world}", "allreduce": (args.allreduce if world > 1 else None),
            "l2": "inputs larger than L2, no flush", "packed_bytes_per_step": total_bytes}


def packed_bytes_per_step(layers: int, K: int) -> float:
    weights = 5120 * (5120 + 2 * 1024) + 5120 * 5120 + 3 * 5120 * 17408
    return float(layers * weights * K // 8)


def traffic_ratio() -> tuple[float | None, str]:
    """DRAM bytes moved per algorithmic byte of the dominant kernel, from the ncu capture whose figures sit beside its
    summary (read + write of one gate|up launch over its packed-weight bytes)."""
    path = os.path.join(ROOT, "profiles", "gemv_kernel_27b_k3_batch1.traffic.json")
    if not os.path.exists(path):
        return None, "no capture recorded"
    with open(path) as f:
        t = json.load(f)
    return (t["dram_bytes_read"] + t["dram_bytes_write"]) / t["algorithmic_bytes"], t.get("source", path)


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    K, cb = args.bits, 0
    runs = []
    for _ in range(args.warmup):
        cpu_sample(K, cb, min_seconds=0.0, max_reps=1)
    for _ in range(args.steps):
        runs.append(cpu_sample(K, cb, min_seconds=0.0, max_reps=1))
    best = max(runs, key=lambda r: r["value"])
    # One step of the workload is `layers` layers; the sample timed one layer, every layer costs the same.
    ms = best["seconds_per_layer"] * 1e3 * args.layers
    line = {"impl": "reference", "metric": METRIC, "value": best["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, args.gpus, packed_bytes_per_step(args.layers, K)),
            "ms_per_step_note": f"{args.layers} x the measured time of one layer ({best['seconds_per_layer'] * 1e3:.1f} ms)",
            "cpu_baseline": {k: best[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": best["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "tok_s": 1e3 / ms, "gpu_launches": 0}
    print(json.dumps(line))


def run_prefill(args) -> None:
    """Secondary workload: the four fused groups of one 27B-shape layer at M = 2048 rows, K = 4, MCG codebook, through the
    fused tcgen05 kernel.  One step = one layer.  Tensor-pipe roofline."""
    import torch
    from trellis_serve_b200.kernels import linear as lin
    from trellis_serve_b200.runtime.layerset import random_packed, random_signs
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(200)
    K, cb, rows = 4, 1, args.rows if args.rows > 1 else 2048
    shapes = [(5120, [5120, 1024, 1024]), (5120, [5120]), (5120, [17408, 17408]), (17408, [5120])]
    groups = []
    for k, ns in shapes:
        packed = torch.cat([random_packed(k, n, K, gen, dev) for n in ns])
        ends = [sum(ns[:i + 1]) for i in range(len(ns) - 1)]
        x = torch.randn((rows, k), device=dev, generator=gen).half()
        groups.append((x, packed, random_signs(k, gen, dev, len(ns)), random_signs(sum(ns), gen, dev).view(-1), ends,
                       torch.empty((rows, sum(ns)), dtype=torch.float16, device=dev)))
    flops = sum(2.0 * rows * k * sum(ns) for k, ns in shapes)

    def step():
        for x, packed, suh, svh, ends, out in groups:
            lin.run_tc(x, packed, suh, svh, ends, cb, out=out)
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clocks:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    lin.device_error(dev)
    peak = 1648.3
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        peak = float(json.load(open(path))["bf16_tflops"])
    tf = flops / ms / 1e9
    print(json.dumps({"metric": "exl3_prefill_tflops_27b_layer_m2048_k4_mcg", "value": tf, "unit": "TFLOP/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                      "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                      "config": {"workload": f"one 27B-shape layer (qkv, o, gate_up, down), {rows} rows, K=4 MCG, fused tcgen05 GEMM",
                                 "rows": rows, "l2": "weights 165 MB per layer, larger than L2"},
                      "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                                   # DRAM bytes of the largest launch (gate|up at 2048 rows) from one ncu capture
                                   "traffic": 264.6e6 if rows == 2048 else None,
                                   "traffic_unit": "bytes of the gate|up launch, one ncu capture",
                                   "traffic_source": "profiles/gemm_tc_pair_kernel_27b_prefill_m2048_k4.md",
                                   "peak_source": "of measured (burst)", "kernel": "gemm_tc_pair_kernel"},
                      # per layer: 4 input rotations, 4 GEMMs, 3 rotations of cut tiles (q|k|v has none on 74 CTA pairs)
                      "gpu_launches": 11 * args.steps, "clocks": clocks.summary()}))


def run_moe(args) -> None:
    """Secondary workload: one MoE layer, hidden 2048, 256 experts, intermediate 512, top-8, K = 3, softmax-of-N(0,1)
    routing, captured in a CUDA graph.  GB/s on the packed bytes of the distinct routed experts."""
    import torch
    from trellis_serve_b200 import _lib
    from trellis_serve_b200.kernels import moe
    from trellis_serve_b200.runtime.layerset import random_packed, random_signs
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    _lib.init_device(0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(300)
    E, H, I, top_k, K, cb = 256, 2048, 512, 8, 3, 0
    T = args.rows
    w13 = torch.stack([torch.cat([random_packed(H, I, K, gen, dev), random_packed(H, I, K, gen, dev)]) for _ in range(E)])
    w2 = torch.stack([random_packed(I, H, K, gen, dev) for _ in range(E)])
    pack = moe.ExpertPack(w13, w2, random_signs(H, gen, dev, E * 2).view(E, 2, H), (random_signs(2 * I, gen, dev, E) / 32).half(),
                          random_signs(I, gen, dev, E), (random_signs(H, gen, dev, E) / 32).half(), cb, H, I, E, K)
    wts, ids = torch.topk(torch.softmax(torch.randn((T, E), device=dev, generator=gen), -1), top_k)
    wts, ids = (wts / wts.sum(-1, keepdim=True)).float(), ids.int()
    x = torch.randn((T, H), device=dev, generator=gen).half()
    out = torch.empty_like(x)
    if args.moe_path != "auto":           # measurement knob: force one path to find the crossover
        moe.TC_ROWS_PER_EXPERT = 0 if args.moe_path == "tc" else 1 << 30
    tensor_core = moe.moe_block_size(T, top_k, E) == 128
    if tensor_core:
        # many rows per expert: the allocation-free layer entry, which sends the class through the grouped tcgen05 GEMM
        mixed = moe.MixedPack([pack], [torch.arange(E, dtype=torch.int32, device=dev)], E, H, I, cb)
        ws = torch.zeros(moe.layer_workspace_bytes([E], H, I, cb, T, top_k), dtype=torch.uint8, device=dev)
        layer = lambda: moe.run_layer(x, wts, ids, mixed, out, ws)
    else:
        layer = lambda: moe.forward(x, wts, ids, pack, out=out)
    for _ in range(args.warmup):
        layer()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        layer()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clocks:
        e0.record()
        for _ in range(args.steps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    distinct = int(torch.unique(ids).numel())
    nbytes = distinct * (H * 2 * I + I * H) * K // 8
    peak, kind = measured_peak_hbm()
    gbs = nbytes / ms / 1e6
    print(json.dumps({"metric": "exl3_moe_layer_gbs_touched_expert_bytes", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
                      "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "f16", "data": "synthetic",
                      "config": {"workload": f"MoE layer hidden 2048, 256 experts, intermediate 512, top-8, K=3 3INST, {T} tokens",
                                 "tokens": T, "distinct_experts": distinct, "touched_bytes": nbytes,
                                 "path": "grouped tcgen05 GEMM, 128-row moe blocks" if tensor_core else "grouped GEMV, 8-row moe blocks",
                                 "tflops": 2.0 * T * top_k * 3 * H * I / ms / 1e9,
                                 "l2": "the layer's working set is L2-resident on replay (302 MB of experts, touched subset smaller)"},
                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                                   "peak_source": f"of {kind}", "kernel": "gemm_tc_kernel (grouped)" if tensor_core else "moe_gemm_kernel"},
                      "gpu_launches": (11 if tensor_core else 6) * args.steps, "clocks": clocks.summary()}))


def _graph_ring_time(run_one, ring: int, reps: int = 5) -> float:
    """Milliseconds per launch of `run_one(i)` for i in range(ring), captured as one CUDA graph over distinct weights
    (larger than L2 together) and replayed `reps` times: best replay."""
    import torch
    for i in range(min(ring, 2)):
        run_one(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(ring):
            run_one(i)
    g.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / ring)
    return best


def single_matrix_rate(dev, k: int, n: int, K: int, rows: int, codebook: int = 0, seed: int = 1) -> dict:
    """One k x n linear at `rows` rows: microseconds per launch and GB/s on packed bytes, over a ring of distinct weights."""
    import torch
    from trellis_serve_b200.kernels import linear as lin
    from trellis_serve_b200.runtime.layerset import random_packed, random_signs
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    nbytes = k * n * K // 8
    ring = max(2, min(64, int(600e6 // nbytes) + 1))
    ws = [random_packed(k, n, K, gen, dev) for _ in range(ring)]
    suh, svh = random_signs(k, gen, dev, 1), random_signs(n, gen, dev).view(-1)
    x = torch.randn((rows, k), device=dev, generator=gen).half()
    out = torch.empty((rows, n), dtype=torch.float16, device=dev)
    ms = _graph_ring_time(lambda i: lin.run(x, ws[i], suh, svh, [], codebook, out=out), ring)
    del ws
    torch.cuda.empty_cache()
    return {"us_per_launch": ms * 1e3, "gbs": nbytes / ms / 1e6, "ring": ring, "packed_bytes": nbytes}


def run_c1(args) -> None:
    """Secondary workload: ONE 4096 x 4096 linear, K = 4, 3INST, batch 1, timed over a ring of 64 distinct matrices
    (537 MB, larger than L2) chained in one CUDA graph.  One step = one launch."""
    import torch
    from trellis_serve_b200.kernels import linear as lin
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    with ClockSampler(0) as clocks:
        r = single_matrix_rate(dev, 4096, 4096, 4, 1)
    lin.device_error(dev)
    peak, kind = measured_peak_hbm()
    print(json.dumps({"metric": "exl3_gemv_hbm_gbs_packed_bytes_4096x4096_k4_batch1", "value": r["gbs"], "unit": UNIT, "n_gpus": 1,
                      "steps": r["ring"], "warmup": args.warmup, "ms_per_step": r["us_per_launch"] / 1e3, "higher_is_better": True,
                      "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                      "config": {"workload": "single EXL3 linear 4096x4096, K=4 3INST, batch 1, ring of 64 distinct matrices in one graph",
                                 "l2": "ring of 64 x 8.4 MB = 537 MB, larger than L2"},
                      "roofline": {"bound": "hbm", "achieved": r["gbs"], "peak": peak, "unit": "GB/s", "frac": r["gbs"] / peak,
                                   "traffic": None, "peak_source": f"of {kind}", "kernel": "gemv_kernel"},
                      "gpu_launches": r["ring"], "clocks": clocks.summary()}))


def decode_sweep(dev, args) -> dict:
    """Outside the timed region: the same captured step at 4 and 16 rows (8 layers, scaled), and every bit rate on the
    17408 x 5120 shape at batch 1."""
    import torch
    from trellis_serve_b200.runtime.layerset import DecodeLayerSet
    peak, _ = measured_peak_hbm()
    out = {"rows": {}, "bits_17408x5120": {}}
    layers = min(args.layers, 8)
    for rows in (4, 16):
        ls = DecodeLayerSet(layers, args.bits, 0, rows, device=dev, seed=900)
        ls.capture(warmup=2)
        for _ in range(3):
            ls.replay()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            ls.replay()
        e1.record()
        torch.cuda.synchronize(dev)
        ms_layer = e0.elapsed_time(e1) / 10 / layers
        out["rows"][str(rows)] = {"ms_per_64_layers": ms_layer * 64, "gbs": ls.packed_bytes / layers / ms_layer / 1e6,
                                  "frac": ls.packed_bytes / layers / ms_layer / 1e6 / peak, "layers_timed": layers}
        del ls
        torch.cuda.empty_cache()
    for K in range(2, 9):
        r = single_matrix_rate(dev, 17408, 5120, K, 1, seed=10 + K)
        out["bits_17408x5120"][str(K)] = {"us_per_launch": r["us_per_launch"], "gbs": r["gbs"], "frac": r["gbs"] / peak}
    return out


def decode_step_rate(dev, args, rank: int, world: int, reducer, dist, layers: int | None = None, context: int = 2048) -> dict:
    """The whole decode step of the 27B-shape transformer (64 layers, 40 query / 8 KV heads of 128, FFN 17408, K bits,
    `context` cached tokens in fp16, batch 1): RMSNorm, q|k|v, RoPE, attention over the cache, o, residual, RMSNorm,
    gate|up, SiLU * up, down, captured in one CUDA graph.  tok/s of the step, the share of the EXL3 linears (the same
    graph without the attention part is not separable, so the linears are timed as their own captured chain) and the
    key / value bytes a token reads."""
    import torch
    from trellis_serve_b200.runtime.decode_step import DecodeStep, ModelShape
    shape = ModelShape(layers=layers or args.layers)
    step = DecodeStep(shape, args.bits, 0, context, rows=1, tp_rank=rank, tp_size=world, device=dev, exchange=reducer)
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)
    step.h_in.copy_(torch.randn(step.h_in.shape, device=dev, generator=gen).to(step.dtype))
    step.capture(warmup=2)

    def timed(fn, reps):
        for _ in range(3):
            fn()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        t = torch.tensor([e0.elapsed_time(e1) / reps], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    ms = timed(step.replay, 20)
    same = True
    if dist is not None and world > 1:
        # The residual stream is replicated: after the exchanges every rank must hold the same bits.
        outs = [torch.empty_like(step.residual) for _ in range(world)]
        dist.all_gather(outs, step.residual)
        same = all(torch.equal(o.view(torch.int16), outs[0].view(torch.int16)) for o in outs)
    hin = torch.randn(step.h_in.shape).to(step.dtype).pin_memory()
    hout = torch.empty(step.out.shape, dtype=step.dtype).pin_memory()
    ms_e2e = timed(lambda: step.forward_host(hin, hout), 20)
    finite = bool(torch.isfinite(step.out).all().item())
    peak, kind = measured_peak_hbm()
    res = {"workload": f"27B-shape transformer decode, {shape.layers} layers, K={args.bits} 3INST, {context}-token fp16 KV, batch 1, tp{world}",
           "ms_per_token": ms, "tok_s": 1e3 / ms, "e2e_ms_per_token": ms_e2e, "e2e_tok_s": 1e3 / ms_e2e,
           "packed_weight_bytes_per_rank": step.packed_bytes, "kv_bytes_per_rank": step.kv_bytes,
           "hbm_gbs_weights_plus_kv_per_rank": (step.packed_bytes + step.kv_bytes) / ms / 1e6,
           "frac_of_hbm_per_rank": (step.packed_bytes + step.kv_bytes) / ms / 1e6 / peak, "peak_source": f"of {kind}",
           "launches_per_token": {"exl3_linears": step.linear_launches, "fused_producers": step.fused_launches,
                                  "attention_and_rope": step.attention_launches or "stock torch"},
           "outputs_finite": finite, "same_bits_on_every_rank": same}
    del step
    torch.cuda.empty_cache()
    return res


def run_step(args) -> None:
    """Secondary workload (single GPU or under torchrun): the full decode step; one step = one token."""
    import torch
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist, reducer = None, None
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        if args.allreduce in ("peer", "fused"):
            from trellis_serve_b200.runtime.allreduce import PeerAllReduce
            reducer = PeerAllReduce(dev, 16 * 5120)
    with ClockSampler(local) as clocks:
        r = decode_step_rate(dev, args, rank, world, reducer if args.allreduce == "fused" else None, dist)
    if rank == 0:
        print(json.dumps({"metric": "exl3_decode_tok_s_27b_k3_ctx2048_batch1", "value": r["tok_s"], "unit": "tok/s", "n_gpus": world,
                          "steps": 20, "warmup": 3, "ms_per_step": r["ms_per_token"], "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": {"workload": r["workload"]},
                          "e2e": {"value": r["e2e_tok_s"], "unit": "tok/s", "h2d_bytes_per_step": 10240, "d2h_bytes_per_step": 10240},
                          "decode_step": r, "gpu_launches": 20 * (r["launches_per_token"]["exl3_linears"] + r["launches_per_token"]["fused_producers"]),
                          "clocks": clocks.summary()}))
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize(dev)
        sys.stdout.flush()
        os._exit(0)


def tp_check(dev, rank: int, world: int, reducer, dist) -> dict:
    """Outside the timed region, N > 1: one row-parallel linear (17408 -> 5120, K = 3, every rank slices ITS rows out of the
    same seeded matrix) summed three ways -- exchange fused into the kernel, the library's stand-alone all-reduce, NCCL --
    and compared with each other, with the ranks' rounded partial results added on the host side of the check in rank order
    in fp32 and rounded once (what the exchange promises, bit for bit) and with the unsharded linear computed on every rank.
    NCCL adds in its own order with fp16 intermediates, so beyond two ranks it may differ from that sum by an ulp."""
    import torch
    from trellis_serve_b200.kernels import linear as lin
    from trellis_serve_b200.runtime.layerset import random_packed, random_signs
    k, n, K, cb = 17408, 5120, 3, 0
    gen = torch.Generator(device=dev)
    gen.manual_seed(4242)                                         # the same on every rank
    full = random_packed(k, n, K, gen, dev)                      # [n/128, k/128, ...]
    suh = random_signs(k, gen, dev, 1)
    svh = (random_signs(n, gen, dev).view(-1) / 64).half()
    x = torch.randn((1, k), device=dev, generator=gen).half()
    kg = k // 128 // world
    shard = full[:, rank * kg:(rank + 1) * kg].contiguous()
    xs, suhs = x[:, rank * kg * 128:(rank + 1) * kg * 128].contiguous(), suh[:, rank * kg * 128:(rank + 1) * kg * 128].contiguous()
    torch.cuda.synchronize(dev)
    whole = lin.run(x, full, suh, svh, [], cb).float()
    y_fused = lin.run(xs, shard, suhs, svh, [], cb, exchange=reducer) if reducer is not None else None
    y_peer = lin.run(xs, shard, suhs, svh, [], cb)
    y_nccl = y_peer.clone()
    parts = [torch.empty_like(y_peer) for _ in range(world)]
    dist.all_gather(parts, y_peer)
    expected = parts[0].float()
    for part in parts[1:]:
        expected = expected + part.float()
    expected = expected.half()
    if reducer is not None:
        reducer(y_peer)
    dist.all_reduce(y_nccl)
    torch.cuda.synchronize(dev)
    rms = float(whole.pow(2).mean().sqrt())
    res = {"shape": f"{k}x{n} K={K}", "max_rel_nccl_vs_unsharded": float((y_nccl.float() - whole).abs().max()) / rms}
    flags = torch.ones(3, dtype=torch.int32, device=dev)
    if reducer is not None:
        flags[0] = int(torch.equal(y_fused.view(torch.int16), y_peer.view(torch.int16)))
        flags[2] = int(torch.equal(y_fused.view(torch.int16), expected.view(torch.int16)))
        res["max_rel_vs_nccl"] = float((y_fused.float() - y_nccl.float()).abs().max()) / rms
        gathered = [torch.empty_like(y_fused) for _ in range(world)]
        dist.all_gather(gathered, y_fused)
        flags[1] = int(all(torch.equal(g.view(torch.int16), gathered[0].view(torch.int16)) for g in gathered))
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    worst = torch.tensor([res["max_rel_nccl_vs_unsharded"], res.get("max_rel_vs_nccl", 0.0)], dtype=torch.float64, device=dev)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    res["max_rel_nccl_vs_unsharded"], worst_nccl = worst.tolist()
    if reducer is not None:
        res["max_rel_vs_nccl"] = worst_nccl
        res["fused_eq_peer"] = bool(flags[0].item())
        res["same_bits_on_every_rank"] = bool(flags[1].item())
        res["fused_eq_rank_order_fp32_sum"] = bool(flags[2].item())
    del full, shard
    torch.cuda.empty_cache()
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--bits", type=int, default=3)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--allreduce", default="fused", choices=["fused", "peer", "nccl"],
                    help="exchange step of row-parallel layers at N > 1: the library's one-shot peer-memory kernel, or NCCL")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "moe", "c1", "step"],
                    help="decode = the headline 27B-shape layer set (default); prefill / moe / c1 = secondary single-GPU workloads; "
                         "step = the whole transformer decode step (attention and KV cache included), any N")
    ap.add_argument("--moe-path", choices=["auto", "gemv", "tc"], default="auto", help="--workload moe: force the grouped GEMV or the grouped tensor-core path")
    ap.add_argument("--no-sweep", action="store_true", help="skip the batch and bit-rate sweep appended to the default line")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload == "prefill":
        run_prefill(args)
        return
    if args.workload == "moe":
        run_moe(args)
        return
    if args.workload == "c1":
        run_c1(args)
        return
    if args.workload == "step":
        run_step(args)
        return

    import torch
    from trellis_serve_b200.kernels import linear as lin
    from trellis_serve_b200.runtime.layerset import DecodeLayerSet

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the EXL3 kernels have no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        # Neither the kernels here nor the exchange use multicast or multimem: keep every library off NVLink multicast
        # objects too (the rank processes leave without tearing the communicator down).
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    K, cb = args.bits, 0
    reducer = None
    if world > 1 and args.allreduce in ("peer", "fused"):
        from trellis_serve_b200.runtime.allreduce import PeerAllReduce
        reducer = PeerAllReduce(dev, 16 * 5120)
    ls = DecodeLayerSet(args.layers, K, cb, args.rows, tp_rank=rank, tp_size=world, device=dev, allreduce=reducer,
                        fused_exchange=args.allreduce == "fused")
    gen = torch.Generator(device=dev)
    gen.manual_seed(7 + rank)
    for buf in (ls.x_hidden, ls.x_attn, ls.x_ffn):
        buf.copy_(torch.randn(buf.shape, device=dev, generator=gen).to(buf.dtype))
    ls.capture(warmup=2)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-resident timing: inputs already in HBM, K replays of the captured step
    for _ in range(args.warmup):
        ls.replay()
    barrier()
    block_ms = []
    with ClockSampler(local) as clocks:
        for _ in range(BLOCKS):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(args.steps):
                ls.replay()
            stop.record()
            barrier()
            block_ms.append(start.elapsed_time(stop))
    lin.device_error(dev)
    if reducer is not None:
        reducer.check()

    # ---- end to end: pinned host inputs -> device, step, result -> host, every step
    hx = [torch.randn(b.shape).to(b.dtype).pin_memory() for b in (ls.x_hidden, ls.x_attn, ls.x_ffn)]
    hy = torch.empty(ls.y_down.shape, dtype=ls.y_down.dtype).pin_memory()
    for _ in range(args.warmup):
        ls.forward_host(*hx, hy)
    barrier()
    e2e_ms = []
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            ls.forward_host(*hx, hy)
        e1.record()
        barrier()
        e2e_ms.append(e0.elapsed_time(e1))

    # every block: the slowest rank's time; then the median block
    t = torch.tensor(block_ms + e2e_ms, dtype=torch.float64, device=dev)
    nbytes = torch.tensor([float(ls.packed_bytes)], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(nbytes, op=dist.ReduceOp.SUM)
    t = t.tolist()
    block_ms, e2e_ms = t[:BLOCKS], t[BLOCKS:]
    ms_total, ms_e2e = statistics.median(block_ms), statistics.median(e2e_ms)
    total_bytes = nbytes.item()
    ls_packed_bytes, ls_launches = ls.packed_bytes, ls.launches_per_step
    check = tp_check(dev, rank, world, reducer, dist) if dist is not None else None
    sweep = decode_sweep(dev, args) if (world == 1 and not args.no_sweep) else None
    full_step = None
    if not args.no_sweep:
        del ls                                            # its weights make room for the full step's
        torch.cuda.empty_cache()
        full_step = decode_step_rate(dev, args, rank, world, reducer if args.allreduce == "fused" else None, dist)
    if rank == 0:
        ms_step = ms_total / args.steps
        value = total_bytes / (ms_step * 1e-3) / 1e9
        e2e_value = total_bytes / (ms_e2e / args.steps * 1e-3) / 1e9
        peak, peak_kind = measured_peak_hbm()
        gemv_launches = args.layers * 4
        per_rank_bytes = ls_packed_bytes
        # Roofline of the dominant kernel (the decode GEMV): algorithmic bytes = packed-weight bytes of a launch.
        # Its average duration is bounded from above by the whole step time divided by the number of GEMV launches
        # (the step also contains the small activation-rotation kernels), so `achieved` is a lower bound.
        avg_launch_ms = ms_step / gemv_launches
        achieved = per_rank_bytes / gemv_launches / (avg_launch_ms * 1e-3) / 1e9
        # DRAM traffic per launch: ncu's dram__bytes_read.sum + dram__bytes_write.sum of one captured gate|up launch,
        # scaled to the average launch by its units; the kernel reads every weight byte exactly once, so traffic grows
        # with the units.
        ratio, traffic_source = traffic_ratio()
        traffic = ratio * per_rank_bytes / gemv_launches if ratio is not None else None
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
                "data": "synthetic",
                "config": workload_config(args, world, total_bytes),
                "tok_s": 1e3 / ms_step,
                "timing": {"blocks": BLOCKS, "steps_per_block": args.steps, "block_ms": [round(b, 4) for b in block_ms],
                           "reported": "median block, slowest rank per block"},
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "traffic": traffic, "traffic_unit": "bytes per launch, from one ncu capture scaled by units",
                             "traffic_source": traffic_source,
                             "peak_source": f"of {peak_kind}", "kernel": "gemv_kernel",
                             "launches_per_step": gemv_launches, "avg_launch_ms_upper_bound": avg_launch_ms},
                "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                        "h2d_bytes_per_step": sum(h.numel() * h.element_size() for h in hx),
                        "d2h_bytes_per_step": hy.numel() * hy.element_size(), "tok_s": 1e3 / (ms_e2e / args.steps)},
                "gpu_launches": ls_launches * args.steps,
                "clocks": clocks.summary()}
        if check is not None:
            line["tp_check"] = check
        if sweep is not None:
            line["sweep"] = sweep
        if full_step is not None:
            line["decode_step"] = full_step
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = {k: v for k, v in cpu_sample(K, cb).items() if k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if dist is not None:
        # The captured step holds NCCL work; tearing the communicator down under it can block for minutes.
        # All results are out, so synchronise, meet once more and leave without the teardown.
        dist.barrier()
        torch.cuda.synchronize(dev)
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
