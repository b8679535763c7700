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
    ms = best["seconds_per_layer"] * 1e3
    line = {"impl": "reference", "metric": METRIC, "value": best["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "layers": args.layers, "bits": K, "codebook": "3inst", "rows": args.rows,
                       "parallelism": f"tp{args.gpus}", "l2": "inputs larger than L2, no flush",
                       "packed_bytes_per_step": 64 * 123863040.0 if K == 3 else None},
            "cpu_baseline": {k: best[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": best["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "tok_s": best["tok_s"], "gpu_launches": 0}
    print(json.dumps(line))


def run_prefill(args) -> None:
    """Secondary workload (BASELINE config 3): the four fused groups of one 27B-shape layer at M = 2048 rows, K = 4,
    MCG codebook, through the fused tcgen05 kernel.  One step = one layer.  Tensor-pipe roofline."""
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
                      "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "traffic": None,
                                   "peak_source": "of measured (burst)", "kernel": "gemm_tc_kernel"},
                      "gpu_launches": 16 * args.steps, "clocks": clocks.summary()}))


def run_moe(args) -> None:
    """Secondary workload (BASELINE config 4): one MoE layer, hidden 2048, 256 experts, intermediate 512, top-8, K = 3,
    softmax-of-N(0,1) routing, captured in a CUDA graph.  GB/s on the packed bytes of the distinct routed experts."""
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
    for _ in range(args.warmup):
        moe.forward(x, wts, ids, pack, out=out)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        moe.forward(x, wts, ids, pack, out=out)
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
                                 "l2": "the layer's working set is L2-resident on replay (302 MB of experts, touched subset smaller)"},
                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                                   "peak_source": f"of {kind}", "kernel": "moe_gemm_kernel"},
                      "gpu_launches": 6 * args.steps, "clocks": clocks.summary()}))


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
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "moe"],
                    help="decode = the headline 27B-shape layer set (default); prefill / moe = secondary single-GPU workloads")
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
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        start.record()
        for _ in range(args.steps):
            ls.replay()
        stop.record()
        barrier()
    ms_total = start.elapsed_time(stop)
    lin.device_error(dev)
    if reducer is not None:
        reducer.check()

    # ---- end to end: pinned host inputs -> device, step, result -> host, every step
    hx = [torch.randn(b.shape).to(b.dtype).pin_memory() for b in (ls.x_hidden, ls.x_attn, ls.x_ffn)]
    hy = torch.empty(ls.y_down.shape, dtype=ls.y_down.dtype).pin_memory()
    for _ in range(args.warmup):
        ls.forward_host(*hx, hy)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        ls.forward_host(*hx, hy)
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)

    t = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
    nbytes = torch.tensor([float(ls.packed_bytes)], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(nbytes, op=dist.ReduceOp.SUM)
    ms_total, ms_e2e = t.tolist()
    total_bytes = nbytes.item()
    if rank == 0:
        ms_step = ms_total / args.steps
        value = total_bytes / (ms_step * 1e-3) / 1e9
        e2e_value = total_bytes / (ms_e2e / args.steps * 1e-3) / 1e9
        peak, peak_kind = measured_peak_hbm()
        gemv_launches = args.layers * 4
        per_rank_bytes = ls.packed_bytes
        # Roofline of the dominant kernel (the decode GEMV): algorithmic bytes = packed-weight bytes of a launch.
        # Its average duration is bounded from above by the whole step time divided by the number of GEMV launches
        # (the step also contains the small activation-rotation kernels), so `achieved` is a lower bound.
        avg_launch_ms = ms_step / gemv_launches
        achieved = per_rank_bytes / gemv_launches / (avg_launch_ms * 1e-3) / 1e9
        # DRAM traffic per launch: ncu's dram__bytes_read.sum + dram__bytes_write.sum of the captured gate|up launch
        # (profiles/gemv_kernel_27b_k3_batch1.md: 67.015 MB + 0.458 MB for 66.847 MB of packed weights) scaled to the
        # average launch by its units; the kernel reads every weight byte exactly once, so traffic grows with the units.
        traffic = (67.015e6 + 0.458e6) / 66.847e6 * per_rank_bytes / gemv_launches
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
                "data": "synthetic",
                "config": {"workload": WORKLOAD, "layers": args.layers, "bits": K, "codebook": "3inst", "rows": args.rows,
                           "parallelism": f"tp{world}", "allreduce": (args.allreduce if world > 1 else None),
                           "l2": "inputs larger than L2, no flush",
                           "packed_bytes_per_step": total_bytes},
                "tok_s": 1e3 / ms_step,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "traffic": traffic, "traffic_unit": "bytes per launch, from one ncu capture scaled by units",
                             "peak_source": f"of {peak_kind}", "kernel": "gemv_kernel",
                             "launches_per_step": gemv_launches, "avg_launch_ms_upper_bound": avg_launch_ms},
                "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                        "h2d_bytes_per_step": sum(h.numel() * h.element_size() for h in hx),
                        "d2h_bytes_per_step": hy.numel() * hy.element_size(), "tok_s": 1e3 / (ms_e2e / args.steps)},
                "gpu_launches": ls.launches_per_step * args.steps,
                "clocks": clocks.summary()}
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
