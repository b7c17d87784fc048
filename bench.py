#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config NAME]

Default workload (N = 1): the NVFP4 W4A4 prefill GEMM of one 512-token chunk, M = 512, K = 5120,
N = 27648 (fused gate+up).  A step = quantize the bf16 activations to NVFP4 on the fly (per-row global
scale, per-16 E4M3 scales) + the block-scaled tcgen05 GEMM with bf16 output.  Inputs are synthetic
(X ~ N(0,1) bf16, W ~ N(0, 0.02^2) quantized the ModelOpt way), seeded.

Prints ONE JSON line: whole-job TFLOP/s with inputs resident in HBM (`value`), the same through the public
API with host buffers (`e2e`), the roofline of the dominant kernel, and the reference's CPU path timed on
the host cores (`cpu_baseline`).  With --gpus N > 1 (launched by torchrun) the weight is sharded over N
column-wise; the bf16 column blocks are written into every rank's output by the GEMM epilogue (symmetric memory, --gather
fused) or all-gathered over NCCL (--gather nccl); strong scaling of the same workload.
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M, K, N = 512, 5120, 27648
WORKLOAD = "nvfp4_w4a4_prefill_gemm_M512_K5120_N27648"
METRIC = "nvfp4_gemm_tflops"
UNIT = "TFLOP/s"
FLOPS_PER_STEP = 2.0 * M * N * K
NCU_DRAM_BYTES_FULL_LAUNCH = 81190144 + 4600064
NOMINAL_NVFP4_TFLOPS = 9000.0


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline(sample_cols: int | None = None, threads: int = 0, target_seconds: float = 12.0):
    """The reference's host path (NVFP4 unpack + f32 triple loop) on a bounded sample: all 512 tokens, all of K,
    the first `sample_cols` output features.  Returns (TFLOP/s, cores, sample description, seconds)."""
    import numpy as np

    from oracle import oracle as o
    rng = np.random.default_rng(0)
    cores = o.max_threads() if threads <= 0 else threads
    x = o.bf16_round(rng.standard_normal((M, K)).astype(np.float32))

    def run(cols):
        w = (rng.standard_normal((cols, K)) * 0.02).astype(np.float32)
        wp, ws, g = o.quantize_weight(w)
        scratch = np.empty(cols * K, np.float32)
        t0 = time.perf_counter()
        o.nvfp4_linear_host(x, wp, ws, float(g), threads=threads, scratch=scratch)
        return time.perf_counter() - t0

    if sample_cols is None:
        probe_cols = 64
        t_probe = run(probe_cols)
        sample_cols = int(max(64, min(N, probe_cols * target_seconds / max(t_probe, 1e-6))))
        sample_cols = max(64, sample_cols // 64 * 64)
    seconds = run(sample_cols)
    tflops = 2.0 * M * sample_cols * K / seconds / 1e12
    sample = f"all {M} tokens x all K={K} x first {sample_cols} of {N} output features (unpack + f32 triple loop)"
    return tflops, cores, sample, seconds


def reference_arm(args):
    """--impl reference: the reference's own CPU implementation of the path (oracle port; the Rust original cannot be
    built here: no cargo/rustc) with all host threads, each step a bounded sample of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np

    from oracle import oracle as o
    rng = np.random.default_rng(0)
    cores = o.max_threads()
    x = o.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    # size the per-step sample so the whole run stays within a couple of minutes
    cols = 64
    w = (rng.standard_normal((cols, K)) * 0.02).astype(np.float32)
    wp, ws, g = o.quantize_weight(w)
    t0 = time.perf_counter()
    o.nvfp4_linear_host(x, wp, ws, float(g))
    t_probe = time.perf_counter() - t0
    budget = 90.0 / max(1, args.steps + args.warmup)
    cols = int(max(64, min(N, cols * budget / max(t_probe, 1e-6)))) // 64 * 64
    cols = max(cols, 64)
    w = (rng.standard_normal((cols, K)) * 0.02).astype(np.float32)
    wp, ws, g = o.quantize_weight(w)
    scratch = np.empty(cols * K, np.float32)
    for _ in range(args.warmup):
        o.nvfp4_linear_host(x, wp, ws, float(g), scratch=scratch)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        o.nvfp4_linear_host(x, wp, ws, float(g), scratch=scratch)
    dt = (time.perf_counter() - t0) / args.steps
    value = 2.0 * M * cols * K / dt / 1e12
    sample = f"all {M} tokens x all K={K} x first {cols} of {N} output features per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3 * (N / cols), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "nvfp4(e2m1+ue4m3) x nvfp4, f32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def _graph_time_us(torch, fn, iters, reps=5):
    """Best-of-`reps` device time per call of fn(i) when `iters` calls are replayed as one CUDA graph."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(iters):
                fn(i)
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    best = float("inf")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(reps):
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / iters * 1e3)
    return best


def config_decode(args):
    """Decode configs on one GPU: NVFP4 W4A16 GEMV (M=1, K=5120, N=13824 and the down projection) and the FP8 QKV
    projection for M in {1, 8, 32, 64}; HBM-bound, reported as GB/s of the algorithmic bytes."""
    import torch

    from eider_b200 import ops
    peaks = load_peaks()
    copies = 6
    out = {"metric": "decode_hbm_gbs", "unit": "GB/s", "n_gpus": 1, "data": "synthetic", "peak_hbm_gbs": peaks["hbm_gbs"],
           "peak_source": peaks["source"], "timing": f"CUDA-graph replay of {args.steps} calls, {copies} rotating weight copies",
           "cases": []}
    for tokens, n, k in [(1, 13824, 5120), (1, 5120, 13824), (8, 13824, 5120), (64, 13824, 5120)]:
        ws = [ops.ModelOptWeight.quantize(torch.randn(n, k, device="cuda") * 0.02) for _ in range(copies)]
        x = torch.randn(tokens, k, device="cuda").to(torch.bfloat16)
        plan = ops.Nvfp4DecodePlan(tokens, n, k)
        y = torch.empty(tokens, n, dtype=torch.bfloat16, device="cuda")
        us = _graph_time_us(torch, lambda i: plan.run(x, ws[i % copies], out=y), args.steps)
        assert plan.status() == 0
        nbytes = n * k // 2 + n * k // 16 + 2 * tokens * k + 2 * tokens * n + 4
        case = {"op": "nvfp4_w4a16_decode", "M": tokens, "K": k, "N": n, "us": us, "bytes": nbytes, "gbs": nbytes / us / 1e3,
                "frac_of_hbm_peak": nbytes / us / 1e3 / peaks["hbm_gbs"]}
        if tokens == 1:
            ys = torch.empty(tokens, n, dtype=torch.bfloat16, device="cuda")
            case["cuda_core_gemv_us"] = _graph_time_us(torch, lambda i: ops.nvfp4_w4a16_matvec(x, ws[i % copies], out=ys), args.steps)
        out["cases"].append(case)
        del ws
    n, k = 7168, 5120
    wq = [torch.randint(0, 120, (n, k), dtype=torch.uint8, device="cuda") for _ in range(copies)]
    sw = torch.rand(n, device="cuda") * 0.01
    plan = ops.Fp8DecodePlan(64, n, k)
    for tokens in (1, 8, 32, 64):
        x = torch.randn(tokens, k, device="cuda").to(torch.bfloat16)
        y = torch.empty(tokens, n, dtype=torch.bfloat16, device="cuda")
        us = _graph_time_us(torch, lambda i: plan.run(x, wq[i % copies], sw, out=y), args.steps)
        assert plan.status() == 0
        nbytes = n * k + 4 * n + 2 * tokens * k + 2 * tokens * n
        out["cases"].append({"op": "fp8_w8a8_decode", "M": tokens, "K": k, "N": n, "us": us, "bytes": nbytes,
                             "gbs": nbytes / us / 1e3, "frac_of_hbm_peak": nbytes / us / 1e3 / peaks["hbm_gbs"],
                             "tflops": 2.0 * tokens * n * k / us / 1e6})
    out["value"] = out["cases"][0]["gbs"]
    out["config"] = {"workload": "decode: nvfp4 gemv M=1 K=5120 N=13824 (value), down projection, fp8 qkv M in {1,8,32,64}"}
    print(json.dumps(out), flush=True)


def config_fp8_gemm(args):
    """FP8 W8A8 prefill GEMM (per-token x per-channel scales in the epilogue) at a few shapes, one GPU."""
    import torch
    from eider_b200 import ops
    peaks = load_peaks()
    cases = []
    for (m, k, n) in [(512, 5120, 7168), (512, 5120, 27648), (2048, 5120, 7168), (4096, 5120, 27648)]:
        ws = [torch.randint(0, 120, (n, k), dtype=torch.uint8, device="cuda") for _ in range(3)]
        wsc = torch.rand(n, device="cuda") * 0.01
        x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        xq, xs = ops.quantize_fp8_dynamic(x)
        y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        plan = ops.Fp8TnMatmulPlan(m, n, k)
        if args.block_n:
            plan.set_block_n(args.block_n)
        for i in range(args.warmup):
            plan.run(xq, ws[i % 3], xs, wsc, out=y)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            plan.run(xq, ws[i % 3], xs, wsc, out=y)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / args.steps
        tf = 2.0 * m * n * k / us / 1e6
        assert plan.status() == 0
        cases.append({"M": m, "K": k, "N": n, "tile_code": plan.block_n, "us": us, "tflops": tf,
                      "frac_of_2x_bf16_peak": tf / (2.0 * peaks["bf16_tflops"])})
    print(json.dumps({"metric": "fp8_gemm_tflops", "unit": "TFLOP/s", "n_gpus": 1, "data": "synthetic",
                      "peak": 2.0 * peaks["bf16_tflops"], "peak_source": f"2 x {peaks['source']} dense bf16 burst",
                      "timing": f"CUDA events over {args.steps} launches, 3 rotating weight copies", "cases": cases}))


def config_moe(args):
    """Routed-MoE prefill: 4096 tokens, 128 experts, top-8, hidden 2048, intermediate 768, one GPU."""
    import torch

    from eider_b200 import ops
    t, e, k8, h, inter = 4096, 128, 8, 2048, 768
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(t, h, device="cuda", generator=g).to(torch.bfloat16)
    logits = torch.randn(t, e, device="cuda", generator=g)
    w_gu = ops.GroupedNvfp4Weights.quantize(torch.randn(e, 2 * inter, h, device="cuda", generator=g) * 0.02)
    w_dn = ops.GroupedNvfp4Weights.quantize(torch.randn(e, h, inter, device="cuda", generator=g) * 0.02)
    moe = ops.GroupedMoe(t, e, k8, h, inter)

    def timed(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps * 1e3

    total = timed(lambda: moe.run(x, logits, w_gu, w_dn))
    assert moe.gate_up_plan.status() == 0 and moe.down_plan.status() == 0
    idx, wts = ops.moe_topk(logits, k8, True)
    stages = {
        "topk": timed(lambda: ops.moe_topk(logits, k8, True)),
        "sort": timed(lambda: moe.routes.sort(idx.reshape(-1))),
        "gather_quantize": timed(lambda: moe.gate_up_in.gather_quantize(x, moe.routes, k8)),
        "gemm_gate_up": timed(lambda: moe.gate_up_plan.run(moe.gate_up_in, w_gu, moe.routes, out=moe.gate_up_out)),
        "silu_mul_quantize": timed(lambda: moe.down_in.silu_mul_halves_quantize(moe.gate_up_out, moe.routes)),
        "gemm_down": timed(lambda: moe.down_plan.run(moe.down_in, w_dn, moe.routes, out=moe.down_out)),
        "combine": timed(lambda: ops.moe_weighted_accumulate(moe.routes, wts.reshape(-1), moe.down_out, t, k8, out=moe.out)),
    }
    flops = 2.0 * t * k8 * (h * 2 * inter + inter * h)
    print(json.dumps({"metric": "moe_prefill_tflops", "value": flops / total / 1e6, "unit": "TFLOP/s", "n_gpus": 1,
                      "us_per_step": total, "stage_us": stages, "min_bytes_gbs": 375391232 / total / 1e3, "data": "synthetic",
                      "config": {"workload": "nvfp4 routed moe prefill: 4096 tokens, 128 experts, top-8, H=2048, I=768"}}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="eider_b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--gather", default="auto", choices=["auto", "fused", "nccl"],
                    help="N > 1: how the column blocks become [M, N] on every rank: GEMM epilogue stores into every "
                         "rank's output (symmetric memory) or NCCL all-gather + re-assembly; auto = fused on 2, 4 and 8 ranks")
    ap.add_argument("--config", default="prefill", choices=["prefill", "decode", "moe", "fp8"],
                    help="prefill (default, the contract line), or the single-GPU decode / MoE / FP8 GEMM configs")
    ap.add_argument("--tokens", type=int, default=0, help="prefill only: M instead of 512 (the larger-chunk configs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.tokens:
        global M, WORKLOAD, FLOPS_PER_STEP
        M = args.tokens
        WORKLOAD = f"nvfp4_w4a4_prefill_gemm_M{M}_K{K}_N{N}"
        FLOPS_PER_STEP = 2.0 * M * N * K
    if args.impl != "reference" and args.config == "decode":
        return config_decode(args)
    if args.impl != "reference" and args.config == "moe":
        return config_moe(args)
    if args.impl != "reference" and args.config == "fp8":
        return config_fp8_gemm(args)

    if args.impl == "reference":
        reference_arm(args)
        return

    import torch

    from eider_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if args.gpus != world:
        if rank == 0:
            print(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}; using {world}", file=sys.stderr)
    peaks = load_peaks()

    # ---- synthetic inputs (seed 0): weights quantized the ModelOpt way on the device --------------------
    n_local = N // world
    assert N % (world * 128) == 0, "N shards must be multiples of 128 rows"
    gen = torch.Generator(device="cuda").manual_seed(0)
    rotate = 4 if world == 1 else 2  # distinct weight copies so the 126 MB L2 cannot hold the working set
    weights = []
    for r in range(rotate):
        wgen = torch.Generator(device="cuda").manual_seed(1000 + r)
        w_full_rows = torch.randn(n_local, K, device="cuda", generator=wgen) * 0.02
        weights.append(ops.ModelOptWeight.quantize(w_full_rows))
        del w_full_rows
    x_host = torch.randn(M, K, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).pin_memory()
    x_dev = x_host.cuda()
    xq = ops.Nvfp4Matrix.zeros(M, K, "cuda", row_scales=True)
    y_local = torch.empty(M, n_local, dtype=torch.bfloat16, device="cuda")
    y_host = torch.empty(M, N if world == 1 else n_local * world, dtype=torch.bfloat16).pin_memory()
    plan = ops.Fp4TnMatmulPlan(M, n_local, K)
    if args.block_n:
        plan.set_block_n(args.block_n)

    from eider_b200 import parallel
    current = {"w": weights[0]}

    def local_linear(x):
        ops.quantize_nvfp4_rowscale(x, out=xq)
        return (sharded.active_plan or plan).run(xq, current["w"], out=y_local)

    sharded = parallel.ColumnShardedLinear(N, local_linear)
    gather = "none" if world == 1 else "nccl"
    FUSED_MEASURED_ON = (2, 4, 8)  # verified on 2, 4 and 8 ranks of one box
    if world > 1 and (args.gather == "fused" or (args.gather == "auto" and world in FUSED_MEASURED_ON)):
        try:
            plan_b = ops.Fp4TnMatmulPlan(M, n_local, K)  # second output buffer: one barrier per step is enough
            for q in (plan, plan_b):
                if args.block_n:
                    q.set_block_n(args.block_n)
                elif M > 128:
                    q.set_block_n(512)  # the CTA-pair kernel writes peers through shared memory and TMA stores
            sharded.fuse_into([plan, plan_b], M)
            gather = "fused"
        except Exception as exc:  # symmetric memory is not available on this box: keep the NCCL path
            if rank == 0:
                print(f"# fused all-gather unavailable ({type(exc).__name__}: {exc}); using NCCL", file=sys.stderr)
    result = {}

    def step(i, x):
        current["w"] = weights[i % rotate]
        y = sharded.forward(x)  # N > 1: all-gather of the bf16 slabs + re-assembly to row-major [M, N]
        result["y"] = y if world == 1 else y.contiguous()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """Device time of `steps` calls of fn(i) in ms, max over ranks."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for i in range(args.warmup):
        step(i, x_dev)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    total_ms = timed(lambda i: step(i, x_dev), args.steps)
    ms_per_step = total_ms / args.steps
    value = FLOPS_PER_STEP / (ms_per_step * 1e-3) / 1e12

    # ---- dominant kernel alone (roofline): CUDA events around the GEMM launches only ----------------------
    gemm_ms = timed(lambda i: plan.run(xq, weights[i % rotate], out=y_local), args.steps) / args.steps
    # the quantizer runs for a few microseconds, less than a Python launch takes: time it as one graph of launches
    quant_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(quant_graph):
        for _ in range(args.steps):
            ops.quantize_nvfp4_rowscale(x_dev, out=xq)
    quant_graph.replay()
    quant_ms = timed(lambda i: quant_graph.replay(), 1) / args.steps
    if rank == 0:
        clocks = sampler.stop()
    status = plan.status()
    assert status == 0, f"GEMM kernel reported status {status:#x}"

    # ---- end to end through the public API with host buffers ------------------------------------------------
    x_stage = torch.empty_like(x_dev)

    def e2e_step(i):
        x_stage.copy_(x_host, non_blocking=True)
        step(i, x_stage)
        y_host.copy_(result["y"], non_blocking=True)

    for i in range(3):
        e2e_step(i)
    e2e_ms = timed(e2e_step, args.steps) / args.steps
    e2e_value = FLOPS_PER_STEP / (e2e_ms * 1e-3) / 1e12

    if rank != 0:
        if dist:
            dist.destroy_process_group()
        return

    gemm_flops_local = 2.0 * M * n_local * K
    achieved = gemm_flops_local / (gemm_ms * 1e-3) / 1e12
    nvfp4_peak = 4.0 * peaks["bf16_tflops"]
    roofline = {
        "bound": "tensor",
        "kernel": ("gemm_pair_kernel<nvfp4> (tcgen05.mma cta_group::2 kind::mxf4nvf4.block_scale, 256x256 tiles on CTA pairs)"
                   if plan.block_n == 512 else
                   f"gemm_kernel<nvfp4, {plan.block_n}> (tcgen05.mma kind::mxf4nvf4.block_scale)"),
        "achieved": achieved, "peak": nvfp4_peak, "unit": "TFLOP/s", "frac": achieved / nvfp4_peak,
        "peak_source": f"4 x {peaks['source']} dense bf16 burst ({peaks['bf16_tflops']} TF/s); NVFP4 is not measured by the driver",
        "frac_of_nominal_9pf": achieved / NOMINAL_NVFP4_TFLOPS,
        "kernel_ms": gemm_ms, "quantize_kernel_ms": quant_ms,
        "hbm_gbs_at_min_bytes": (n_local * K * 9 / 16 + M * K * 9 / 16 + 2.0 * M * n_local) / (gemm_ms * 1e-3) / 1e9,
        # dram__bytes_read + dram__bytes_write of one launch of this kernel at the full shape (85.8 MB, one ncu
        # capture, see profiles/), scaled by this rank's share of the weight rows
        "traffic": NCU_DRAM_BYTES_FULL_LAUNCH * n_local / N, "traffic_unit": "bytes per launch",
    }
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "nvfp4(e2m1+ue4m3) x nvfp4, f32 accumulate, bf16 out", "data": "synthetic",
        "config": {"workload": WORKLOAD, "M": M, "K": K, "N": N, "partition": f"N column-sharded x{world}" +
                   ({"nccl": " + NCCL all-gather of bf16 outputs", "none": "",
                     "fused": " + all-gather fused into the GEMM epilogue (stores into every rank's output over NVLink)"}[gather]),
                   "l2": f"inputs larger than L2: {rotate} rotating weight copies of {n_local * K * 9 // 16 // 2**20} MiB each"},
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": M * K * 2,
                "d2h_bytes_per_step": M * N * 2, "note": "weights stay resident in HBM (model state); X from and Y to pinned host memory"},
        "gpu_launches": 2 * args.steps, "clocks": clocks, "roofline": roofline,
    }
    if not args.no_cpu_baseline and world == 1:
        tflops, cores, sample, seconds = cpu_baseline()
        line["cpu_baseline"] = {"value": tflops, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                "seconds": seconds}
    print(json.dumps(line), flush=True)
    if dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
