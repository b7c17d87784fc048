#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config NAME]

Default workload (N = 1): the NVFP4 W4A4 prefill GEMM of one 512-token chunk, M = 512, K = 5120,
N = 27648 (fused gate+up).  A step = quantize the bf16 activations to NVFP4 on the fly (per-row global
scale, per-16 E4M3 scales) + the block-scaled tcgen05 GEMM with bf16 output.  Inputs are synthetic
(X ~ N(0,1) bf16, W ~ N(0, 0.02^2) quantized the ModelOpt way), seeded.

Prints ONE JSON line: whole-job TFLOP/s with inputs resident in HBM (`value`: K steps replayed as one CUDA graph), the
same through the public API with host buffers (`e2e`), the roofline of the dominant kernel, the parity of the timed
weights against the host path (`parity`; a failure exits non-zero before anything is timed) and the reference's CPU path
timed on the host cores (`cpu_baseline`).  With --gpus N > 1 (launched by torchrun) the weight is sharded over N
column-wise and the bf16 column blocks are written into every rank's output by the GEMM epilogue over NVLink (one
multimem.st per tile through the switch, or one TMA store per peer with --no-multicast) or all-gathered over NCCL
(--gather nccl); strong scaling of the same workload, with `scaling_detail` and the expert-parallel MoE in `extra.moe_ep`.
Other configs: --config decode | moe | fp8 | sweep, --tokens / --in-features / --out-features.
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


def full_config(world: int) -> dict:
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": WORKLOAD, "M": M, "K": K, "N": N, "n_shards": world}


def cpu_reference_product(a, wp, ws, g, cols=None, threads: int = 0, target_seconds: float = 15.0):
    """The reference's host path (NVFP4 unpack + f32 triple loop, crates/eider-format/src/modelopt.rs:741-757 +
    crates/eider-cuda/src/format.rs:379-392) on the activations `a` [M, K] f32 and the first `cols` weight rows (all of
    them when the probe says the whole product fits about `target_seconds`).  Returns (Y [M, cols] f32, seconds, cols)."""
    import numpy as np

    from oracle import oracle as o
    n = wp.shape[0]
    if cols is None:
        probe = min(64, n)
        t0 = time.perf_counter()
        o.nvfp4_linear_host(a, wp[:probe], ws[:probe], float(g), threads=threads)
        t_probe = time.perf_counter() - t0
        cols = n if t_probe * n / probe <= target_seconds else max(64, int(probe * target_seconds / max(t_probe, 1e-6)) // 64 * 64)
        cols = min(cols, n)
    scratch = np.empty(cols * a.shape[1], np.float32)
    t0 = time.perf_counter()
    y = o.nvfp4_linear_host(a, np.ascontiguousarray(wp[:cols]), np.ascontiguousarray(ws[:cols]), float(g), threads=threads, scratch=scratch)
    return y, time.perf_counter() - t0, cols


def parity_report(y, ref, rel=1e-2, abs_frac=1e-2):
    """|y - ref| <= max(tau, rel * |ref|), tau = abs_frac * rms(ref): the criterion of the GEMM parity tests (the reference's
    mixed bound, crates/eider-cuda/src/cublaslt/fp4_tn.rs:1534, with the floor scaled to the data)."""
    import numpy as np
    y = np.asarray(y, np.float64)
    ref = np.asarray(ref, np.float64)
    tau = abs_frac * float(np.sqrt(np.mean(ref * ref))) + 1e-30
    err = np.abs(y - ref)
    bad = err > np.maximum(tau, rel * np.abs(ref))
    big = np.abs(ref) >= tau
    return {"max_rel_err": float(np.max(err[big] / np.abs(ref[big]))) if big.any() else 0.0, "bad": int(bad.sum()),
            "checked_elements": int(bad.size), "criterion": f"|y - ref| <= max({abs_frac} * rms(ref), {rel} * |ref|) against host dequantize + f32 matmul"}


def reference_arm(args):
    """--impl reference: the reference's own CPU implementation of the path (oracle port; the Rust original cannot be
    built here: no cargo/rustc) with all host threads.  A step = the whole workload when the run then stays within a few
    minutes, else the first columns that do."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np

    from oracle import oracle as o
    rng = np.random.default_rng(0)
    cores = o.max_threads()
    xp, xs, xr = o.quantize_nvfp4_rowscale(o.bf16_round(rng.standard_normal((M, K)).astype(np.float32)))
    x = o.dequantize_tiled(xp, xs) * xr[:, None]  # the NVFP4 activations as the host sees them
    probe = 64
    w = (rng.standard_normal((probe, K)) * 0.02).astype(np.float32)
    wp, ws, g = o.quantize_weight(w)
    t0 = time.perf_counter()
    o.nvfp4_linear_host(x, wp, ws, float(g))
    t_probe = time.perf_counter() - t0
    budget = 150.0 / max(1, args.steps + args.warmup)
    cols = N if t_probe * N / probe <= budget else max(64, int(probe * budget / max(t_probe, 1e-6)) // 64 * 64)
    # one block of random weights tiled over the sample: the host path's time does not depend on the values
    reps = (cols + probe - 1) // probe
    wp, ws = np.tile(wp, (reps, 1))[:cols], np.tile(ws, (reps, 1))[:cols]
    scratch = np.empty(cols * K, np.float32)
    for _ in range(args.warmup):
        o.nvfp4_linear_host(x, wp, ws, float(g), scratch=scratch)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        o.nvfp4_linear_host(x, wp, ws, float(g), scratch=scratch)
    dt = (time.perf_counter() - t0) / args.steps
    value = 2.0 * M * cols * K / dt / 1e12
    sample = (f"the whole workload per step ({M} tokens x K={K} x {N} output features)" if cols == N else
              f"all {M} tokens x all K={K} x first {cols} of {N} output features per step")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3 * (N / cols), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "nvfp4(e2m1+ue4m3) x nvfp4, f32 accumulate, bf16 out", "data": "synthetic",
        "config": full_config(args.gpus),
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
        if tokens <= 8:
            # the same GEMV on an operand its producer has already expanded (once per x, shared by the linears that read x);
            # "pair" times the expansion kernel and the GEMV together, call after call
            operand = ops.Nvfp4DecodeOperand(8, k)
            operand.expand(x)
            case["prepared_us"] = _graph_time_us(torch, lambda i: plan.run_prepared(operand, ws[i % copies], out=y), args.steps)
            case["prepared_frac_of_hbm_peak"] = nbytes / case["prepared_us"] / 1e3 / peaks["hbm_gbs"]
            case["expand_plus_prepared_us"] = _graph_time_us(
                torch, lambda i: plan.run_prepared(operand.expand(x), ws[i % copies], out=y), args.steps)
            assert plan.status() == 0
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
        case = {"op": "fp8_w8a8_decode", "M": tokens, "K": k, "N": n, "us": us, "bytes": nbytes,
                "gbs": nbytes / us / 1e3, "frac_of_hbm_peak": nbytes / us / 1e3 / peaks["hbm_gbs"],
                "tflops": 2.0 * tokens * n * k / us / 1e6}
        # the same linear on activations their producer has already quantized (codes + one scale per token)
        xq, xs = ops.quantize_fp8_dynamic(x)
        case["quantized_us"] = _graph_time_us(torch, lambda i: plan.run_quantized(xq, xs, wq[i % copies], sw, out=y), args.steps)
        case["quantized_frac_of_hbm_peak"] = (nbytes - tokens * k) / case["quantized_us"] / 1e3 / peaks["hbm_gbs"]
        assert plan.status() == 0
        out["cases"].append(case)
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


def measure_moe(torch, dist, world, rank, steps, warmup, stages=True):
    """Routed-MoE prefill (4096 tokens, 128 experts, top-8, hidden 2048, intermediate 768).  One GPU: the staged pipeline;
    N > 1: experts split evenly, tokens sharded by rows, routes dispatched and returned by peer stores with device-resident
    counts, the whole step replayed as a CUDA graph.  Returns the dict of the JSON line (rank 0) or None."""
    from eider_b200 import ops, parallel
    t, e, k8, h, inter = 4096, 128, 8, 2048, 768
    tl = t // world
    g = torch.Generator(device="cuda").manual_seed(0)
    x_all = torch.randn(t, h, device="cuda", generator=g).to(torch.bfloat16)
    logits_all = torch.randn(t, e, device="cuda", generator=g)
    per = e // world
    gw = torch.Generator(device="cuda").manual_seed(100 + rank)
    w_gu = ops.GroupedNvfp4Weights.quantize(torch.randn(per, 2 * inter, h, device="cuda", generator=gw) * 0.02)
    w_dn = ops.GroupedNvfp4Weights.quantize(torch.randn(per, h, inter, device="cuda", generator=gw) * 0.02)
    x = x_all[rank * tl:(rank + 1) * tl].contiguous()
    logits = logits_all[rank * tl:(rank + 1) * tl].contiguous()
    stream = torch.cuda.Stream()
    flops = 2.0 * t * k8 * (h * 2 * inter + inter * h)

    def timed(fn, iters):
        graph = _graph_of(torch, lambda i: fn(), iters, stream)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = float("inf")
        with torch.cuda.stream(stream):
            graph.replay()
            for _ in range(3):
                if world > 1:
                    dist.barrier()
                torch.cuda.synchronize()
                if world > 1:
                    layer.barrier.arrive_and_wait(2)
                e0.record()
                graph.replay()
                e1.record()
                torch.cuda.synchronize()
                ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
                if world > 1:
                    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
                best = min(best, float(ms.item()))
        return best / iters * 1e3

    if world == 1:
        moe = ops.GroupedMoe(t, e, k8, h, inter)
        w_gu_i = w_gu.interleave_gate_up()  # once, at load: lets the gate/up GEMM's epilogue run the SiLU * up quantizer
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                moe.run(x, logits, w_gu, w_dn, w_gate_up_interleaved=w_gu_i)
        total = timed(lambda: moe.run(x, logits, w_gu, w_dn, w_gate_up_interleaved=w_gu_i), steps)
        staged_total = timed(lambda: moe.run(x, logits, w_gu, w_dn), steps)
        assert moe.gate_up_plan.status() == 0 and moe.down_plan.status() == 0
        out = {"metric": "moe_prefill_tflops", "value": flops / total / 1e6, "unit": "TFLOP/s", "n_gpus": 1, "us_per_step": total,
               "us_per_step_unfused_silu": staged_total, "min_bytes_gbs": 375391232 / total / 1e3, "data": "synthetic",
               "timing": f"{steps} steps replayed as one CUDA graph, CUDA events, best of 3",
               "config": {"workload": "nvfp4 routed moe prefill: 4096 tokens, 128 experts, top-8, H=2048, I=768"}}
        if stages:
            idx, wts = ops.moe_topk(logits, k8, True)
            out["stage_us"] = {
                "topk": timed(lambda: ops.moe_topk(logits, k8, True), steps),
                "sort": timed(lambda: moe.routes.sort(idx.reshape(-1)), steps),
                "gather_quantize": timed(lambda: moe.gate_up_in.gather_quantize(x, moe.routes, k8), steps),
                "gemm_gate_up_silu_quantize_fused": timed(lambda: moe.gate_up_plan.run_silu_quantize(moe.gate_up_in, w_gu_i, moe.routes, moe.down_in), steps),
                "gemm_gate_up": timed(lambda: moe.gate_up_plan.run(moe.gate_up_in, w_gu, moe.routes, out=moe.gate_up_out), steps),
                "silu_mul_quantize": timed(lambda: moe.down_in.silu_mul_halves_quantize(moe.gate_up_out, moe.routes), steps),
                "gemm_down": timed(lambda: moe.down_plan.run(moe.down_in, w_dn, moe.routes, out=moe.down_out), steps),
                "combine": timed(lambda: ops.moe_weighted_accumulate(moe.routes, wts.reshape(-1), moe.down_out, t, k8, out=moe.out), steps),
            }
        return out
    layer, step = parallel.peer_expert_parallel_moe(None, tl, e, k8, h, inter, w_gu, w_dn)
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            step(x, logits)
        torch.cuda.synchronize()
    # parity gate: this rank's tokens through the single-GPU pipeline over ALL experts (every rank can regenerate every
    # rank's weights from the seeds) must equal what the expert-parallel step returns, bit for bit
    parts_gu, parts_dn = [], []
    for r in range(world):
        gr = torch.Generator(device="cuda").manual_seed(100 + r)
        parts_gu.append(ops.GroupedNvfp4Weights.quantize(torch.randn(per, 2 * inter, h, device="cuda", generator=gr) * 0.02))
        parts_dn.append(ops.GroupedNvfp4Weights.quantize(torch.randn(per, h, inter, device="cuda", generator=gr) * 0.02))
    cat = lambda parts: ops.GroupedNvfp4Weights.from_checkpoint(torch.cat([p.packed for p in parts]),
                                                                torch.cat([p.scales_row_major for p in parts]),
                                                                torch.cat([p.alpha for p in parts]))
    full_gu, full_dn = cat(parts_gu), cat(parts_dn)
    with torch.cuda.stream(stream):
        ref = ops.GroupedMoe(tl, e, k8, h, inter).run(x, logits, full_gu, full_dn, w_gate_up_interleaved=full_gu.interleave_gate_up()).clone()
        got = step(x, logits).clone()
        torch.cuda.synchronize()
    same = torch.tensor([1.0 if torch.equal(ref, got) else 0.0], device="cuda")
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    parity_ok = bool(same.item() == 1.0)
    del parts_gu, parts_dn, full_gu, full_dn, ref
    if not parity_ok:
        return {"metric": "moe_prefill_tflops", "error": "expert-parallel output differs from the single-GPU pipeline, nothing was timed"} if rank == 0 else None
    total = timed(lambda: step(x, logits), steps)
    compute = timed(lambda: layer.run_experts_and_return(), steps)  # the owner's share: two grouped GEMMs, SiLU quantizer, return stores
    # each phase replayed on its own (the buffers hold the last step's routes; peer stores included, no waiting in any of them)
    phase_us = {"route_sort_publish": timed(lambda: layer.route_and_publish(x, logits), steps),
                "offsets_quantize_dispatch": timed(lambda: layer.dispatch(), steps),
                "experts_and_return": compute,
                "combine": timed(lambda: layer.combine(), steps),
                "barrier": timed(lambda: layer.barrier.arrive_and_wait(3), steps)}
    assert layer.status() == 0
    layer.barrier.check()
    received = torch.tensor([float(layer.recv_total.item())], device="cuda")
    most = received.clone()
    dist.all_reduce(received, op=dist.ReduceOp.SUM)
    dist.all_reduce(most, op=dist.ReduceOp.MAX)
    assert int(received.item()) == t * k8, "routes were lost on the way"
    if rank != 0:
        return None
    route_bytes_out, route_bytes_back = h * 9 // 16, 2 * h
    return {"metric": "moe_prefill_tflops", "value": flops / total / 1e6, "unit": "TFLOP/s", "n_gpus": world, "us_per_step": total,
            "experts_and_return_us": compute, "phase_us": phase_us,
            "parity": {"bit_identical_to_single_gpu_pipeline": True, "checked": "every rank's tokens, all experts"},
            "most_routes_on_one_rank": int(most.item()), "routes": t * k8,
            "nvlink_bytes_per_rank": (world - 1) / world * tl * k8 * (route_bytes_out + route_bytes_back),
            "partition": f"experts split evenly x{world}, tokens sharded by rows, NVFP4 rows dispatched and bf16 rows returned by peer "
                         "stores over NVLink, counts resident on the device, three bounded device barriers per step (two alternating buffer sets)",
            "timing": f"{steps} steps replayed as one CUDA graph per rank, ranks aligned on the device, max over ranks, best of 3",
            "data": "synthetic", "config": {"workload": "nvfp4 routed moe prefill: 4096 tokens, 128 experts, top-8, H=2048, I=768",
                                            "n_shards": world}}


def config_moe(args):
    """--config moe [--gpus N]: the routed-MoE layer on one GPU or expert-parallel on N."""
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
    out = measure_moe(torch, dist, world, rank, args.steps, max(3, args.warmup))
    if out is not None:
        print(json.dumps(out), flush=True)
    if dist:
        dist.destroy_process_group()


def config_sweep(args):
    """--config sweep: the large dense W4A4 sweep on one GPU, M in {128, 512, 2048, 8192, 16384} x {(K 5120, N 27648), (K 13824,
    N 5120)}; a step = per-row-scale quantizer + GEMM, replayed as a CUDA graph; rotating weight copies larger than L2."""
    import torch
    from eider_b200 import ops
    peaks = load_peaks()
    cases = []
    for (k, n) in [(5120, 27648), (13824, 5120)]:
        copies = 4
        ws = [ops.ModelOptWeight.quantize(torch.randn(n, k, device="cuda") * 0.02) for _ in range(copies)]
        for m in (128, 512, 2048, 8192, 16384):
            x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
            xq = ops.Nvfp4Matrix.zeros(m, k, "cuda", row_scales=True)
            y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            plan = ops.Fp4TnMatmulPlan(m, n, k)

            def step(i):
                ops.quantize_nvfp4_rowscale(x, out=xq)
                plan.run(xq, ws[i % copies], out=y)

            iters = max(4, min(args.steps, int(4000 / max(1.0, m / 64))))
            # the large cases run into the power cap and the SM clock takes about a second to come back: without a pause the
            # case measured next inherits the lowered clock (measured: 35.4 us instead of 24.7 us for M = 512, K = 13824)
            torch.cuda.synchronize()
            time.sleep(2.0)
            us_step = _graph_time_us(torch, step, iters, reps=3)
            torch.cuda.synchronize()
            time.sleep(2.0)
            us_gemm = _graph_time_us(torch, lambda i: plan.run(xq, ws[i % copies], out=y), iters, reps=3)
            assert plan.status() == 0
            fl = 2.0 * m * n * k
            nbytes = n * k * 9 / 16 + m * k * 9 / 16 + 2.0 * m * n
            cases.append({"M": m, "K": k, "N": n, "tile_code": plan.block_n, "step_us": us_step, "gemm_us": us_gemm,
                          "gemm_tflops": fl / us_gemm / 1e6, "step_tflops": fl / us_step / 1e6,
                          "gemm_frac_of_nominal_9pf": fl / us_gemm / 1e6 / NOMINAL_NVFP4_TFLOPS,
                          "gemm_frac_of_4x_measured_bf16": fl / us_gemm / 1e6 / (4.0 * peaks["bf16_tflops"]),
                          "gemm_gbs_at_min_bytes": nbytes / us_gemm / 1e3,
                          "bound": "hbm" if m < 512 else "tensor"})
            del x, xq, y, plan
        del ws
    print(json.dumps({"metric": METRIC, "unit": UNIT, "n_gpus": 1, "data": "synthetic", "config": {"workload": "dense NVFP4 W4A4 sweep"},
                      "timing": "CUDA-graph replay, best of 3, 4 rotating weight copies, 2 s idle before every measurement (clock recovery after a power-capped case)", "peak_hbm_gbs": peaks["hbm_gbs"],
                      "peak_source": peaks["source"], "cases": cases}), flush=True)


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
    ap.add_argument("--config", default="prefill", choices=["prefill", "decode", "moe", "fp8", "sweep"],
                    help="prefill (default, the contract line), or the single-GPU decode / MoE / FP8 GEMM configs")
    ap.add_argument("--tokens", type=int, default=0, help="prefill only: M instead of 512 (the larger-chunk configs)")
    ap.add_argument("--no-multicast", action="store_true", help="N > 1: one store per peer instead of one multimem.st per tile")
    ap.add_argument("--multicast", action="store_true", help="N > 1: one multimem.st per tile also below eight ranks")
    ap.add_argument("--no-extra", action="store_true", help="skip the short decode / larger-chunk measurements of the default line")
    ap.add_argument("--in-features", type=int, default=0, help="prefill only: K instead of 5120 (13824 with --out-features 5120 = the down projection)")
    ap.add_argument("--out-features", type=int, default=0, help="prefill only: N instead of 27648")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.tokens or args.in_features or args.out_features:
        global M, K, N, WORKLOAD, FLOPS_PER_STEP, NCU_DRAM_BYTES_FULL_LAUNCH
        M = args.tokens or M
        K = args.in_features or K
        N = args.out_features or N
        WORKLOAD = f"nvfp4_w4a4_prefill_gemm_M{M}_K{K}_N{N}"
        FLOPS_PER_STEP = 2.0 * M * N * K
        NCU_DRAM_BYTES_FULL_LAUNCH = None  # the ncu capture belongs to the default shape only
    if args.impl != "reference" and args.config == "decode":
        return config_decode(args)
    if args.impl != "reference" and args.config == "moe":
        return config_moe(args)
    if args.impl != "reference" and args.config == "fp8":
        return config_fp8_gemm(args)
    if args.impl != "reference" and args.config == "sweep":
        return config_sweep(args)

    if args.impl == "reference":
        reference_arm(args)
        return

    run_prefill(args)


def _graph_of(torch, fn, iters, stream):
    """`iters` calls of fn(i) captured as one CUDA graph on `stream` (after three eager calls)."""
    with torch.cuda.stream(stream):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(iters):
                fn(i)
    torch.cuda.synchronize()
    return graph


def run_prefill(args):
    import numpy as np
    import torch

    from eider_b200 import ops, parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if args.gpus != world and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}; using {world}", file=sys.stderr)
    peaks = load_peaks()
    steps = args.steps

    # ---- synthetic inputs (seed 0): weights quantized the ModelOpt way on the device --------------------
    n_local = N // world
    assert N % (world * 128) == 0, "N shards must be multiples of 128 rows"
    shard_mib = n_local * K * 9 / 16 / 2**20
    l2_mib = torch.cuda.get_device_properties(local_rank).L2_cache_size / 2**20
    rotate = max(4, int(2.0 * l2_mib / shard_mib) + 1)  # rotating weight copies: at least twice the L2 in total

    def shard_weights(copy: int, shard: int):
        """Weight rows [shard * n_local, (shard + 1) * n_local) of weight copy `copy`: any rank can regenerate any shard."""
        wgen = torch.Generator(device="cuda").manual_seed(1000 + 64 * copy + shard)
        w = torch.randn(n_local, K, device="cuda", generator=wgen) * 0.02
        return ops.ModelOptWeight.quantize(w)

    weights = [shard_weights(r, rank) for r in range(rotate)]
    x_host = torch.randn(M, K, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).pin_memory()
    x_dev = x_host.cuda()
    xq = ops.Nvfp4Matrix.zeros(M, K, "cuda", row_scales=True)
    y_local = torch.empty(M, n_local, dtype=torch.bfloat16, device="cuda")
    plan_local = ops.Fp4TnMatmulPlan(M, n_local, K)  # writes this rank's slab only (compute-only timing, NCCL path)
    if args.block_n:
        plan_local.set_block_n(args.block_n)
    current = {"w": weights[0]}

    def local_linear(x):
        ops.quantize_nvfp4_rowscale(x, out=xq)
        return (sharded.active_plan or plan_local).run(xq, current["w"], out=y_local)

    sharded = parallel.ColumnShardedLinear(N, local_linear)
    gather = "none" if world == 1 else "nccl"
    if world > 1 and args.gather in ("fused", "auto"):
        try:
            fused_plans = [ops.Fp4TnMatmulPlan(M, n_local, K) for _ in range(2)]  # two output buffers: one barrier per step
            for q in fused_plans:
                if args.block_n:
                    q.set_block_n(args.block_n)
                elif M > 128 and q.block_n not in (512, 384):
                    q.set_block_n(512)  # the CTA-pair kernels stage whole tiles for the stores that leave the GPU
            # one multimem.st per tile pays from eight ranks on (measured: one TMA store per peer is faster on two and four)
            use_multicast = (not args.no_multicast) and (world >= 8 or args.multicast)
            sharded.fuse_into(fused_plans, M, multicast=use_multicast)
            gather = "fused-multicast" if sharded.multicast else "fused"
        except Exception as exc:  # symmetric memory is not available on this box: keep the NCCL path
            if rank == 0:
                print(f"# fused all-gather unavailable ({type(exc).__name__}: {exc}); using NCCL", file=sys.stderr)
    result = {}

    def step(i, x):
        current["w"] = weights[i % rotate]
        y = sharded.forward(x)  # N > 1: every rank ends up with row-major [M, N]
        result["y"] = y if (world == 1 or gather != "nccl") else y.contiguous()

    def host_barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    align = parallel.PeerBarrier() if (world > 1 and gather != "nccl") else None
    stream = torch.cuda.Stream()

    def timed_graph(fn, iters, reps=3):
        """Device time in ms of `iters` calls of fn(i) replayed as one CUDA graph, ranks aligned on the device right
        before the first event; best of `reps`, max over ranks."""
        graph = _graph_of(torch, fn, iters, stream)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = float("inf")
        with torch.cuda.stream(stream):
            graph.replay()
            for _ in range(reps):
                host_barrier()
                if align is not None:
                    align.arrive_and_wait(2)
                e0.record()
                graph.replay()
                e1.record()
                host_barrier()
                ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
                if world > 1:
                    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
                best = min(best, float(ms.item()))
        return best

    # ---- parity gate: the timed weights, checked against the host path before anything is timed ---------------
    def check_parity():
        """One step on weight copy 0 against the host product; -> (ok on every rank, parity dict on rank 0, cpu_baseline dict)."""
        with torch.cuda.stream(stream):
            step(0, x_dev)
            torch.cuda.synchronize()
            y_check = result["y"].float().cpu().numpy()
        parity, cpu_line = None, None
        if rank == 0:
            from oracle import oracle as o
            xp, xs, xr = xq.packed.cpu().numpy(), xq.scales.cpu().numpy(), xq.row_scales.cpu().numpy()
            a = o.dequantize_tiled(xp, xs) * xr[:, None]
            if world == 1:
                w0 = weights[0]
                ref, seconds, cols = cpu_reference_product(a, w0.packed.cpu().numpy(), w0.scales_row_major.cpu().numpy(), w0.weight_scale_2,
                                                           cols=None if not args.no_cpu_baseline else 1024)
                parity = parity_report(y_check[:, :cols], ref)
                sample = (f"the whole workload ({M} tokens x K={K} x {N} output features; unpack + f32 triple loop)" if cols == N else
                          f"all {M} tokens x all K={K} x first {cols} of {N} output features (unpack + f32 triple loop)")
                cpu_line = {"value": 2.0 * M * cols * K / seconds / 1e12, "unit": UNIT, "cores": o.max_threads(), "kind": "port",
                            "sample": sample, "seconds": seconds}
            else:
                # the gathered [M, N] on rank 0: the first and last 128 columns of every rank's block, weights regenerated here
                got, want = [], []
                for shard in range(world):
                    ws_ = shard_weights(0, shard)
                    wp_h, ws_h = ws_.packed.cpu().numpy(), ws_.scales_row_major.cpu().numpy()
                    for c0 in (0, n_local - 128):
                        ref, _, _ = cpu_reference_product(a, wp_h[c0:c0 + 128], ws_h[c0:c0 + 128], ws_.weight_scale_2, cols=128)
                        want.append(ref)
                        got.append(y_check[:, shard * n_local + c0: shard * n_local + c0 + 128])
                    del ws_
                parity = parity_report(np.concatenate(got, axis=1), np.concatenate(want, axis=1))
                parity["columns"] = "first and last 128 columns of every rank's block of the gathered output on rank 0"
        ok = torch.tensor([1 if (parity is None or parity["bad"] == 0) else 0], device="cuda")
        if world > 1:
            dist.broadcast(ok, 0)
        return bool(int(ok.item())), parity, cpu_line

    ok, parity, cpu_line = check_parity()
    if not ok and gather == "fused-multicast":
        # the multicast epilogue is the newest path: fall back to one store per peer rather than give up on the run
        if rank == 0:
            print(f"# multicast all-gather failed the parity check ({parity}); falling back to per-peer stores", file=sys.stderr)
        for q in fused_plans:
            q.set_output_multicast(0)
        sharded.multicast = False
        gather = "fused"
        ok, parity, cpu_line = check_parity()
    if not ok:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "error": "parity check failed, nothing was timed", "parity": parity}), flush=True)
        if dist:
            dist.destroy_process_group()
        sys.exit(3)

    # ---- the timed region: W warm-up steps, then exactly K steps ---------------------------------------------------
    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            step(i, x_dev)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    total_ms = timed_graph(lambda i: step(i, x_dev), steps)
    ms_per_step = total_ms / steps
    value = FLOPS_PER_STEP / (ms_per_step * 1e-3) / 1e12

    # ---- kernels alone, each as one graph of launches ----------------------------------------------------------
    active = sharded.active_plan or plan_local
    gemm_ms = timed_graph(lambda i: active.run(xq, weights[i % rotate], out=y_local), steps) / steps  # as in the step (peer stores included)
    gemm_local_ms = (timed_graph(lambda i: plan_local.run(xq, weights[i % rotate], out=y_local), steps) / steps) if world > 1 else gemm_ms
    quant_ms = timed_graph(lambda i: ops.quantize_nvfp4_rowscale(x_dev, out=xq), steps) / steps
    barrier_ms = (timed_graph(lambda i: sharded._barrier.arrive_and_wait(3), steps) / steps) if (world > 1 and gather != "nccl") else 0.0
    if rank == 0:
        clocks = sampler.stop()
    status = active.status()
    assert status == 0, f"GEMM kernel reported status {status:#x}"
    sharded.check()

    # ---- end to end through the public API with host buffers ------------------------------------------------
    # (steps are streamed: the upload of step i + 1 and the download of step i - 1 run on their own streams while step i
    # computes, two buffer sets; every step's copies are inside the timed region)
    from eider_b200 import host_io
    rows_lo, rows_hi = (rank * M) // world, ((rank + 1) * M) // world  # N > 1: every rank returns its share of the rows
    y_hosts = [torch.empty(rows_hi - rows_lo, N, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    streamer = host_io.HostStreamer(tuple(x_dev.shape), x_dev.dtype, (rows_hi - rows_lo, N), torch.bfloat16, depth=2)
    e2e_count = [0]

    def e2e_compute(x):
        step(e2e_count[0], x)
        return result["y"]

    def e2e_step():
        streamer.submit(x_host, e2e_compute, y_hosts[e2e_count[0] % 2], take=lambda y: y[rows_lo:rows_hi])
        e2e_count[0] += 1

    with torch.cuda.stream(stream):
        for i in range(3):
            e2e_step()
        streamer.drain()
        host_barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if align is not None:
            align.arrive_and_wait(2)
        e0.record()
        streamer.start_after(e0)
        for i in range(steps):
            e2e_step()
        streamer.drain()
        e1.record()
        host_barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        # what came back over PCIe for the last step against what the device holds for that step
        e2e_same = bool(torch.equal(y_hosts[(e2e_count[0] - 1) % 2], result["y"][rows_lo:rows_hi].cpu()))
    e2e_ms = float(ms.item()) / steps
    e2e_value = FLOPS_PER_STEP / (e2e_ms * 1e-3) / 1e12

    # ---- N > 1: the unsharded step on this GPU, for the compute-only and end-to-end speed-ups ---------------------
    detail = None
    if world > 1:
        full_w = []
        for r in range(4):
            wgen = torch.Generator(device="cuda").manual_seed(5000 + r)
            full_w.append(ops.ModelOptWeight.quantize(torch.randn(N, K, device="cuda", generator=wgen) * 0.02))
        y_full = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        plan_full = ops.Fp4TnMatmulPlan(M, N, K)

        def single_step(i):
            ops.quantize_nvfp4_rowscale(x_dev, out=xq)
            plan_full.run(xq, full_w[i % 4], out=y_full)

        single_ms = timed_graph(single_step, steps) / steps
        single_gemm_ms = timed_graph(lambda i: plan_full.run(xq, full_w[i % 4], out=y_full), steps) / steps
        nvlink_bound_us = (world - 1) / world * 2.0 * M * N / 770e9 * 1e6
        detail = {"step_us": ms_per_step * 1e3, "gemm_us": gemm_ms * 1e3, "gemm_without_peer_stores_us": gemm_local_ms * 1e3,
                  "quantize_us": quant_ms * 1e3, "barrier_us": barrier_ms * 1e3,
                  "other_us": (ms_per_step - gemm_ms - quant_ms - barrier_ms) * 1e3,
                  "single_gpu_step_us": single_ms * 1e3,
                  "compute_only_speedup": single_ms / (gemm_local_ms + quant_ms),
                  # the activation quantizer is replicated on every rank (each needs all of x); the GEMM alone:
                  "single_gpu_gemm_us": single_gemm_ms * 1e3,
                  "gemm_only_speedup": single_gemm_ms / gemm_local_ms,
                  "end_to_end_speedup": single_ms / ms_per_step,
                  "nvlink_bound_us": nvlink_bound_us,
                  "nvlink_bound_note": f"every rank receives (g-1)/g * 2MN = {(world - 1) / world * 2.0 * M * N / 1e6:.1f} MB per step; "
                                       "at the measured 770 GB/s per direction that alone takes this long, whatever g is"}
        del full_w, y_full

    extra = {}
    if rank == 0 and world == 1 and not args.no_extra:
        extra = single_gpu_extras(args, torch, ops, peaks)
    if not args.no_extra:
        try:
            moe = measure_moe(torch, dist, world, rank, 10, 3, stages=False)  # (every rank takes part)
            if moe is not None:
                extra["moe" if world == 1 else "moe_ep"] = moe
        except Exception as exc:
            if rank == 0:
                extra["moe" if world == 1 else "moe_ep"] = {"error": f"{type(exc).__name__}: {exc}"}

    if rank != 0:
        if dist:
            dist.destroy_process_group()
        return

    gemm_flops_local = 2.0 * M * n_local * K
    achieved = gemm_flops_local / (gemm_ms * 1e-3) / 1e12
    nvfp4_peak = 4.0 * peaks["bf16_tflops"]
    roofline = {
        "bound": "tensor",
        "kernel": (f"gemm_pair_kernel<nvfp4> (tcgen05.mma cta_group::2 kind::mxf4nvf4.block_scale, 256x{256 if active.block_n == 512 else 192} tiles on CTA pairs)"
                   if active.block_n in (512, 384) else
                   f"gemm_kernel<nvfp4, {active.block_n}> (tcgen05.mma kind::mxf4nvf4.block_scale)"),
        "achieved": achieved, "peak": nvfp4_peak, "unit": "TFLOP/s", "frac": achieved / nvfp4_peak,
        "peak_source": f"4 x {peaks['source']} dense bf16 burst ({peaks['bf16_tflops']} TF/s); NVFP4 is not measured by the driver",
        "frac_of_nominal_9pf": achieved / NOMINAL_NVFP4_TFLOPS,
        "kernel_ms": gemm_ms, "quantize_kernel_ms": quant_ms,
        "hbm_gbs_at_min_bytes": (n_local * K * 9 / 16 + M * K * 9 / 16 + 2.0 * M * n_local) / (gemm_ms * 1e-3) / 1e9,
        # dram__bytes_read + dram__bytes_write of one launch of this kernel at the full shape (one ncu capture of this
        # command), scaled by this rank's share of the weight rows
        "traffic": (NCU_DRAM_BYTES_FULL_LAUNCH * n_local / N) if NCU_DRAM_BYTES_FULL_LAUNCH else None, "traffic_unit": "bytes per launch",
    }
    partition = {"none": "one GPU", "nccl": f"N column-sharded x{world} + NCCL all-gather of bf16 outputs",
                 "fused": f"N column-sharded x{world}, all-gather fused into the GEMM epilogue (one TMA store per peer over NVLink)",
                 "fused-multicast": f"N column-sharded x{world}, all-gather fused into the GEMM epilogue (one multimem.st per tile, "
                                    "replicated by NVSwitch)"}[gather]
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "nvfp4(e2m1+ue4m3) x nvfp4, f32 accumulate, bf16 out", "data": "synthetic",
        "config": full_config(world),
        "partition": partition,
        "l2": f"inputs larger than L2 ({l2_mib:.0f} MiB): {rotate} rotating weight copies of {shard_mib:.1f} MiB each per GPU",
        "timing": f"{steps} steps replayed as one CUDA graph per rank, ranks aligned on the device before the first event, "
                  "CUDA events on the launching stream, max over ranks",
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": M * K * 2 * world,
                "d2h_bytes_per_step": M * N * 2,
                "note": ("weights stay resident in HBM (model state); every rank copies X from pinned host memory and returns its "
                         "share of the rows of Y to pinned host memory" if world > 1 else
                         "weights stay resident in HBM (model state); X from and Y to pinned host memory") +
                        "; steps streamed (eider_b200.host_io.HostStreamer): the upload of step i+1 and the download of step i-1 "
                        "overlap step i on their own streams, two buffer sets",
                "last_result_matches_device": e2e_same},
        "gpu_launches": (2 + (1 if barrier_ms else 0)) * steps, "clocks": clocks, "roofline": roofline, "parity": parity,
    }
    if cpu_line is not None:
        line["cpu_baseline"] = cpu_line
    if detail is not None:
        line["scaling_detail"] = detail
    if extra:
        line["extra"] = extra
    print(json.dumps(line), flush=True)
    if dist:
        dist.destroy_process_group()


def single_gpu_extras(args, torch, ops, peaks):
    """Short measurements of the other configs on one GPU, folded into the default line: decode GEMV (HBM GB/s), the
    4096-token prefill chunk and the routed-MoE layer."""
    extra = {}
    copies = 6
    cases = []
    for op, tokens, n, k in [("nvfp4_w4a16_decode", 1, 13824, 5120), ("fp8_w8a8_decode", 1, 7168, 5120), ("fp8_w8a8_decode", 8, 7168, 5120),
                             ("fp8_w8a8_decode", 32, 7168, 5120), ("fp8_w8a8_decode", 64, 7168, 5120)]:
        x = torch.randn(tokens, k, device="cuda").to(torch.bfloat16)
        y = torch.empty(tokens, n, dtype=torch.bfloat16, device="cuda")
        if op.startswith("nvfp4"):
            ws = [ops.ModelOptWeight.quantize(torch.randn(n, k, device="cuda") * 0.02) for _ in range(copies)]
            plan = ops.Nvfp4DecodePlan(tokens, n, k)
            us = _graph_time_us(torch, lambda i: plan.run(x, ws[i % copies], out=y), 50)
            nbytes = n * k // 2 + n * k // 16 + 2 * tokens * k + 2 * tokens * n + 4
            # the same GEMV on an operand the producer of x has expanded once (shared by every linear that reads x)
            operand = ops.Nvfp4DecodeOperand(8, k).expand(x)
            prepared_us = _graph_time_us(torch, lambda i: plan.run_prepared(operand, ws[i % copies], out=y), 50)
        else:
            ws = [torch.randint(0, 120, (n, k), dtype=torch.uint8, device="cuda") for _ in range(copies)]
            sw = torch.rand(n, device="cuda") * 0.01
            plan = ops.Fp8DecodePlan(64, n, k)
            us = _graph_time_us(torch, lambda i: plan.run(x, ws[i % copies], sw, out=y), 50)
            nbytes = n * k + 4 * n + 2 * tokens * k + 2 * tokens * n
            # the same linear on activations their producer has already quantized (codes + one scale per token)
            xq, xs = ops.quantize_fp8_dynamic(x)
            prepared_us = _graph_time_us(torch, lambda i: plan.run_quantized(xq, xs, ws[i % copies], sw, out=y), 50)
        assert plan.status() == 0
        cases.append({"op": op, "M": tokens, "K": k, "N": n, "us": us, "gbs": nbytes / us / 1e3,
                      "frac_of_hbm_peak": nbytes / us / 1e3 / peaks["hbm_gbs"], "prepared_activation_us": prepared_us,
                      "prepared_activation_frac_of_hbm_peak": nbytes / prepared_us / 1e3 / peaks["hbm_gbs"]})
        del ws
    extra["decode"] = {"unit": "GB/s of the algorithmic bytes", "peak_hbm_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"],
                       "timing": f"CUDA-graph replay of 50 calls, {copies} rotating weight copies",
                       "prepared_activation": "the same GEMV on an activation its producer has expanded (NVFP4) or quantized (FP8) once",
                       "cases": cases}
    # the 4096-token chunk of the sweep
    m4 = 4096
    ws = [ops.ModelOptWeight.quantize(torch.randn(N, K, device="cuda") * 0.02) for _ in range(3)]
    x4 = torch.randn(m4, K, device="cuda").to(torch.bfloat16)
    xq4 = ops.Nvfp4Matrix.zeros(m4, K, "cuda", row_scales=True)
    y4 = torch.empty(m4, N, dtype=torch.bfloat16, device="cuda")
    plan4 = ops.Fp4TnMatmulPlan(m4, N, K)

    def step4(i):
        ops.quantize_nvfp4_rowscale(x4, out=xq4)
        plan4.run(xq4, ws[i % 3], out=y4)

    us_step = _graph_time_us(torch, step4, 10, reps=3)
    us_gemm = _graph_time_us(torch, lambda i: plan4.run(xq4, ws[i % 3], out=y4), 10, reps=3)
    assert plan4.status() == 0
    fl = 2.0 * m4 * N * K
    extra["prefill_m4096"] = {"step_us": us_step, "gemm_us": us_gemm, "step_tflops": fl / us_step / 1e6, "gemm_tflops": fl / us_gemm / 1e6,
                              "gemm_frac_of_nominal_9pf": fl / us_gemm / 1e6 / NOMINAL_NVFP4_TFLOPS,
                              "gemm_frac_of_4x_measured_bf16": fl / us_gemm / 1e6 / (4.0 * peaks["bf16_tflops"])}
    del ws, y4
    return extra


if __name__ == "__main__":
    main()
