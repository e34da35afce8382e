#!/usr/bin/env python3
"""Benchmark of the MoE-layer hot path (MoELayerPlugin::enqueue) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one forward pass of the MoE layer over one batch of synthetic input.
With N = 1 the workload is the CPM-2-style layer the headline metric is quoted on
(E=32, d_model=4096, d_ff=10240, 8x512 tokens, all experts resident).  With N > 1
(launched under torch.distributed.run, one rank per GPU) the experts are sharded
expert-parallel, every rank keeps the same number of local tokens and local
experts (weak scaling), and rows and results move by peer stores over NVLink
(infmoe_ep_forward; NCCL only as the barrier).

One JSON line is printed by rank 0.  `value` is whole-job tokens/s with the input
already in HBM, timed on the device with CUDA events (max over ranks); `e2e` is
the same metric through the host-buffer entry point of the C ABI with the
host<->device copies inside the timed region, one blocking call per step; beside
it `e2e.two_in_flight` (infmoe_layer_submit_host / infmoe_ep_submit_host and
the matching _wait_host: two steps in flight from one context) and, at N = 1,
`e2e.two_contexts` (two clones driven by two host threads) give the rate when a
step's copies may overlap its neighbours' passes.  `roofline` describes
the dominant kernel (the gated wi_0/wi_1 grouped GEMM): `frac` against the
ceiling of the MMAs it issues, `frac_3xtf32` against plain 3xTF32; `cpu_baseline`
is the CPU restatement of the reference's math timed on this box's host cores on
a bounded sample.  N > 1 adds `per_rank` (expert time, wait time, received rows
and SM clock of every rank) and the fixed-size 128-expert case under `ep_cpm2`.

--impl reference times that CPU restatement alone (the reference itself has no CPU
path and its TensorRT plugin cannot be built here), on all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from infmoe_b200 import synth  # noqa: E402

# DRAM bytes the wi_0/wi_1 GEMM moves per weight element: dram__bytes_read.sum + dram__bytes_write.sum of one ncu
# capture of workload cpm2_profile (profiles/ffn_umma_kernel_cpm2_profile.md) divided by the weight elements that
# launch streams; 4 = each raw FP32 weight crosses HBM once.  It is a figure from that capture, scaled by the
# elements this launch streams -- it is not measured by this run.
TRAFFIC_BYTES_PER_WEIGHT = 4.27
TRAFFIC_SOURCE = "ncu capture of cpm2_profile (profiles/ffn_umma_kernel_cpm2_profile.md), bytes per weight element x elements streamed"

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()      # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = max(mx, float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU arm: the restatement of the reference's math on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_sample_setup(w: synth.Workload, sample_experts: int, tokens_per_expert: int):
    """A bounded slice of workload `w`: `sample_experts` experts and the tokens they would get."""
    from oracle import oracle

    # all host cores, whatever OMP_NUM_THREADS says (torchrun sets it to 1 for every rank)
    oracle.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    ws = synth.scaled(w, expert_count=sample_experts, batch=1, seq_len=sample_experts * tokens_per_expert)
    x, cent, ln = synth.gen_inputs(ws)
    experts = [synth.gen_expert_numpy(ws, e) for e in range(sample_experts)]
    return oracle, ws, x, cent, ln, experts


def cpu_step(oracle, ws, x, cent, ln, experts):
    t0 = time.perf_counter()
    oracle.layer_forward_f32(x, ws.variant, cent, ln, experts)
    return time.perf_counter() - t0


def run_reference_arm(args, w, scaling="weak"):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_experts = 2 if w.embedding_size * w.hidden_size > (1 << 24) else min(w.expert_count, 4)
    tpe = max(1, min(w.tokens // w.expert_count, 128))
    oracle, ws, x, cent, ln, experts = cpu_sample_setup(w, sample_experts, tpe)
    for _ in range(args.warmup):
        cpu_step(oracle, ws, x, cent, ln, experts)
    t = sum(cpu_step(oracle, ws, x, cent, ln, experts) for _ in range(args.steps))
    value = ws.tokens * args.steps / t
    sample = (f"{sample_experts} of {w.expert_count} experts x {tpe} tokens of workload {w.name} per step, "
              f"weights in host memory")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps, "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference's math (oracle/oracle.c, OpenMP + AVX2); the reference has no CPU "
                "path and its TensorRT plugin cannot be built on this box",
    }
    print(json.dumps(line), flush=True)


def workload_config(w, n_gpus):
    return {"workload": w.name, "moe_variant": w.variant, "expert_count": w.expert_count,
            "d_model": w.embedding_size, "d_ff": w.hidden_size,
            "tokens": w.tokens, "experts": "streamed" if w.streamed else "resident",
            "parallelism": f"ep{n_gpus}" if n_gpus > 1 else "single",
            "l2": "expert weights (GBs) stream through L2 every step; nothing is flushed explicitly"}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def build_layer(w, device, torch, cache_slots=0):
    from infmoe_b200 import MoELayer

    x, cent, ln = synth.gen_inputs(w)
    layer = MoELayer.create(w.expert_count, w.embedding_size, w.hidden_size, w.max_concurrency, cent, None, "T5_FF",
                            w.variant, ln)
    if w.streamed:
        for e in range(w.expert_count):
            ws = [t.cpu().numpy() for t in synth.gen_expert_torch(w, e, device)]
            layer.set_expert(e, *ws)
        layer.set_residency(0)
        if cache_slots:
            layer.set_expert_cache(cache_slots)
    else:
        for e in range(w.expert_count):
            layer.set_expert(e, *synth.gen_expert_torch(w, e, device))
        layer.set_residency(1)
    torch.cuda.synchronize()
    return layer, x, cent, ln


def ref_gpu_baseline(w, torch, sample_experts=8, reps=3):
    """Times the reference's own kernels + cuBLAS SGEMM in the order MoELayerPlugin::enqueue issues them
    (oracle/_ref, built from the reference checkout; the TensorRT plugin itself cannot be built here), on a bounded
    slice of workload `w`: `sample_experts` experts with their share of tokens.  Two figures: the literal behaviour
    (every used expert copied from pinned host memory on every call) and the same sequence with the copies sourced
    from device memory."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libinfmoe_ref_kernels.so")
    if not os.path.exists(path) or w.streamed:
        return None
    lib = ctypes.CDLL(path)
    tpe = max(1, w.tokens // w.expert_count)
    ws = synth.scaled(w, expert_count=sample_experts, batch=1, seq_len=sample_experts * tpe)
    T, D, E, F, mc = ws.tokens, ws.embedding_size, ws.expert_count, ws.hidden_size, ws.max_concurrency
    x, cent, ln = synth.gen_inputs(ws)
    dev = torch.device("cuda")
    dx, dc = torch.from_numpy(x).to(dev), torch.from_numpy(cent).to(dev)
    dl = torch.from_numpy(ln).to(dev) if ln is not None else None
    on_dev = [synth.gen_expert_torch(ws, e, dev) for e in range(E)]
    on_host = [[t.cpu().pin_memory() for t in ex] for ex in on_dev]
    nbytes = mc * (4 * D + 12 * D * F + 4 * T * (D + 2 * F)) + 4 * (T * E + 2 * T + 2 * T * D) + 8 * T + 1024
    wsp = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    out = torch.empty_like(dx)
    flags = (1 if ws.variant == "cpm_2" else 0) | (2 if ws.variant == "base_layer" else 0) | 4
    res = {}
    for label, src, kind in (("streamed_from_pinned_host", on_host, 0), ("weights_on_device", on_dev, 1)):
        tabs = [(ctypes.c_void_p * E)(*[ex[i].data_ptr() for ex in src]) for i in range(4)]
        def call():
            rc = lib.ref_layer_call(T, D, E, F, mc, flags, ctypes.c_void_p(dx.data_ptr()), ctypes.c_void_p(dc.data_ptr()),
                                    ctypes.c_void_p(dl.data_ptr() if dl is not None else 0), tabs[0], tabs[1], tabs[2],
                                    tabs[3], kind, ctypes.c_void_p(wsp.data_ptr()), ctypes.c_void_p(out.data_ptr()))
            assert rc == 0, rc
        call()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            call()
        res[label] = {"value": T * reps / (time.perf_counter() - t0), "unit": UNIT}
    res["sample"] = f"{E} of {w.expert_count} experts x {tpe} tokens of workload {w.name}, max_concurrency {mc}"
    res["what"] = ("reference kernels (moe.cu, layernorm.cu, gelu.cu) + cublasSgemm_v2 FP32, launch/copy/sync order of "
                   "MoELayerPlugin::enqueue restated; final gather reads the expert output")
    return res


def gemm_roofline(kernel, achieved_tflops, kernel_ms, peaks, clock_summary, timed_s):
    """Roofline object of the grouped expert GEMM.

    `peak` is the ceiling of the MMAs this kernel actually issues: per product one TF32 MMA (half the bf16 rate) and
    two BF16 MMAs with K = 16 (the bf16 rate), i.e. measured bf16 / 4.  The burst figure is the denominator while the
    timed region is short and the SM clock sampled during it stays near its maximum; a long region that runs into
    the power cap is held against the sustained figure.  `frac_3xtf32` is against what plain 3xTF32 (three TF32 MMAs
    per product, the arithmetic the kernel replaces) could reach: bf16 / 6."""
    sm, mx = clock_summary.get("sm_mhz"), clock_summary.get("sm_max_mhz")
    burst = timed_s < 1.0 and sm is not None and mx and sm >= 0.9 * mx
    bf16 = peaks["bf16_tflops"] if burst else peaks["bf16_sustained"]
    regime = "burst" if burst else "sustained"
    return {"kernel": kernel, "bound": "tensor", "achieved": achieved_tflops, "peak": bf16 / 4.0, "unit": "TFLOP/s",
            "frac": achieved_tflops / (bf16 / 4.0), "peak_3xtf32": bf16 / 6.0,
            "frac_3xtf32": achieved_tflops / (bf16 / 6.0),
            "peak_source": f"bf16 {regime} {bf16} TFLOP/s of {peaks['source']} / 4 (per product 1 TF32 MMA at half the "
                           f"bf16 rate + 2 BF16 K=16 MMAs); 3xTF32 = bf16 / 6; regime chosen from the timed region "
                           f"({timed_s:.2f} s) and the sampled SM clock ({sm} of {mx} MHz)",
            "ms": kernel_ms}


def routing_differences(w, x, cent, ln, gate, torch):
    """How many tokens of this workload the fused FP32 routing sends elsewhere than (a) an FP64 evaluation and (b)
    FP32 in cuBLAS's summation order followed by the reference's own select kernel (oracle/_ref, when it was
    built), with the largest top-1/top-2 score margin (FP64) among those tokens: the distance between the
    canonical summation order and the reference's, which only shows at near-ties."""
    import ctypes
    from oracle import oracle
    gamma = ln if w.variant == "cpm_2" else None
    g64, top1, top2 = oracle.route_f64(x, cent, gamma)
    margin = top1 - top2
    d64 = np.nonzero(g64 != gate)[0]
    res = {"tokens": int(gate.size), "fp64_flips": int(d64.size),
           "fp64_max_margin": float(margin[d64].max()) if d64.size else 0.0,
           "score_std": float(np.std(top1))}
    path = os.path.join(ROOT, "oracle", "_ref", "libinfmoe_ref_kernels.so")
    if os.path.exists(path):
        ref = ctypes.CDLL(path)
        T, D, E = x.shape[0], x.shape[1], cent.shape[0]
        dev = torch.device("cuda")
        dx, dc = torch.from_numpy(x).to(dev), torch.from_numpy(cent).to(dev)
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        if gamma is not None:
            dn = torch.empty_like(dx)
            assert ref.ref_layernorm(p(dn), p(dx), T, D, p(torch.from_numpy(gamma).to(dev))) == 0
            dx = dn
        aff = torch.empty(T, E, dtype=torch.float32, device=dev)
        assert ref.ref_gating_sgemm(T, D, E, p(dc), p(dx), p(aff)) == 0
        rg = torch.empty(T, dtype=torch.int32, device=dev)
        rw = torch.empty(T, dtype=torch.float32, device=dev)
        assert ref.ref_select(T, E, p(aff), p(rg), p(rw)) == 0
        torch.cuda.synchronize()
        dref = np.nonzero(rg.cpu().numpy() != gate)[0]
        res.update({"reference_order_flips": int(dref.size),
                    "reference_order_max_margin": float(margin[dref].max()) if dref.size else 0.0,
                    "reference_order": "layernorm_gpu + cublasSgemm_v2 + expert_select_top1_kernel (oracle/_ref)"})
    return res


def run_single(args, w):
    import torch

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    peaks = _peaks()
    layer, x, cent, ln = build_layer(w, dev, torch, args.cache_slots)
    T, D, F, E = w.tokens, w.embedding_size, w.hidden_size, w.expert_count
    hx = torch.from_numpy(x).pin_memory()
    hout = torch.empty_like(hx).pin_memory()
    dx = hx.to(dev)
    dout = torch.empty_like(dx)
    stream = torch.cuda.current_stream()

    # ---- device-resident timing ----
    clocks = ClockSampler(0)
    clocks.__enter__()      # sampling runs through warm-up and both timed regions
    for _ in range(args.warmup):
        layer.forward(dx, dout)
    layer.sync_status(stream.cuda_stream)
    layer.set_profiling(True)
    launches0 = layer.kernel_launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    if True:
        start.record(stream)
        for _ in range(args.steps):
            layer.forward(dx, dout)
        stop.record(stream)
        torch.cuda.synchronize()
    layer.sync_status(stream.cuda_stream)
    ms = start.elapsed_time(stop) / args.steps
    launches = layer.kernel_launches - launches0
    stage_ms, calls = layer.stage_ms()
    layer.set_profiling(False)

    # ---- end to end through the host-buffer entry point ----
    for _ in range(min(args.warmup, 3)):
        layer.forward_host_ptr(hx.data_ptr(), hout.data_ptr(), T)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        layer.forward_host_ptr(hx.data_ptr(), hout.data_ptr(), T)
    e2e_s = (time.perf_counter() - t0) / args.steps

    # ---- the same call from two execution contexts: a clone each, with its own stream and host buffers, driven by
    # ---- its own host thread (TensorRT gives every execution context a clone of the plugin).  The upload of one
    # ---- context's input runs behind the other's GEMMs.  Reported beside the one-context figure, not instead of it.
    # ---- the same steps with two in flight from ONE context (infmoe_layer_submit_host / _wait_host): a step's
    # ---- upload runs on a copy stream behind the pass of the step before
    two_in_flight = None
    if not w.streamed:
        hx_b, hout_b = hx.clone().pin_memory(), torch.empty_like(hx).pin_memory()
        bufs = [(hx, hout), (hx_b, hout_b)]
        for i in range(2):                      # warm-up: the first submission creates streams and staging buffers
            layer.submit_host_ptr(bufs[i][0].data_ptr(), bufs[i][1].data_ptr(), T)
        layer.wait_host()
        layer.wait_host()
        keep = hout.clone()
        hout.zero_()
        t0 = time.perf_counter()
        for i in range(args.steps):
            a, b = bufs[i & 1]
            layer.submit_host_ptr(a.data_ptr(), b.data_ptr(), T)
            if i >= 1:
                layer.wait_host()
        layer.wait_host()
        tif_s = (time.perf_counter() - t0) / args.steps
        two_in_flight = {"value": T / tif_s, "unit": UNIT, "ms_per_step": 1e3 * tif_s,
                         "same_output": bool(torch.equal(hout, keep))}

    two_ctx = None
    if not w.streamed and not args.no_two_contexts:
        import threading
        other = layer.clone()
        hx2, hout2 = hx.clone().pin_memory(), torch.empty_like(hx).pin_memory()
        other.forward_host_ptr(hx2.data_ptr(), hout2.data_ptr(), T)
        ctx = [(layer, hx, hout, (args.steps + 1) // 2), (other, hx2, hout2, args.steps // 2)]
        failed = []

        def drive(lay, hin, ho, n):
            try:
                for _ in range(n):
                    lay.forward_host_ptr(hin.data_ptr(), ho.data_ptr(), T)
            except Exception as e:      # noqa: BLE001 -- reported below, the line must still be printed
                failed.append(repr(e))

        threads = [threading.Thread(target=drive, args=c) for c in ctx]
        t0 = time.perf_counter()
        for th in threads:
            th.start()
        for th in threads:
            th.join()
        two_s = (time.perf_counter() - t0) / args.steps
        two_ctx = {"value": T / two_s, "unit": UNIT, "ms_per_step": 1e3 * two_s, "contexts": 2,
                   "same_output": bool(torch.equal(hout2, hout)), "errors": failed}
        other.terminate()
    clocks.__exit__()

    # ---- roofline of the dominant kernel (expert GEMM 1: wi_0 / wi_1 + gelu) ----
    gate_p = layer.last_routing()[0]
    from infmoe_b200.devmem import read_device
    gate = read_device(gate_p, T, np.int32)
    active = int(np.count_nonzero(np.bincount(gate, minlength=E)))
    g1_ms = stage_ms["ffn_gemm1"] if stage_ms["ffn_gemm1"] > 0 else None
    useful_flops = 4.0 * T * D * F                    # algorithmic flops of h wi_0^T and h wi_1^T
    clock_summary = clocks.summary()
    roofline = None
    if g1_ms:
        achieved = useful_flops / (g1_ms * 1e-3) / 1e12
        weight_bytes = (2 * D * F * 4.0) * active      # raw FP32 interleaved wi_0/wi_1 matrix of every active expert
        traffic = TRAFFIC_BYTES_PER_WEIGHT * active * 2.0 * F * D if not w.streamed else None
        roofline = gemm_roofline("ffn_umma_kernel<EPI_GELU_PAIR>", achieved, g1_ms, peaks, clock_summary,
                                 timed_s=ms * 1e-3 * args.steps)
        roofline.update({"traffic": traffic, "traffic_source": TRAFFIC_SOURCE if traffic else None,
                         "algorithmic_bytes": weight_bytes, "weight_stream_gbs": weight_bytes / (g1_ms * 1e-3) / 1e9,
                         "hbm_peak_gbs": peaks["hbm_gbs"], "hbm_frac": weight_bytes / (g1_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]})

    # ---- CPU baseline on a bounded sample ----
    cpu = None
    if not args.no_cpu:
        sample_experts = 2
        tpe = max(1, min(T // E, 128))
        oracle, ws, cx, ccent, cln, cexp = cpu_sample_setup(w, sample_experts, tpe)
        cpu_step(oracle, ws, cx, ccent, cln, cexp)
        reps, t = 0, 0.0
        while t < 10.0 and reps < 20:
            t += cpu_step(oracle, ws, cx, ccent, cln, cexp)
            reps += 1
        cpu = {"value": ws.tokens * reps / t, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
               "sample": f"{sample_experts} of {E} experts x {tpe} tokens of workload {w.name}, {reps} passes"}

    line = {
        "metric": METRIC, "value": T / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 (split-operand tensor-core products: TF32 head + BF16 corrections, FP32 accumulate)", "data": "synthetic",
        "config": dict(workload_config(w, 1), **({"expert_cache_slots": args.cache_slots} if args.cache_slots else {})),
        "e2e": {"value": T / e2e_s, "unit": UNIT, "h2d_bytes_per_step": int(hx.numel() * 4),
                "d2h_bytes_per_step": int(hout.numel() * 4), "ms_per_step": 1e3 * e2e_s,
                "two_in_flight": two_in_flight, "two_contexts": two_ctx},
        "gpu_launches": int(launches), "stage_ms": stage_ms, "active_experts": active,
        "ffn_useful_tflops": 6.0 * T * D * F / ((stage_ms["ffn_gemm1"] + stage_ms["ffn_gemm2"]) * 1e-3) / 1e12
        if (stage_ms["ffn_gemm1"] + stage_ms["ffn_gemm2"]) > 0 else None,
        "roofline": roofline, "cpu_baseline": cpu, "clocks": clock_summary,
        "routing_vs_other_orders": routing_differences(w, x, cent, ln, gate, torch) if not args.no_cpu else None,
    }
    layer.terminate()
    if not args.no_cpu:
        line["ref_gpu_baseline"] = ref_gpu_baseline(w, torch)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-two-contexts", action="store_true",
                    help="skip the end-to-end leg that drives two clones from two host threads")
    ap.add_argument("--no-ep-cpm2", action="store_true",
                    help="N > 1: skip the fixed-size expert-parallel case that is otherwise run after the weak one")
    ap.add_argument("--seq-len", type=int, default=None, help="override the workload's sequence length (tuning)")
    ap.add_argument("--cache-slots", type=int, default=0,
                    help="streamed workloads: experts the layer keeps on the device across calls (0 = none, as the "
                         "reference)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    w, scaling = resolve_workload(args)
    if args.seq_len:
        w = synth.scaled(w, seq_len=args.seq_len)
    if args.impl == "reference":
        run_reference_arm(args, w, scaling)
        return
    if args.gpus == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        run_single(args, w)
    else:
        from infmoe_b200 import ep_bench
        ep_bench.run(args, w, scaling, METRIC, UNIT, ClockSampler, _peaks, workload_config, gemm_roofline)


def resolve_workload(args):
    """-> (whole-job workload, "weak" | "strong").

    One GPU: the named workload (default cpm2).  N GPUs: by default N copies of that per-GPU share (32 N experts,
    4096 N tokens: weak scaling, and N = 1 is the single-GPU workload itself); `--workload ep_cpm2` is the
    fixed-size expert-parallel case (E = 128, 65536 tokens in total) sharded over the ranks."""
    n = max(args.gpus, int(os.environ.get("WORLD_SIZE", "1")))
    if n == 1:
        return synth.WORKLOADS[args.workload or "cpm2"], "weak"
    if args.workload == "ep_cpm2":
        return synth.WORKLOADS["ep_cpm2"], "strong"
    base = synth.WORKLOADS[args.workload or "cpm2"]
    return synth.scaled(base, expert_count=base.expert_count * n, batch=base.batch * n), "weak"


if __name__ == "__main__":
    main()
