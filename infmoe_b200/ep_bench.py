"""Multi-GPU leg of bench.py: the expert-parallel MoE layer, one rank per GPU under torch.distributed.run.

Default (weak scaling): every rank keeps the single-GPU benchmark's share -- 32 experts and 4096 local tokens of
the CPM-2-style layer -- so at N ranks the layer has 32 N experts and 4096 N tokens, and N = 1 is the single-GPU
workload itself.  `--workload ep_cpm2` runs the fixed-size case instead (E=128, 65536 tokens in total, sharded
over the ranks; strong scaling); by default that case is also run after the weak one, with fewer steps, and
reported under the extra key "ep_cpm2".

The layer pass itself runs inside the library (infmoe_ep_forward: routing, peer stores of the rows over NVLink,
local experts, peer stores of the results; the only cross-GPU synchronisation is a two-word NCCL all-reduce).
torch.distributed is used here for the launch plumbing: handing out the communicator id, barriers around the timed
regions and the max over ranks.  After the timed regions rank 0 checks what it computed against the CPU oracle and
prints the outcome under "parity".
"""
from __future__ import annotations

import json
import os
import time

import numpy as np

from . import synth


def _parity(total, x_local, out_local, gate_local, score_local, dev, torch, rows_for_gate=1024, experts_checked=3,
            rows_per_expert=4):
    """Rank 0's own tokens against the oracle: routing bit for bit on the first rows, sampled output rows of sampled
    experts within 1e-5 relative L2 of the FP64 evaluation."""
    from oracle import oracle

    oracle.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    _, cent, ln = synth.gen_inputs(synth.scaled(total, batch=1, seq_len=1))
    gamma = ln if total.variant == "cpm_2" else None
    n = min(rows_for_gate, x_local.shape[0])
    ogate, oscore = oracle.route(x_local[:n], cent, gamma)
    gate_equal = bool(np.array_equal(ogate, gate_local[:n]) and
                      np.array_equal(oscore.view(np.uint32), score_local[:n].view(np.uint32)))
    rng = np.random.default_rng(0)
    hit = np.unique(gate_local[gate_local >= 0])
    chosen = rng.choice(hit, size=min(experts_checked, hit.size), replace=False)
    worst, rows_checked = 0.0, 0
    for e in chosen:
        rows = np.nonzero(gate_local == e)[0]
        rows = rng.choice(rows, size=min(rows_per_expert, rows.size), replace=False)
        ws = [t.cpu().numpy() for t in synth.gen_expert_torch(total, int(e), dev)]
        y64 = oracle.expert_ffn_f64(x_local[rows], *ws)
        if total.variant == "base_layer":
            alpha = 1.0 / (1.0 + np.exp(-score_local[rows].astype(np.float64)))[:, None]
            y64 = alpha * y64 + (1 - alpha) * x_local[rows]
        worst = max(worst, oracle.rel_l2(out_local[rows], y64))
        rows_checked += int(rows.size)
    return {"gate_equal": gate_equal, "gate_rows_checked": int(n), "rel_l2": float(worst), "rel_l2_tolerance": 1e-5,
            "rows_checked": rows_checked, "experts_checked": [int(e) for e in chosen],
            "return_path": "results stored by the owner's GEMM epilogue into the source rank's output buffer (peer memory)",
            "ok": bool(gate_equal and worst <= 1e-5 and np.isfinite(out_local).all())}


def _bind_to_gpu_numa_node(torch, local_rank):
    """Runs this rank on the CPUs of its GPU's NUMA node (when the node and its CPUs can be read and some of them
    are available to the process), so that the page-locked host buffers it allocates next are local to the GPU.
    -> a short description for the result line."""
    try:
        p = torch.cuda.get_device_properties(local_rank)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read())
        if node < 0:
            return "numa node unknown"
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        usable = cpus & os.sched_getaffinity(0)
        if not usable:
            return f"gpu on numa node {node}, none of its cpus available to this process"
        os.sched_setaffinity(0, usable)
        return f"bound to {len(usable)} cpus of numa node {node}"
    except (OSError, ValueError, AttributeError) as exc:
        return f"not bound ({type(exc).__name__})"


def _measure(total, scaling, steps, warmup, torch, dist, dev, rank, world, peaks, clock_sampler_cls, local_rank,
             gemm_roofline, with_e2e=True):
    """Builds this rank's share of workload `total`, times it, checks rank 0's result.  -> dict (rank 0) or None."""
    from .devmem import read_device
    from .ep_native import NativeExpertParallel, unique_id
    from .plugin import MoELayer

    E, D, F = total.expert_count, total.embedding_size, total.hidden_size
    T_local = total.tokens // world
    per = E // world
    lo, hi = rank * per, (rank + 1) * per
    _, cent, ln = synth.gen_inputs(synth.scaled(total, batch=1, seq_len=1))
    x_local, _, _ = synth.gen_inputs(synth.scaled(total, batch=1, seq_len=T_local, seed=total.seed + 1000 + rank))
    local = MoELayer.create(hi - lo, D, F, total.max_concurrency, cent[lo:hi], None, "T5_FF", "default", None)
    for e in range(lo, hi):
        local.set_expert(e - lo, *synth.gen_expert_torch(total, e, dev))
    local.set_residency(1)
    uid = torch.zeros(128, dtype=torch.uint8, device=dev)
    if rank == 0:
        uid.copy_(torch.frombuffer(bytearray(unique_id()), dtype=torch.uint8))
    dist.broadcast(uid, src=0)
    ep = NativeExpertParallel.create(local, cent, ln, total.variant, rank, world, bytes(uid.cpu().numpy().tobytes()),
                                     max_tokens=T_local)
    hx = torch.from_numpy(x_local).pin_memory()
    hout = torch.empty_like(hx).pin_memory()
    dx = hx.to(dev)
    stream = torch.cuda.current_stream()

    def sync_all():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    clocks = clock_sampler_cls(local_rank)
    clocks.__enter__()
    for _ in range(warmup):
        ep.forward(dx)
    ep.sync_status()
    local.set_profiling(True)
    ep.set_profiling(True)
    launches0 = local.kernel_launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    start.record(stream)
    for _ in range(steps):
        ep.forward(dx)
    stop.record(stream)
    sync_all()
    ms = torch.tensor([start.elapsed_time(stop) / steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    launches = torch.tensor([local.kernel_launches - launches0], device=dev, dtype=torch.int64)
    dist.all_reduce(launches, op=dist.ReduceOp.SUM)
    stage_ms, _ = local.stage_ms()
    phase_ms, _ = ep.phase_ms()
    ep.set_profiling(False)
    local.set_profiling(False)
    ep.sync_status()
    out_dev = ep.forward(dx).clone()
    ep.sync_status()

    e2e = None
    if with_e2e:
        # end to end: host rows in, host rows out, every step (the library's host-buffer entry point blocks)
        for _ in range(2):
            ep.forward_host_ptr(hx.data_ptr(), hout.data_ptr(), T_local)
        sync_all()
        t0 = time.perf_counter()
        for _ in range(steps):
            ep.forward_host_ptr(hx.data_ptr(), hout.data_ptr(), T_local)
        sync_all()
        e2e_ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / steps], device=dev)
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
        # the same steps with two in flight (infmoe_ep_submit_host): a step's upload runs behind the experts of the
        # step before, its download under the step after
        hx2, hout2 = hx.clone().pin_memory(), torch.empty_like(hx).pin_memory()
        bufs = [(hx, hout), (hx2, hout2)]
        for i in range(2):          # warm-up: the first submission creates the copy streams and staging buffers
            ep.submit_host_ptr(bufs[i][0].data_ptr(), bufs[i][1].data_ptr(), T_local)
        ep.wait_host()
        ep.wait_host()
        hout.zero_()
        sync_all()
        t0 = time.perf_counter()
        for i in range(steps):
            a, b = bufs[i & 1]
            ep.submit_host_ptr(a.data_ptr(), b.data_ptr(), T_local)
            if i >= 1:
                ep.wait_host()
        ep.wait_host()
        sync_all()
        pipe_ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / steps], device=dev)
        dist.all_reduce(pipe_ms, op=dist.ReduceOp.MAX)
        pipe_same = bool(torch.equal(hout, out_dev.cpu())) and (steps < 2 or bool(torch.equal(hout2, out_dev.cpu())))
        # host <-> device copy rates with every rank copying at once (they share the host's memory and PCIe roots)
        rates = []
        for src, dst in ((hx, dx), (out_dev, hout)):
            sync_all()
            t0 = time.perf_counter()
            for _ in range(5):
                dst.copy_(src, non_blocking=True)
            torch.cuda.synchronize()
            rates.append(5 * hx.numel() * 4 / (time.perf_counter() - t0) / 1e9)
        rates_t = torch.tensor(rates, device=dev)
        dist.all_reduce(rates_t, op=dist.ReduceOp.MIN)
        e2e = {"ms": float(e2e_ms.item()), "h2d_gbs_per_rank_min": float(rates_t[0].item()),
               "d2h_gbs_per_rank_min": float(rates_t[1].item()),
               "same_bits_as_device_path": bool(torch.equal(hout, out_dev.cpu())),
               "two_in_flight_ms": float(pipe_ms.item()), "two_in_flight_same_bits": pipe_same}
    clocks.__exit__()

    cnt_p, _, _, _ = ep.received()
    received = int(read_device(cnt_p, world, np.int32).sum())
    # every rank's share of the step: the rank that takes longest over its experts keeps the others waiting
    mine = torch.tensor([phase_ms.get("experts", 0.0), phase_ms.get("wait_results", 0.0), stage_ms["ffn_gemm1"],
                         stage_ms["ffn_gemm2"], float(received), float(clocks.summary().get("sm_mhz") or 0.0)],
                        device=dev, dtype=torch.float32)
    every = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    per_rank = {k: [round(float(t[i].item()), 3) for t in every]
                for i, k in enumerate(("experts_ms", "wait_results_ms", "gemm1_ms", "gemm2_ms", "rows_received", "sm_mhz"))}
    result = None
    if rank == 0:
        gate = read_device(ep.last_routing()[0], T_local, np.int32)
        score = read_device(ep.last_routing()[1], T_local, np.float32)
        parity = _parity(total, x_local, out_dev.cpu().numpy(), gate, score, dev, torch)
        g1 = stage_ms["ffn_gemm1"]
        clock_summary = clocks.summary()
        roofline = None
        if g1 > 0:
            roofline = gemm_roofline("ffn_umma_kernel<EPI_GELU_PAIR> (rank 0)", 4.0 * received * D * F / (g1 * 1e-3) / 1e12,
                                     g1, peaks, clock_summary, timed_s=float(ms.item()) * 1e-3 * steps)
            roofline["traffic"] = None
        result = {"ms": float(ms.item()), "tokens": T_local * world, "tokens_per_gpu": T_local, "experts_per_gpu": per,
                  "launches": int(launches.item()), "stage_ms_rank0": stage_ms, "phase_ms_rank0": phase_ms,
                  "rows_received_rank0": received, "per_rank": per_rank, "roofline": roofline, "clocks": clock_summary, "parity": parity,
                  "e2e": e2e, "hx_bytes": int(hx.numel() * 4)}
    dist.barrier()
    ep.destroy()
    local.terminate()
    del out_dev, dx
    torch.cuda.empty_cache()
    return result


def run(args, total, scaling, metric, unit, clock_sampler_cls, peaks_fn, workload_config, gemm_roofline):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    peaks = peaks_fn()
    numa = _bind_to_gpu_numa_node(torch, local_rank)
    warmup = max(args.warmup, 3)
    main = _measure(total, scaling, args.steps, warmup, torch, dist, dev, rank, world, peaks, clock_sampler_cls,
                    local_rank, gemm_roofline)
    extra = None
    if total.name != "ep_cpm2" and not args.no_ep_cpm2:
        # the fixed-size expert-parallel case (E = 128, 65536 tokens in total), a few steps
        c4 = synth.WORKLOADS["ep_cpm2"]
        if c4.expert_count % world == 0 and c4.tokens % world == 0:
            try:
                r = _measure(c4, "strong", max(3, min(args.steps, 5)), 3, torch, dist, dev, rank, world, peaks,
                             clock_sampler_cls, local_rank, gemm_roofline)
                if r is not None:
                    extra = {"workload": "ep_cpm2", "scaling": "strong", "expert_count": c4.expert_count,
                             "tokens": c4.tokens, "value": c4.tokens / (r["ms"] * 1e-3), "unit": unit,
                             "ms_per_step": r["ms"], "phase_ms_rank0": r["phase_ms_rank0"],
                             "stage_ms_rank0": r["stage_ms_rank0"], "parity": r["parity"],
                             "e2e": {"value": c4.tokens / (r["e2e"]["ms"] * 1e-3), "ms_per_step": r["e2e"]["ms"],
                                     "two_in_flight_ms_per_step": r["e2e"]["two_in_flight_ms"]}
                             if r["e2e"] else None}
            except Exception as exc:  # the headline line must not depend on the extra case
                extra = {"workload": "ep_cpm2", "error": f"{type(exc).__name__}: {exc}"}
    if rank == 0:
        T_total = main["tokens"]
        cfg = workload_config(total, world)
        cfg.update({"parallelism": f"ep{world}", "tokens_per_gpu": main["tokens_per_gpu"],
                    "experts_per_gpu": main["experts_per_gpu"],
                    "exchange": "rows stored into the owner's receive buffer and results into the source rank's "
                                "output buffer by the kernels themselves (CUDA IPC peer memory over NVLink); "
                                "two 2-word NCCL all-reduces per pass as barriers; no host synchronisation"})
        e2e = main["e2e"]
        line = {
            "metric": metric, "value": T_total / (main["ms"] * 1e-3), "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": main["ms"],
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "f32 (split-operand tensor-core products: TF32 head + BF16 corrections, FP32 accumulate)",
            "data": "synthetic", "config": cfg,
            "e2e": {"value": T_total / (e2e["ms"] * 1e-3), "unit": unit,
                    "h2d_bytes_per_step": main["hx_bytes"] * world, "d2h_bytes_per_step": main["hx_bytes"] * world,
                    "ms_per_step": e2e["ms"], "h2d_gbs_per_rank_min": e2e["h2d_gbs_per_rank_min"],
                    "d2h_gbs_per_rank_min": e2e["d2h_gbs_per_rank_min"],
                    "same_bits_as_device_path": e2e["same_bits_as_device_path"], "host_placement_rank0": numa,
                    "two_in_flight": {"value": T_total / (e2e["two_in_flight_ms"] * 1e-3), "unit": unit,
                                      "ms_per_step": e2e["two_in_flight_ms"],
                                      "same_output": e2e["two_in_flight_same_bits"]}},
            "gpu_launches": main["launches"], "stage_ms_rank0": main["stage_ms_rank0"],
            "phase_ms_rank0": main["phase_ms_rank0"], "rows_received_rank0": main["rows_received_rank0"],
            "per_rank": main["per_rank"], "parity": main["parity"], "roofline": main["roofline"], "cpu_baseline": None, "clocks": main["clocks"],
            "ep_cpm2": extra,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
