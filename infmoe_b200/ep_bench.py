"""Multi-GPU leg of bench.py: the expert-parallel MoE layer, one rank per GPU under torch.distributed.run.

Default (weak scaling): every rank keeps the single-GPU benchmark's share -- 32 experts and 4096 local tokens of
the CPM-2-style layer -- so at N ranks the layer has 32 N experts and 4096 N tokens, and N = 1 is the single-GPU
workload itself.  `--workload ep_cpm2` runs the fixed-size case instead (E=128, 65536 tokens in total, sharded
over the ranks; strong scaling).
"""
from __future__ import annotations

import json
import os
import time

import numpy as np

from . import synth


def run(args, total, scaling, metric, unit, clock_sampler_cls, peaks_fn, workload_config):
    import torch
    import torch.distributed as dist

    from .ep import CudaStages, ExpertParallelMoE, expert_range
    from .plugin import MoELayer

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    E, D, F = total.expert_count, total.embedding_size, total.hidden_size
    T_local = total.tokens // world
    lo, hi = expert_range(E, world, rank)

    # small tensors: the same centroids on every rank, each rank's own rows
    _, cent, ln = synth.gen_inputs(synth.scaled(total, batch=1, seq_len=1))
    x_local, _, _ = synth.gen_inputs(synth.scaled(total, batch=1, seq_len=T_local, seed=total.seed + 1000 + rank))
    local = MoELayer.create(hi - lo, D, F, total.max_concurrency, cent[lo:hi], None, "T5_FF", "default", None)
    for e in range(lo, hi):
        local.set_expert(e - lo, *synth.gen_expert_torch(total, e, dev))
    local.set_residency(1)
    # Return path: peer stores from the GEMM epilogue (INFMOE_EP_PEER_OUTPUT=1) or a second all-to-all (=0).  The
    # default is the peer path on 2 GPUs, where it has been run and checked bit for bit; larger worlds keep the
    # all-to-all until the peer path has been run there too.
    peer_output = os.environ.get("INFMOE_EP_PEER_OUTPUT", "1" if world == 2 else "0") != "0" and world > 1
    moe = ExpertParallelMoE(CudaStages(local, cent, ln, total.variant), E, peer_output=peer_output)

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
    for _ in range(max(args.warmup, 3)):
        moe.forward(dx)
    moe.stages.check()
    local.set_profiling(True)
    moe.set_timing(True)
    launches0 = local.kernel_launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    start.record(stream)
    for _ in range(args.steps):
        moe.forward(dx)
    stop.record(stream)
    sync_all()
    ms = torch.tensor([start.elapsed_time(stop) / args.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    launches = torch.tensor([local.kernel_launches - launches0], device=dev, dtype=torch.int64)
    dist.all_reduce(launches, op=dist.ReduceOp.SUM)
    stage_ms, _ = local.stage_ms()
    phase_ms = moe.phase_ms()
    moe.set_timing(False)
    local.set_profiling(False)
    moe.stages.check()

    # end to end: host rows in, host rows out, every step
    def e2e_step():
        d = hx.to(dev, non_blocking=True)
        hout.copy_(moe.forward(d), non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(2):
        e2e_step()
    sync_all()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    sync_all()
    e2e_ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / args.steps], device=dev)
    dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    clocks.__exit__()

    received = int(moe.last["recv_counts"].sum())
    peaks = peaks_fn()
    g1 = stage_ms["ffn_gemm1"]
    roofline = None
    if g1 > 0:
        useful = 4.0 * received * D * F
        peak = peaks["bf16_sustained"] / 6.0
        achieved = useful / (g1 * 1e-3) / 1e12
        roofline = {"kernel": "ffn_umma_kernel<EPI_GELU_PAIR> (rank 0)", "bound": "tensor", "achieved": achieved,
                    "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None, "ms": g1,
                    "peak_source": f"bf16 sustained {peaks['bf16_sustained']} TFLOP/s of {peaks['source']} / 6"}
    if rank == 0:
        T_total = T_local * world
        cfg = workload_config(total, world)
        cfg.update({"parallelism": f"ep{world}", "tokens_per_gpu": T_local, "experts_per_gpu": hi - lo,
                    "exchange": ("NCCL all_to_all_single (counts, rows out); results stored by the owner's GEMM epilogue into the "
                                 "source rank's output buffer (CUDA IPC peer memory)") if peer_output
                    else "NCCL all_to_all_single (counts, rows out, rows back)"})
        line = {
            "metric": metric, "value": T_total / (float(ms.item()) * 1e-3), "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": float(ms.item()),
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "f32 (split-operand tensor-core products: TF32 head + BF16 corrections, FP32 accumulate)", "data": "synthetic", "config": cfg,
            "e2e": {"value": T_total / (float(e2e_ms.item()) * 1e-3), "unit": unit,
                    "h2d_bytes_per_step": int(hx.numel() * 4 * world), "d2h_bytes_per_step": int(hout.numel() * 4 * world),
                    "ms_per_step": float(e2e_ms.item())},
            "gpu_launches": int(launches.item()), "stage_ms_rank0": stage_ms, "phase_ms_rank0": phase_ms,
            "rows_received_rank0": received,
            "roofline": roofline, "cpu_baseline": None, "clocks": clocks.summary(),
        }
        print(json.dumps(line), flush=True)
    moe.close()
    local.terminate()
    dist.barrier()
    dist.destroy_process_group()
