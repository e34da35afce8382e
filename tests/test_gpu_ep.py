"""Expert-parallel layer on 2 GPUs (NCCL) against the single-GPU layer and the CPU oracle."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _workload(variant):
    from infmoe_b200 import synth
    return synth.scaled(synth.WORKLOADS["cpm2"], variant=variant, expert_count=8, embedding_size=256, hidden_size=512,
                        batch=2, seq_len=333)


def _worker(rank, world, port, variant, peer_output, ret):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from infmoe_b200 import MoELayer, synth
        from infmoe_b200.ep import CudaStages, ExpertParallelMoE, expert_range
        w = _workload(variant)
        x, c, ln = synth.gen_inputs(w)
        lo, hi = expert_range(w.expert_count, world, rank)
        local = MoELayer.create(hi - lo, w.embedding_size, w.hidden_size, 2, c[lo:hi], None, "T5_FF", "default", None)
        for e in range(lo, hi):
            local.set_expert(e - lo, *synth.gen_expert_numpy(w, e))
        moe = ExpertParallelMoE(CudaStages(local, c, ln, variant), w.expert_count, peer_output=peer_output)
        per = w.tokens // world
        out = moe.forward(torch.from_numpy(x[rank * per:(rank + 1) * per].copy()).cuda())
        moe.stages.check()
        out2 = moe.forward(torch.from_numpy(x[rank * per:(rank + 1) * per].copy()).cuda())   # buffers are reusable
        torch.cuda.synchronize()
        assert torch.equal(out, out2)
        ret[rank] = dict(out=out.cpu().numpy(), gate=moe.last["gate"].cpu().numpy())
        moe.close()
        local.terminate()
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("peer_output", [False, True])
@pytest.mark.parametrize("variant", ["cpm_2", "base_layer"])
def test_two_gpus_match_single_gpu_and_oracle(oracle, variant, peer_output):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), variant, peer_output, ret), nprocs=world, join=True)
        res = [ret[r] for r in range(world)]
    from infmoe_b200 import MoELayer, synth
    w = _workload(variant)
    x, c, ln = synth.gen_inputs(w)
    experts = [synth.gen_expert_numpy(w, e) for e in range(w.expert_count)]
    ref = oracle.layer_forward_f32(x, variant, c, ln, experts)
    out = np.concatenate([r["out"] for r in res])
    np.testing.assert_array_equal(np.concatenate([r["gate"] for r in res]), ref["gate"])
    o64 = oracle.layer_forward_f64(x, variant, ref["gate"], ref["score"], experts)
    assert oracle.rel_l2(out, o64) <= 1e-5
    # the same rows meet the same weights with the same K chunking: identical bits to the single-GPU layer
    single = MoELayer.create(w.expert_count, w.embedding_size, w.hidden_size, 2, c, None, "T5_FF", variant, ln)
    for e, ex in enumerate(experts):
        single.set_expert(e, *ex)
    np.testing.assert_array_equal(out, single.forward_host(x))
    single.terminate()
