"""Expert-parallel exchange logic on two CPU ranks (gloo).  The compute steps are played by the CPU oracle
(a stand-in defined here, in the tests), so what is under test is the sharding, the count and row exchange,
the reassembly, and that the result equals the single-process layer on the concatenated batch."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


class OracleStages:
    """CPU stand-in for infmoe_b200.ep.CudaStages, backed by the oracle."""

    def __init__(self, oracle, variant, centroids, gating_ln, local_experts):
        self.o, self.variant, self.c, self.ln, self.weights = oracle, variant, centroids, gating_ln, local_experts

    def route(self, x):
        gate, score = self.o.route(x.numpy(), self.c, self.ln if self.variant == "cpm_2" else None)
        return torch.from_numpy(gate), torch.from_numpy(score)

    def dispatch(self, gate, E):
        count, _, pos = self.o.dispatch(gate.numpy(), E)
        return torch.from_numpy(count), torch.from_numpy(pos)

    def scatter(self, x, score, pos):
        routed, rscore = self.o.scatter(x.numpy(), score.numpy(), pos.numpy())
        return torch.from_numpy(routed), torch.from_numpy(rscore)

    def experts(self, rows, expert_of_row):
        rows, idx = rows.numpy(), expert_of_row.numpy()
        out = np.empty_like(rows)
        for e, w in enumerate(self.weights):
            sel = np.nonzero(idx == e)[0]
            if sel.size:
                out[sel] = self.o.expert_ffn_f32(rows[sel], *w)
        return torch.from_numpy(out)

    def combine(self, post, routed, rscore, pos):
        if self.variant == "base_layer":
            return torch.from_numpy(self.o.mix_gather(post.numpy(), routed.numpy(), rscore.numpy(), pos.numpy()))
        return torch.from_numpy(self.o.gather(post.numpy(), pos.numpy()))


def _worker(rank, world, port, variant, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from infmoe_b200 import synth
        from infmoe_b200.ep import ExpertParallelMoE, expert_range
        from oracle import oracle
        oracle.set_num_threads(1)
        w = synth.scaled(synth.WORKLOADS["tiny_default"], variant=variant, expert_count=6, embedding_size=32,
                         hidden_size=48, batch=2, seq_len=37)
        x, c, ln = synth.gen_inputs(w)
        per = w.tokens // world
        lo, hi = expert_range(w.expert_count, world, rank)
        local = [synth.gen_expert_numpy(w, e) for e in range(lo, hi)]
        moe = ExpertParallelMoE(OracleStages(oracle, variant, c, ln, local), w.expert_count)
        out = moe.forward(torch.from_numpy(x[rank * per:(rank + 1) * per].copy()))
        ret[rank] = dict(out=out.numpy(), gate=moe.last["gate"].numpy(), pos=moe.last["pos"].numpy(),
                         count=moe.last["count"].numpy(), recv=moe.last["recv_counts"].numpy())
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("variant", ["cpm_2", "base_layer"])
def test_two_ranks_equal_single_process(oracle, variant):
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), variant, ret), nprocs=world, join=True)
        res = [ret[r] for r in range(world)]
    from infmoe_b200 import synth
    w = synth.scaled(synth.WORKLOADS["tiny_default"], variant=variant, expert_count=6, embedding_size=32,
                     hidden_size=48, batch=2, seq_len=37)
    x, c, ln = synth.gen_inputs(w)
    experts = [synth.gen_expert_numpy(w, e) for e in range(w.expert_count)]
    ref = oracle.layer_forward_f32(x, variant, c, ln, experts)
    per = w.tokens // world
    # routing is per token, so the rank-major concatenation equals the single-process result bit for bit
    np.testing.assert_array_equal(np.concatenate([r["gate"] for r in res]), ref["gate"])
    np.testing.assert_array_equal(sum(r["count"] for r in res), ref["count"])
    # rows of one expert, taken rank by rank in each rank's local order, are the single-process stable order
    glob = [r["pos"] + i * per for i, r in enumerate(res)]
    for e in range(w.expert_count):
        seg = []
        for i, r in enumerate(res):
            off = int(r["count"][:e].sum())
            seg.append(glob[i][off:off + r["count"][e]])
        np.testing.assert_array_equal(np.concatenate(seg), ref["pos"][ref["offset"][e]:ref["offset"][e + 1]])
    # what a rank received is what the others counted for its experts
    for dst in range(world):
        for src in range(world):
            np.testing.assert_array_equal(res[dst]["recv"][src], res[src]["count"][dst * 3:(dst + 1) * 3])
    # every expert sees the same rows with the same weights: identical bits to the single-process layer
    np.testing.assert_array_equal(np.concatenate([r["out"] for r in res]), ref["out"])


def test_expert_range_checks():
    from infmoe_b200.ep import expert_range
    assert expert_range(128, 8, 3) == (48, 64)
    with pytest.raises(ValueError):
        expert_range(10, 4, 0)
