"""The expert-parallel entry points of the C ABI (infmoe_ep_*).

On one GPU all ranks are built inside this process (loopback): the same kernels, buffers and row maps as between
processes, with one stream in the place of the barriers.  With two GPUs the ranks are separate processes that
exchange rows over CUDA IPC peer memory and synchronise through NCCL.  Either way the concatenated outputs must be
the bits of the single-GPU layer, routing must equal the oracle's, and the result must be within 1e-5 of FP64."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-5


def _workload(variant, E=8, D=256, F=512, T=666):
    from infmoe_b200 import synth
    return synth.scaled(synth.WORKLOADS["cpm2"], variant=variant, expert_count=E, embedding_size=D, hidden_size=F,
                        batch=1, seq_len=T)


def _local_layers(w, world, c, experts=None, device_experts=False):
    import torch
    from infmoe_b200 import MoELayer, synth
    per = w.expert_count // world
    layers = []
    for r in range(world):
        lo = r * per
        layer = MoELayer.create(per, w.embedding_size, w.hidden_size, 2, c[lo:lo + per], None, "T5_FF", "default", None)
        for e in range(lo, lo + per):
            layer.set_expert(e - lo, *(experts[e] if experts is not None else synth.gen_expert_numpy(w, e)))
        layer.set_residency(1)
        layers.append(layer)
    return layers


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("variant", ["cpm_2", "base_layer", "default"])
def test_loopback_ranks_match_single_gpu_and_oracle(oracle, variant, world):
    import torch
    assert torch.cuda.is_available(), "this test needs a GPU"
    from infmoe_b200 import MoELayer, synth
    from infmoe_b200.ep_native import NativeExpertParallel, loopback_forward
    from infmoe_b200.devmem import read_device
    w = _workload(variant)
    x, c, ln = synth.gen_inputs(w)
    experts = [synth.gen_expert_numpy(w, e) for e in range(w.expert_count)]
    # ranks bring different numbers of tokens (one of them a single token)
    bounds = {2: [0, 301, w.tokens], 4: [0, 1, 300, 301, w.tokens],
              8: [0, 1, 100, 101, 200, 301, 400, 401, w.tokens]}[world]     # at eight ranks: one expert per rank
    locals_ = _local_layers(w, world, c, experts)
    eps = NativeExpertParallel.create_loopback(locals_, c, ln, variant, max_tokens=400)
    xs = [torch.from_numpy(x[bounds[r]:bounds[r + 1]].copy()).cuda() for r in range(world)]
    outs = loopback_forward(eps, xs)
    for ep in eps:
        ep.sync_status()
    out = np.concatenate([o.cpu().numpy() for o in outs])
    gate = np.concatenate([read_device(ep.last_routing()[0], xs[r].shape[0], np.int32) for r, ep in enumerate(eps)])
    ref = oracle.layer_forward_f32(x, variant, c, ln, experts)
    np.testing.assert_array_equal(gate, ref["gate"])
    o64 = oracle.layer_forward_f64(x, variant, ref["gate"], ref["score"], experts)
    assert oracle.rel_l2(out, o64) <= TOL
    # what every rank received: rows of its own experts only, as many as the routing says
    per = w.expert_count // world
    for r, ep in enumerate(eps):
        cnt_p, exp_p, home_p, region = ep.received()
        cnt = read_device(cnt_p, world, np.int32)
        assert region == 400
        for s_ in range(world):
            g_src = ref["gate"][bounds[s_]:bounds[s_ + 1]]
            assert cnt[s_] == np.count_nonzero((g_src >= r * per) & (g_src < (r + 1) * per))
    # the same rows meet the same weights with the same K chunking: identical bits to the single-GPU layer
    single = MoELayer.create(w.expert_count, w.embedding_size, w.hidden_size, 2, c, None, "T5_FF", variant, ln)
    for e, ex in enumerate(experts):
        single.set_expert(e, *ex)
    want = single.forward_host(x)
    np.testing.assert_array_equal(out, want)
    # buffers are reusable: a second pass with the ranks' rows swapped around
    xs2 = [torch.from_numpy(x[bounds[r]:bounds[r + 1]][::-1].copy()).cuda() for r in range(world)]
    outs2 = loopback_forward(eps, xs2)
    for ep in eps:
        ep.sync_status()
    out2 = np.concatenate([o.cpu().numpy()[::-1] for o in outs2])
    np.testing.assert_array_equal(out2, want)
    for ep in eps:
        ep.destroy()
    for l in locals_ + [single]:
        l.terminate()


def test_loopback_reports_nan_rows_and_serves_the_others(oracle):
    import torch
    assert torch.cuda.is_available()
    from infmoe_b200 import capi, synth
    from infmoe_b200.ep_native import NativeExpertParallel, loopback_forward
    w = _workload("cpm_2", T=500)
    x, c, ln = synth.gen_inputs(w)
    experts = [synth.gen_expert_numpy(w, e) for e in range(w.expert_count)]
    locals_ = _local_layers(w, 2, c, experts)
    eps = NativeExpertParallel.create_loopback(locals_, c, ln, "cpm_2", max_tokens=250)
    bad = x.copy()
    bad_rows = np.array([3, 100, 249])
    bad[bad_rows, 0] = np.nan                       # all on rank 0
    xs = [torch.from_numpy(bad[:250].copy()).cuda(), torch.from_numpy(bad[250:].copy()).cuda()]
    for ep in eps:                                   # previous contents of the output buffers
        ep.output_view(250).fill_(-7.0)
    outs = loopback_forward(eps, xs)
    with pytest.raises(capi.InfMoEError) as e:
        eps[0].sync_status()
    assert e.value.status == 3
    eps[1].sync_status()                             # its own tokens are fine
    out = np.concatenate([o.cpu().numpy() for o in outs])
    assert np.all(out[bad_rows] == -7.0)
    good = np.setdiff1d(np.arange(w.tokens), bad_rows)
    ref = oracle.layer_forward_f32(x[good], "cpm_2", c, ln, experts)
    o64 = oracle.layer_forward_f64(x[good], "cpm_2", ref["gate"], ref["score"], experts)
    assert oracle.rel_l2(out[good], o64) <= TOL
    for ep in eps:
        ep.destroy()
    for l in locals_:
        l.terminate()


def _pipelined_steps(ep, hx, want, tokens, steps=5):
    """Steps submitted with two in flight: step k brings the rows rolled by k; every token must get the bits of the
    synchronous call, whatever runs beside it on the copy streams."""
    import torch
    from infmoe_b200 import capi
    ins = [torch.roll(hx, k, 0).contiguous().pin_memory() for k in range(steps)]
    outs = [torch.full_like(hx, float("nan")).pin_memory() for _ in range(steps)]
    for k in range(steps):
        ep.submit_host_ptr(ins[k].data_ptr(), outs[k].data_ptr(), tokens)
        if k >= 1:
            ep.wait_host()
    # one step is still in flight: a synchronous call is refused, a second submission is fine, a third is refused
    extra = torch.full_like(hx, float("nan")).pin_memory()
    with pytest.raises(capi.InfMoEError):
        ep.forward_host_ptr(ins[0].data_ptr(), extra.data_ptr(), tokens)
    ep.submit_host_ptr(ins[0].data_ptr(), extra.data_ptr(), tokens)
    with pytest.raises(capi.InfMoEError):
        ep.submit_host_ptr(ins[0].data_ptr(), extra.data_ptr(), tokens)
    ep.wait_host()
    ep.wait_host()
    with pytest.raises(capi.InfMoEError):        # nothing left to wait for
        ep.wait_host()
    assert torch.equal(extra, want)
    for k in range(steps):
        assert torch.equal(outs[k], torch.roll(want, k, 0)), k


def test_world_of_one_is_the_single_gpu_layer(oracle):
    import torch
    assert torch.cuda.is_available()
    from infmoe_b200 import MoELayer, synth
    from infmoe_b200.ep_native import NativeExpertParallel
    w = _workload("base_layer", T=300)
    x, c, ln = synth.gen_inputs(w)
    experts = [synth.gen_expert_numpy(w, e) for e in range(w.expert_count)]
    (local,) = _local_layers(w, 1, c, experts)
    ep = NativeExpertParallel.create(local, c, ln, "base_layer", 0, 1, None, max_tokens=300)
    hx = torch.from_numpy(x).pin_memory()
    hout = torch.empty_like(hx).pin_memory()
    ep.forward_host_ptr(hx.data_ptr(), hout.data_ptr(), w.tokens)
    single = MoELayer.create(w.expert_count, w.embedding_size, w.hidden_size, 2, c, None, "T5_FF", "base_layer", ln)
    for e, ex in enumerate(experts):
        single.set_expert(e, *ex)
    np.testing.assert_array_equal(hout.numpy(), single.forward_host(x))
    _pipelined_steps(ep, hx, hout.clone(), w.tokens)
    ep.forward_host_ptr(hx.data_ptr(), hout.data_ptr(), w.tokens)       # the synchronous call works again afterwards
    np.testing.assert_array_equal(hout.numpy(), single.forward_host(x))
    ep.destroy()
    local.terminate()
    single.terminate()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, variant, ret):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from infmoe_b200 import synth
        from infmoe_b200.ep_native import NativeExpertParallel, unique_id
        from infmoe_b200.devmem import read_device
        w = _workload(variant)
        x, c, ln = synth.gen_inputs(w)
        uid = [unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        local = _local_layers(w, world, c)[rank]
        per = w.tokens // world
        ep = NativeExpertParallel.create(local, c, ln, variant, rank, world, uid[0], max_tokens=per)
        dx = torch.from_numpy(x[rank * per:(rank + 1) * per].copy()).cuda()
        out = ep.forward(dx).clone()
        ep.sync_status()
        out2 = ep.forward(dx).clone()                      # buffers are reusable
        ep.sync_status()
        assert torch.equal(out, out2)
        hx = torch.from_numpy(x[rank * per:(rank + 1) * per].copy()).pin_memory()
        hout = torch.empty_like(hx).pin_memory()
        ep.forward_host_ptr(hx.data_ptr(), hout.data_ptr(), per)
        assert torch.equal(hout, out.cpu())
        _pipelined_steps(ep, hx, out.cpu(), per)
        ret[rank] = dict(out=out.cpu().numpy(), gate=read_device(ep.last_routing()[0], per, np.int32))
        dist.barrier()
        ep.destroy()
        local.terminate()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("variant", ["cpm_2", "base_layer"])
def test_two_processes_match_single_gpu_and_oracle(oracle, variant):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), variant, ret), nprocs=world, join=True)
        res = [ret[r] for r in range(world)]
    from infmoe_b200 import MoELayer, synth
    w = _workload(variant)
    x, c, ln = synth.gen_inputs(w)
    experts = [synth.gen_expert_numpy(w, e) for e in range(w.expert_count)]
    ref = oracle.layer_forward_f32(x, variant, c, ln, experts)
    out = np.concatenate([r["out"] for r in res])
    np.testing.assert_array_equal(np.concatenate([r["gate"] for r in res]), ref["gate"])
    o64 = oracle.layer_forward_f64(x, variant, ref["gate"], ref["score"], experts)
    assert oracle.rel_l2(out, o64) <= TOL
    single = MoELayer.create(w.expert_count, w.embedding_size, w.hidden_size, 2, c, None, "T5_FF", variant, ln)
    for e, ex in enumerate(experts):
        single.set_expert(e, *ex)
    np.testing.assert_array_equal(out, single.forward_host(x))
    single.terminate()
