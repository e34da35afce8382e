"""The C++ plugin classes end to end on the GPU: create -> configure -> workspace -> initialize -> enqueue,
compared with the Python binding over the same C ABI and with the oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_plugin_enqueue_matches_binding_and_oracle(oracle, tmp_path):
    import torch
    assert torch.cuda.is_available()
    from infmoe_b200 import MoELayerConfig, MoELayerPlugin, synth
    from tests import plugin_util as pu
    w = synth.scaled(synth.WORKLOADS["cpm2"], expert_count=6, embedding_size=128, hidden_size=256, batch=3, seq_len=50)
    x, c, ln = synth.gen_inputs(w)
    path = synth.write_npz(w, str(tmp_path / "w.npz"))
    arr, n, keep = pu.make_fields(expert_count=6, embedding_size=128, hidden_size=256, max_concurrency=2,
                                  expert_centroids=c, expert_weight_file=path, expert_sublayer_type="T5_FF",
                                  moe_variant="cpm_2", layernorm_weight=ln)
    L = pu.lib()
    p = L.trtmoe_create_plugin(L.trtmoe_get_creator(b"MoELayerPlugin", b"1"), b"moe", arr, n)
    assert p
    L.trtmoe_plugin_configure(p, w.batch, w.seq_len, w.embedding_size)
    ws_bytes = L.trtmoe_plugin_workspace(p, w.batch, w.seq_len, w.embedding_size)
    assert L.trtmoe_plugin_initialize(p) == 0
    clone = L.trtmoe_plugin_clone(p)                      # TensorRT runs clones; weights are shared
    dx = torch.from_numpy(x).cuda()
    out = torch.empty_like(dx)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert L.trtmoe_plugin_enqueue(clone, w.batch, w.seq_len, w.embedding_size, dx.data_ptr(), out.data_ptr(),
                                   ws.data_ptr(), s) == 0
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    # the Python mirror of the reference binding, same weight file
    cfg = MoELayerConfig(seq_len=w.seq_len, expert_count=6, embedding_size=128, hidden_size=256, max_concurrency=2,
                         moe_variant="cpm_2", sublayer_type="T5_FF", max_batch_size=w.batch, expert_centroids=c,
                         layernorm_weight=ln, weight_file_path=path)
    layer = MoELayerPlugin(cfg).create_plugin()
    layer.initialize()
    np.testing.assert_array_equal(layer.forward_host(x), got)
    experts = [synth.gen_expert_numpy(w, e) for e in range(6)]
    r = oracle.layer_forward_f32(x, "cpm_2", c, ln, experts)
    assert oracle.rel_l2(got, oracle.layer_forward_f64(x, "cpm_2", r["gate"], r["score"], experts)) <= 1e-5
    layer.terminate()
    L.trtmoe_plugin_delete(clone)
    L.trtmoe_plugin_delete(p)


def _ep_plugin_worker(rank, world, id_file, npz, variant, ret):
    import os
    os.environ.update(INFMOE_EP_WORLD=str(world), INFMOE_EP_RANK=str(rank), INFMOE_EP_ID_FILE=id_file,
                      NCCL_NVLS_ENABLE="0")
    import torch
    torch.cuda.set_device(rank)
    from infmoe_b200 import synth
    from tests import plugin_util as pu
    w = synth.scaled(synth.WORKLOADS["cpm2"], variant=variant, expert_count=8, embedding_size=128, hidden_size=256,
                     batch=4, seq_len=50)
    x, c, ln = synth.gen_inputs(w)
    extra = {} if ln is None else {"layernorm_weight": ln}       # only cpm_2 has a pre-gating LayerNorm
    arr, n, keep = pu.make_fields(expert_count=8, embedding_size=128, hidden_size=256, max_concurrency=2,
                                  expert_centroids=c, expert_weight_file=npz, expert_sublayer_type="T5_FF",
                                  moe_variant=variant, **extra)
    L = pu.lib()
    p = L.trtmoe_create_plugin(L.trtmoe_get_creator(b"MoELayerPlugin", b"1"), b"moe", arr, n)
    assert p
    b = w.batch // world                                   # every rank runs its own batch items
    L.trtmoe_plugin_configure(p, b, w.seq_len, w.embedding_size)
    assert L.trtmoe_plugin_initialize(p) == 0              # collective: loads this rank's experts, joins the others
    clone = L.trtmoe_plugin_clone(p)
    rows = x.reshape(w.batch, w.seq_len, -1)[rank * b:(rank + 1) * b].reshape(-1, w.embedding_size)
    dx = torch.from_numpy(np.ascontiguousarray(rows)).cuda()
    out = torch.empty_like(dx)
    ws = torch.empty(max(L.trtmoe_plugin_workspace(p, b, w.seq_len, w.embedding_size), 16), dtype=torch.uint8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert L.trtmoe_plugin_enqueue(clone, b, w.seq_len, w.embedding_size, dx.data_ptr(), out.data_ptr(), ws.data_ptr(), s) == 0
    torch.cuda.synchronize()
    ret[rank] = out.cpu().numpy()
    L.trtmoe_plugin_delete(clone)
    L.trtmoe_plugin_delete(p)


@pytest.mark.parametrize("variant", ["cpm_2", "base_layer"])
def test_plugin_runs_expert_parallel_on_two_gpus(oracle, tmp_path, variant):
    """The C++ plugin classes with INFMOE_EP_WORLD=2: each process creates the plugin from the WHOLE layer's
    attributes, as TensorRT would on every rank, and enqueue() goes through infmoe_ep_forward."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from infmoe_b200 import MoELayer, synth
    w = synth.scaled(synth.WORKLOADS["cpm2"], variant=variant, expert_count=8, embedding_size=128, hidden_size=256,
                     batch=4, seq_len=50)
    x, c, ln = synth.gen_inputs(w)
    npz = synth.write_npz(w, str(tmp_path / "w.npz"))
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_ep_plugin_worker, args=(2, str(tmp_path / "ep.id"), npz, variant, ret), nprocs=2, join=True)
        out = np.concatenate([ret[0], ret[1]])
    single = MoELayer.create(8, 128, 256, 2, c, npz, "T5_FF", variant, ln)
    single.initialize()
    np.testing.assert_array_equal(out, single.forward_host(x))
    single.terminate()
