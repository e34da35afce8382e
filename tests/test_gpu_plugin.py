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
