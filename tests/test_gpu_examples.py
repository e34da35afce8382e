"""The stacked-layers example (the reference's python/examples/stacked_moe.py without TensorRT) against the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_stacked_moe_matches_oracle(oracle, tmp_path):
    from infmoe_b200.examples.stacked_moe import run_stacked_moe

    layers, E, D, F = 3, 4, 64, 128
    r = run_stacked_moe(layers, E, D, F, seq_len=8, batch=2, max_concurrency=2, moe_variant="cpm_2",
                        weight_file=str(tmp_path / "w.npz"), resident=-1, repeats=1, return_output=True)
    assert r["finite"] and r["shape"] == (2, 8, D)
    w = np.load(r["weight_file"])
    experts = [tuple(np.ascontiguousarray(w[f"{e}/{k}"]) for k in
                     ("layer_norm_weight", "wi_0_weight", "wi_1_weight", "wo_weight")) for e in range(E)]
    y = r["input"].reshape(-1, D)
    for _ in range(layers):
        y = oracle.layer_forward_f32(y, "cpm_2", r["centroids"], r["layernorm_weight"], experts)["out"]
    # tolerance per layer 1e-5 (relative L2); the layers amplify nothing: each adds its FFN term to the residual
    assert oracle.rel_l2(r["output"].reshape(-1, D), y) <= layers * 1e-5


def test_reference_helper_flow(oracle, tmp_path):
    """The demo flow of the reference (python/examples/stacked_moe.py): config -> MoELayerPlugin -> create_plugin ->
    create_layer_from_plugin -> engine -> allocate_buffers -> do_inference, here on the TensorRT-free stand-ins of
    infmoe_b200.utils, two stacked layers, compared with the oracle applied twice."""
    import torch
    assert torch.cuda.is_available()
    from infmoe_b200 import (MoELayerConfig, MoELayerPlugin, allocate_buffers, create_layer_from_plugin, do_inference,
                             synth)
    from infmoe_b200.utils import LayerNetwork
    w = synth.scaled(synth.WORKLOADS["cpm2"], expert_count=6, embedding_size=128, hidden_size=256, batch=3, seq_len=40)
    x, c, ln = synth.gen_inputs(w)
    path = synth.write_npz(w, str(tmp_path / "w.npz"))
    cfg = MoELayerConfig(seq_len=w.seq_len, expert_count=6, embedding_size=128, hidden_size=256, max_concurrency=2,
                         moe_variant="cpm_2", sublayer_type="T5_FF", max_batch_size=w.batch, expert_centroids=c,
                         layernorm_weight=ln, weight_file_path=path)
    network = LayerNetwork("input")
    prev = ["input"]
    for i in range(2):
        plugin = MoELayerPlugin(cfg).create_plugin(f"moe_{i}")
        layer = create_layer_from_plugin(network, plugin, prev, f"moe_{i}_output")
        prev = [layer.get_output(0)]
    engine = network.build_engine((w.seq_len, w.embedding_size), max_batch_size=w.batch)
    context = engine.create_execution_context()
    inputs, outputs, bindings, stream = allocate_buffers(engine)
    np.copyto(inputs[0].host, x.ravel())
    (out,) = do_inference(context, bindings, inputs, outputs, stream, batch_size=w.batch)
    got = out.reshape(x.shape)
    experts = [synth.gen_expert_numpy(w, e) for e in range(6)]
    y = x
    for _ in range(2):
        r = oracle.layer_forward_f32(y, "cpm_2", c, ln, experts)
        y = oracle.layer_forward_f64(y, "cpm_2", r["gate"], r["score"], experts).astype(np.float32)
    assert oracle.rel_l2(got, y) <= 2e-5      # two layers deep
