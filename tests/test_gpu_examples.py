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
