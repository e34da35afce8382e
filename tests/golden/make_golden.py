"""Generates the committed fixtures of tests/golden.

    python tests/golden/make_golden.py [--reference /path/to/InfMoE]

1. kat.npz: known-answer cases whose arithmetic is exact in FP32 (small integers
   and powers of two), so every summation order gives the same bits.  The
   expected values are computed here with plain numpy in float64 and are
   independent of the C oracle and of the CUDA kernels.
2. ref_generated_weights.npz: an expert weight file written by the REFERENCE's own
   helper MoELayerConfig.generate_random_weight_file (python/infmoe/config.py:31-54),
   imported from the reference checkout; it carries the transposed `wo_weight`
   view (fortran_order=True) that the reference reader takes as C order.
   ref_generated_sums.npy holds the per-tensor sums numpy sees for the raw bytes.
"""
import argparse
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def gelu_dot64(a, b):
    return a * (0.5 * (1.0 + np.tanh(a * (0.035677408136300125 * a * a + 0.7978845608028654)))) * b


def kat_cases():
    out = {}
    # --- routing: integer inputs, scores are exact small integers ------------------------------
    rng = np.random.default_rng(7)
    T, D, E = 24, 20, 6   # D not a multiple of 4*32: exercises the tail of the lane-strided order
    x = rng.integers(-3, 4, size=(T, D)).astype(np.float32)
    c = rng.integers(-2, 3, size=(E, D)).astype(np.float32)
    c[3] = c[1]                       # experts 1 and 3 always tie: the lower index must win
    x[5] = 0                          # all scores equal (0): gate 0
    aff = x.astype(np.float64) @ c.astype(np.float64).T
    out["route_x"], out["route_c"] = x, c
    out["route_gate"] = aff.argmax(1).astype(np.int32)     # numpy argmax = first maximum
    out["route_score"] = aff.max(1).astype(np.float32)
    # --- dispatch: hand-written gate vector with empty experts at both ends ---------------------
    gate = np.array([3, 1, 3, 3, 1, 4, 1, 3, 4, 1, 1, 3], np.int32)   # experts 0, 2, 5 empty, E = 6
    out["disp_gate"] = gate
    out["disp_count"] = np.array([0, 5, 0, 5, 2, 0], np.int32)
    out["disp_offset"] = np.array([0, 0, 5, 5, 10, 12, 12], np.int32)
    out["disp_pos"] = np.array([1, 4, 6, 9, 10, 0, 2, 3, 7, 11, 5, 8], np.int32)
    # --- LayerNorm: rows of +-a have mean 0 and variance a^2 exactly -----------------------------
    D2 = 64
    signs = np.where(np.arange(D2) % 2 == 0, 1.0, -1.0)
    rows = np.stack([signs * 1.0, signs * 2.0, -signs * 0.5]).astype(np.float32)
    gamma = (np.arange(D2) % 4 + 1).astype(np.float32)
    var = np.array([1.0, 4.0, 0.25], np.float32)
    rstd = (np.float32(1.0) / np.sqrt(var + np.float32(1e-6))).astype(np.float32)   # correctly rounded steps
    out["ln_x"], out["ln_gamma"] = rows, gamma
    out["ln_out"] = (gamma[None, :] * (rows * rstd[:, None]).astype(np.float32)).astype(np.float32)
    # --- expert FFN with analytically known output -------------------------------------------------
    # wi_0 = wi_1 = first F rows of the identity (F <= D), wo = its transpose, ln weight 1:
    # y[d] = x[d] + gelu(h[d]) * h[d] for d < F, x[d] beyond;  h = LN(x)
    D3, F3 = 32, 16
    xe = rng.standard_normal((5, D3)).astype(np.float32)
    eye = np.eye(F3, D3, dtype=np.float32)
    m = xe.astype(np.float64).mean(1, keepdims=True)
    v = ((xe - m) ** 2).mean(1, keepdims=True)
    h = (xe - m) / np.sqrt(v + 1e-6)
    y = xe.astype(np.float64).copy()
    y[:, :F3] += gelu_dot64(h[:, :F3], h[:, :F3])
    out["ffn_x"], out["ffn_eye"], out["ffn_y64"] = xe, eye, y
    # --- base_layer mix with score 0 -> alpha = 0.5 exactly ----------------------------------------
    post = rng.integers(-8, 9, size=(4, 8)).astype(np.float32)
    routed = rng.integers(-8, 9, size=(4, 8)).astype(np.float32)
    pos = np.array([2, 0, 3, 1], np.int32)
    mix = np.empty_like(post)
    mix[pos] = 0.5 * post + 0.5 * routed
    out["mix_post"], out["mix_routed"], out["mix_pos"], out["mix_out"] = post, routed, pos, mix
    return out


def reference_weight_file(ref_root):
    spec = importlib.util.spec_from_file_location("ref_config", os.path.join(ref_root, "python/infmoe/config.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ref_config"] = mod   # dataclasses looks the module up while decorating
    spec.loader.exec_module(mod)
    np.random.seed(20240607)
    cfg = mod.MoELayerConfig(seq_len=4, expert_count=2, embedding_size=8, hidden_size=16, max_concurrency=2,
                             moe_variant="default", sublayer_type="T5_FF", max_batch_size=1, expert_centroids=None,
                             layernorm_weight=None, weight_file_path="")
    path = os.path.join(HERE, "ref_generated_weights.npz")
    cfg.generate_random_weight_file(path, overwrite=True)
    z = np.load(path)
    sums = np.zeros((2, 4))
    for e in range(2):
        for k, key in enumerate(["layer_norm_weight", "wi_0_weight", "wi_1_weight", "wo_weight"]):
            sums[e, k] = z[f"{e}/{key}"].astype(np.float64).sum()
    np.save(os.path.join(HERE, "ref_generated_sums.npy"), sums)
    # what a reader that ignores fortran_order (the reference's cnpy) sees for expert 0's wo: the
    # raw bytes of the [F][D] matrix taken as [D][F]
    raw = np.ascontiguousarray(z["0/wi_0_weight"]).reshape(8, 16)
    np.save(os.path.join(HERE, "ref_generated_wo_as_read.npy"), raw)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("INFMOE_REFERENCE") or
                    os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))),
                                 "reference"), help="the InfMoE checkout (default: a directory `reference` beside this repository)")
    args = ap.parse_args()
    np.savez(os.path.join(HERE, "kat.npz"), **kat_cases())
    if os.path.isdir(args.reference):
        reference_weight_file(args.reference)
    print("written:", sorted(os.listdir(HERE)))
