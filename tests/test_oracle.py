"""The CPU oracle against the committed golden vectors and its own invariants (no GPU)."""
import os

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st


@pytest.fixture(scope="module")
def kat(golden_dir):
    return np.load(os.path.join(golden_dir, "kat.npz"))


def test_route_known_answers(oracle, kat):
    gate, score = oracle.route(kat["route_x"], kat["route_c"])
    np.testing.assert_array_equal(gate, kat["route_gate"])
    np.testing.assert_array_equal(score, kat["route_score"])
    assert gate[5] == 0                      # all scores equal: first expert
    assert not np.any(gate == 3)             # expert 3 duplicates expert 1: the lower index always wins


def test_select_top1_matches_route(oracle, kat):
    _, _, aff = oracle.route(kat["route_x"], kat["route_c"], want_aff=True)
    gate, score = oracle.select_top1(aff)
    np.testing.assert_array_equal(gate, kat["route_gate"])
    np.testing.assert_array_equal(score, kat["route_score"])


def test_route_nan_is_an_error(oracle):
    x = np.full((2, 8), np.nan, np.float32)
    c = np.ones((3, 8), np.float32)
    with pytest.raises(FloatingPointError):
        oracle.route(x, c)


def test_dispatch_known_answer(oracle, kat):
    count, offset, pos = oracle.dispatch(kat["disp_gate"], 6)
    np.testing.assert_array_equal(count, kat["disp_count"])
    np.testing.assert_array_equal(offset, kat["disp_offset"])
    np.testing.assert_array_equal(pos, kat["disp_pos"])


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 40), st.integers(0, 400), st.integers(0, 2**31 - 1))
def test_dispatch_properties(E, T, seed):
    from oracle import oracle
    gate = np.random.default_rng(seed).integers(0, E, size=T).astype(np.int32)
    count, offset, pos = oracle.dispatch(gate, E)
    assert count.sum() == T and offset[0] == 0 and offset[E] == T
    np.testing.assert_array_equal(np.diff(offset), count)                 # offsets = exclusive scan
    np.testing.assert_array_equal(np.sort(pos), np.arange(T))             # bijection
    np.testing.assert_array_equal(pos, np.argsort(gate, kind="stable"))  # stable counting sort


def test_layernorm_known_answer_and_reference_order(oracle, kat):
    out = oracle.layernorm(kat["ln_x"], kat["ln_gamma"])
    np.testing.assert_array_equal(out, kat["ln_out"])
    np.testing.assert_array_equal(oracle.layernorm_reference_order(kat["ln_x"], kat["ln_gamma"]), kat["ln_out"])
    # on random data the canonical order and the reference's Welford order agree to rounding
    rng = np.random.default_rng(1)
    for D in (64, 1000, 4096):
        x = rng.standard_normal((16, D)).astype(np.float32) * 3 + 1
        g = (1 + 0.01 * rng.standard_normal(D)).astype(np.float32)
        a, b = oracle.layernorm(x, g), oracle.layernorm_reference_order(x, g)
        assert oracle.rel_l2(a, b) < 1e-6
        m = x.astype(np.float64).mean(1, keepdims=True)
        v = x.astype(np.float64).var(1, keepdims=True)
        ref = g * (x - m) / np.sqrt(v + 1e-6)
        assert oracle.rel_l2(a, ref) < 1e-6


def test_scatter_gather_roundtrip(oracle):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((50, 12)).astype(np.float32)
    score = rng.standard_normal(50).astype(np.float32)
    gate = rng.integers(0, 7, 50).astype(np.int32)
    _, _, pos = oracle.dispatch(gate, 7)
    routed, rscore = oracle.scatter(x, score, pos)
    np.testing.assert_array_equal(routed, x[pos])
    np.testing.assert_array_equal(rscore, score[pos])
    np.testing.assert_array_equal(oracle.gather(routed, pos), x)


def test_mix_gather_known_answer(oracle, kat):
    out = oracle.mix_gather(kat["mix_post"], kat["mix_routed"], np.zeros(4, np.float32), kat["mix_pos"])
    np.testing.assert_array_equal(out, kat["mix_out"])      # score 0 -> alpha = 0.5 exactly


def test_expert_ffn_known_answer(oracle, kat):
    x, eye = kat["ffn_x"], kat["ffn_eye"]
    ln = np.ones(x.shape[1], np.float32)
    wo = np.ascontiguousarray(eye.T)
    y32 = oracle.expert_ffn_f32(x, ln, eye, eye, wo)
    y64 = oracle.expert_ffn_f64(x, ln, eye, eye, wo)
    assert oracle.rel_l2(y64, kat["ffn_y64"]) < 1e-7
    assert oracle.rel_l2(y32, kat["ffn_y64"]) < 1e-6


def test_sgemm_against_numpy(oracle):
    rng = np.random.default_rng(3)
    for M, N, K in [(1, 1, 1), (7, 33, 19), (130, 70, 300), (64, 256, 512)]:
        A = rng.standard_normal((M, K)).astype(np.float32)
        B = rng.standard_normal((N, K)).astype(np.float32)
        C0 = rng.standard_normal((M, N)).astype(np.float32)
        ref = A.astype(np.float64) @ B.astype(np.float64).T
        assert oracle.rel_l2(oracle.sgemm_nt(A, B), ref) < 1e-6
        assert oracle.rel_l2(oracle.sgemm_nt(A, B, C0), ref + C0) < 1e-6


@pytest.mark.parametrize("variant", ["default", "cpm_2", "base_layer"])
def test_layer_f32_against_f64_and_numpy(oracle, variant):
    from infmoe_b200 import synth
    w = synth.scaled(synth.WORKLOADS["tiny_default"], variant=variant, name="t")
    x, c, ln = synth.gen_inputs(w)
    experts = [synth.gen_expert_numpy(w, e) for e in range(w.expert_count)]
    r = oracle.layer_forward_f32(x, variant, c, ln, experts)
    o64 = oracle.layer_forward_f64(x, variant, r["gate"], r["score"], experts)
    assert oracle.rel_l2(r["out"], o64) < 1e-6
    # independent numpy restatement of the whole layer in float64
    xs = x.astype(np.float64)
    if variant == "cpm_2":
        m, v = xs.mean(1, keepdims=True), xs.var(1, keepdims=True)
        xs = ln * (xs - m) / np.sqrt(v + 1e-6)
    aff = xs @ c.astype(np.float64).T
    np.testing.assert_array_equal(aff.argmax(1), r["gate"])
    ref = np.empty_like(o64)
    for t in range(w.tokens):
        lnw, wi0, wi1, wo = [a.astype(np.float64) for a in experts[r["gate"][t]]]
        row = x[t].astype(np.float64)
        h = lnw * (row - row.mean()) / np.sqrt(row.var() + 1e-6)
        a, b = wi0 @ h, wi1 @ h
        g = a * (0.5 * (1 + np.tanh(a * (0.035677408136300125 * a * a + 0.7978845608028654)))) * b
        y = row + wo @ g
        if variant == "base_layer":
            al = 1 / (1 + np.exp(-aff[t].max()))
            y = al * y + (1 - al) * row
        ref[t] = y
    assert oracle.rel_l2(o64, ref) < 1e-6
    # the literal reference returns its input for cpm_2/default (gather reads the scattered input)
    if variant != "base_layer":
        lit = oracle.layer_forward_f32(x, variant, c, ln, experts, literal_gather=True)
        np.testing.assert_array_equal(lit["out"], x)


def test_layer_skips_empty_experts(oracle):
    rng = np.random.default_rng(5)
    D, F, E, T = 16, 32, 5, 9
    x = rng.standard_normal((T, D)).astype(np.float32)
    c = np.zeros((E, D), np.float32)
    c[2] = 1.0
    x[:, :] = np.abs(x)        # all scores positive for expert 2, zero elsewhere -> everything to expert 2
    experts = [None, None, (np.ones(D, np.float32), rng.standard_normal((F, D)).astype(np.float32),
                            rng.standard_normal((F, D)).astype(np.float32),
                            rng.standard_normal((D, F)).astype(np.float32)), None, None]
    r = oracle.layer_forward_f32(x, "default", c, None, experts)
    np.testing.assert_array_equal(r["count"], [0, 0, T, 0, 0])
    np.testing.assert_array_equal(r["pos"], np.arange(T))
