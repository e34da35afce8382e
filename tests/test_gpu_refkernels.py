"""The reference's OWN kernels (plugin/cuda/moe.cu, ops/layernorm.cu, ops/gelu.cu, compiled unmodified into
oracle/_ref by `make -C oracle ref`) and its cuBLAS calls, run on the GPU: they pin the CPU oracle, and they are
compared with this library's kernels on the same inputs."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libinfmoe_ref_kernels.so")


@pytest.fixture(scope="module")
def ref():
    import torch
    assert torch.cuda.is_available(), "these tests need a GPU"
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref was not built (needs the reference checkout at build time)")
    torch.zeros(1, device="cuda")            # context first
    return ctypes.CDLL(REF_LIB)


@pytest.fixture(scope="module")
def g():
    from tests import gpu_util
    return gpu_util


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def test_reference_layernorm_pins_the_oracle(ref, g, oracle):
    import torch
    from infmoe_b200 import capi
    rng = np.random.default_rng(0)
    for n, D in [(7, 64), (33, 1000), (16, 4096)]:
        x = (rng.standard_normal((n, D)) * 2 + 0.3).astype(np.float32)
        gamma = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
        dx, dg = g.dev(x), g.dev(gamma)
        out = torch.empty_like(dx)
        assert ref.ref_layernorm(_p(out), _p(dx), n, D, _p(dg)) == 0
        got = out.cpu().numpy()
        # the restatement of the reference's Welford/Chan order agrees to the last bits (rsqrt is approximate on the GPU)
        np.testing.assert_allclose(got, oracle.layernorm_reference_order(x, gamma), rtol=3e-6, atol=1e-6)
        # and the canonical order used by this library is the same function to rounding
        assert oracle.rel_l2(got, oracle.layernorm(x, gamma)) < 1e-6
        ours = torch.empty_like(dx)
        capi.check(capi.lib().infmoe_layernorm(ours.data_ptr(), dx.data_ptr(), n, D, dg.data_ptr(), g.stream()))
        assert oracle.rel_l2(ours.cpu().numpy(), got) < 1e-6


def test_reference_select_count_scatter_gather(ref, g, oracle):
    import torch
    rng = np.random.default_rng(1)
    T, E, D = 3000, 37, 96
    aff = rng.integers(-5, 6, size=(T, E)).astype(np.float32)          # plenty of exact ties
    da = g.dev(aff)
    gate = torch.empty(T, dtype=torch.int32, device="cuda")
    wt = torch.empty(T, dtype=torch.float32, device="cuda")
    assert ref.ref_select(T, E, _p(da), _p(gate), _p(wt)) == 0
    og, os_ = oracle.select_top1(aff)
    np.testing.assert_array_equal(gate.cpu().numpy(), og)
    np.testing.assert_array_equal(wt.cpu().numpy(), os_)
    # moe_expert_count: the reference's host loops, through its own D2H/H2D copies
    pos = torch.empty(T, dtype=torch.int32, device="cuda")
    h_count = np.zeros(E, np.int32)
    h_offset = np.zeros(E + 1, np.int32)
    h_offset[E] = T
    assert ref.ref_count(T, E, _p(gate), _p(pos), h_count.ctypes.data_as(ctypes.c_void_p),
                         h_offset.ctypes.data_as(ctypes.c_void_p)) == 0
    oc, oo, op = oracle.dispatch(og, E)
    np.testing.assert_array_equal(h_count, oc)
    np.testing.assert_array_equal(h_offset, oo)
    np.testing.assert_array_equal(pos.cpu().numpy(), op)
    c2, o2, p2, _ = g.expert_count(og, E)                                  # this library's device kernel
    np.testing.assert_array_equal(p2, op)
    np.testing.assert_array_equal(c2, oc)
    np.testing.assert_array_equal(o2, oo)
    # scatter / gather / mix
    x = rng.standard_normal((T, D)).astype(np.float32)
    dx = g.dev(x)
    routed = torch.empty_like(dx)
    rs = torch.empty(T, dtype=torch.float32, device="cuda")
    assert ref.ref_scatter(T, D, _p(dx), _p(wt), _p(pos), _p(routed), _p(rs)) == 0
    o_routed, o_rs = oracle.scatter(x, os_, op)
    np.testing.assert_array_equal(routed.cpu().numpy(), o_routed)
    np.testing.assert_array_equal(rs.cpu().numpy(), o_rs)
    out = torch.empty_like(dx)
    assert ref.ref_gather(T, D, _p(routed), _p(pos), _p(out)) == 0
    np.testing.assert_array_equal(out.cpu().numpy(), x)
    post = g.dev(rng.standard_normal((T, D)).astype(np.float32))
    coeff = g.dev((rng.standard_normal(T) * 2).astype(np.float32))
    assert ref.ref_mix_gather(T, D, _p(pos), _p(routed), _p(post), _p(coeff), _p(out)) == 0
    want = oracle.mix_gather(post.cpu().numpy(), o_routed, coeff.cpu().numpy(), op)
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=2e-6, atol=1e-6)
    from infmoe_b200 import capi
    ours = torch.empty_like(dx)
    capi.check(capi.lib().infmoe_expert_mix_gather(T, D, pos.data_ptr(), routed.data_ptr(), post.data_ptr(),
                                                   coeff.data_ptr(), ours.data_ptr(), g.stream()))
    np.testing.assert_allclose(ours.cpu().numpy(), out.cpu().numpy(), rtol=2e-6, atol=1e-6)


def test_reference_gelu_dot(ref, g, oracle):
    import torch
    from infmoe_b200 import capi
    rng = np.random.default_rng(2)
    a = (rng.standard_normal(200001) * 3).astype(np.float32)
    b = rng.standard_normal(200001).astype(np.float32)
    da, db = g.dev(a), g.dev(b)
    assert ref.ref_gelu_dot(_p(da), _p(db), ctypes.c_size_t(a.size)) == 0
    got = db.cpu().numpy()
    np.testing.assert_allclose(got, oracle.gelu_dot(a, b), rtol=1e-5, atol=1e-6)
    da2, db2 = g.dev(a), g.dev(b)
    capi.check(capi.lib().infmoe_gelu_dot(da2.data_ptr(), db2.data_ptr(), a.size, g.stream()))
    np.testing.assert_allclose(db2.cpu().numpy(), got, rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("n,D,F", [(5, 64, 256), (139, 256, 512), (64, 1024, 2048)])
def test_reference_t5ff_sequence(ref, g, oracle, n, D, F):
    """layernorm_gpu + 3 x cublasSgemm_v2 + fused_gelu_dot_gpu with the arguments of T5FFLayer::run."""
    import torch
    rng = np.random.default_rng(n + D)
    x = rng.standard_normal((n, D)).astype(np.float32)
    ln = (1 + 0.01 * rng.standard_normal(D)).astype(np.float32)
    wi0 = (rng.standard_normal((F, D)) / np.sqrt(D)).astype(np.float32)
    wi1 = (rng.standard_normal((F, D)) / np.sqrt(D)).astype(np.float32)
    wo = (rng.standard_normal((D, F)) / np.sqrt(F)).astype(np.float32)
    dx, dl, d0, d1, do = g.dev(x), g.dev(ln), g.dev(wi0), g.dev(wi1), g.dev(wo)
    y = torch.empty_like(dx)
    ws = torch.empty(n * D + 2 * n * F, dtype=torch.float32, device="cuda")
    assert ref.ref_t5ff_run(n, D, F, _p(dl), _p(d0), _p(d1), _p(do), _p(dx), _p(y), _p(ws)) == 0
    y_ref = y.cpu().numpy()
    y64 = oracle.expert_ffn_f64(x, ln, wi0, wi1, wo)
    assert oracle.rel_l2(y_ref, y64) <= 1e-5              # the oracle describes what the reference computes
    assert oracle.rel_l2(oracle.expert_ffn_f32(x, ln, wi0, wi1, wo), y_ref) <= 5e-6
    ours = g.t5ff_run(x, ln, wi0, wi1, wo)
    assert oracle.rel_l2(ours, y_ref) <= 1e-5             # this library against the reference's own sequence
    assert oracle.rel_l2(ours, y64) <= 1e-5


@pytest.mark.parametrize("T,D,E,ln", [(2048, 1024, 32, False), (2048, 1024, 32, True), (1024, 4096, 32, True)])
def test_reference_gating_against_fused_routing(ref, g, oracle, T, D, E, ln):
    """[layernorm_gpu +] cuBLAS SGEMM scores + the reference's select vs the fused FP32 routing: same expert except
    at near-ties, where the summation order decides; the tokens that differ are the ones FP64 calls a near-tie."""
    import torch
    rng = np.random.default_rng(3 + D + int(ln))
    x = rng.standard_normal((T, D)).astype(np.float32)
    c = (rng.standard_normal((E, D)) * 0.02).astype(np.float32)
    gamma = (1 + 0.01 * rng.standard_normal(D)).astype(np.float32) if ln else None
    dx, dc = g.dev(x), g.dev(c)
    if ln:
        dn = torch.empty_like(dx)
        assert ref.ref_layernorm(_p(dn), _p(dx), T, D, _p(g.dev(gamma))) == 0
        dx = dn
    aff = torch.empty(T, E, dtype=torch.float32, device="cuda")
    assert ref.ref_gating_sgemm(T, D, E, _p(dc), _p(dx), _p(aff)) == 0
    gate = torch.empty(T, dtype=torch.int32, device="cuda")
    wt = torch.empty(T, dtype=torch.float32, device="cuda")
    assert ref.ref_select(T, E, _p(aff), _p(gate), _p(wt)) == 0
    ours, score, _ = g.route(x, c, gamma)
    g64, top1, top2 = oracle.route_f64(x, c, gamma)
    diff = np.nonzero(gate.cpu().numpy() != ours)[0]
    diff64 = np.nonzero(g64 != ours)[0]
    print(f"T={T} D={D} ln={ln}: {diff.size} tokens differ from the reference's order, {diff64.size} from FP64; "
          f"largest FP64 top-2 margin among them {np.max((top1 - top2)[diff], initial=0):.2e}")
    assert diff.size <= 2 and diff64.size <= 2               # FP32 summation order only matters at near-ties
    assert np.all((top1 - top2)[diff] < 1e-5)
    np.testing.assert_allclose(score, wt.cpu().numpy(), rtol=1e-4, atol=2e-6)


@pytest.mark.parametrize("variant", ["cpm_2", "default", "base_layer"])
def test_reference_layer_sequence(ref, g, oracle, variant):
    """The whole launch sequence of MoELayerPlugin::enqueue on the reference's kernels: with the final gather
    reading the expert output it equals the oracle and this library; literally (gather of the scattered input,
    plugin/MoELayerPlugin.cc:411) cpm_2/default return their input."""
    import torch
    from infmoe_b200 import MoELayer, synth
    w = synth.scaled(synth.WORKLOADS["tiny_default"], variant=variant, expert_count=6, embedding_size=128,
                     hidden_size=256, batch=2, seq_len=150)
    x, c, ln = synth.gen_inputs(w)
    experts = [synth.gen_expert_numpy(w, e) for e in range(w.expert_count)]
    T, D, E, F, mc = w.tokens, w.embedding_size, w.expert_count, w.hidden_size, 2
    dx, dc = g.dev(x), g.dev(c)
    dl = g.dev(ln) if ln is not None else None
    dev_w = [[g.dev(a) for a in ex] for ex in experts]
    tabs = [(ctypes.c_void_p * E)(*[ex[i].data_ptr() for ex in dev_w]) for i in range(4)]
    nbytes = mc * (4 * D + 12 * D * F + 4 * T * (D + 2 * F)) + 4 * (T * E + 2 * T + 2 * T * D) + 8 * T + 1024
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    out = torch.empty_like(dx)
    base = (1 if variant == "cpm_2" else 0) | (2 if variant == "base_layer" else 0)

    def call(flags):
        rc = ref.ref_layer_call(T, D, E, F, mc, flags, _p(dx), _p(dc), _p(dl) if dl is not None else None, tabs[0],
                                tabs[1], tabs[2], tabs[3], 1, _p(ws), _p(out))
        assert rc == 0
        return out.cpu().numpy()

    fixed = call(base | 4)
    r = oracle.layer_forward_f32(x, variant, c, ln, experts)
    o64 = oracle.layer_forward_f64(x, variant, r["gate"], r["score"], experts)
    assert oracle.rel_l2(fixed, o64) <= 1e-5
    layer = MoELayer.create(E, D, F, mc, c, None, "T5_FF", variant, ln)
    for e, ex in enumerate(experts):
        layer.set_expert(e, *ex)
    assert oracle.rel_l2(layer.forward_host(x), fixed) <= 1e-5
    layer.terminate()
    if variant != "base_layer":
        np.testing.assert_array_equal(call(base), x)
        np.testing.assert_array_equal(oracle.layer_forward_f32(x, variant, c, ln, experts, literal_gather=True)["out"], x)
