"""GPU parity of every stage entry point of the C ABI against the CPU oracle.

Integer results (gate, count, offset, pos) and the canonical-order FP32 results (score,
LayerNorm) must be bit-equal; the expert FFN must be within 1e-5 relative L2 of the
FP64-accumulated oracle (the tolerance the path's specification states)."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

FFN_TOL = 1e-5


@pytest.fixture(scope="module")
def g():
    import torch
    assert torch.cuda.is_available(), "these tests need a GPU"
    from tests import gpu_util
    return gpu_util


@pytest.fixture(scope="module")
def kat(golden_dir):
    return np.load(os.path.join(golden_dir, "kat.npz"))


def test_route_known_answers(g, kat):
    gate, score, status = g.route(kat["route_x"], kat["route_c"])
    np.testing.assert_array_equal(gate, kat["route_gate"])
    np.testing.assert_array_equal(score, kat["route_score"])
    assert status == 0


@pytest.mark.parametrize("T,D,E,ln", [(1, 64, 4, False), (32, 64, 4, False), (33, 64, 4, True), (7, 10, 1, True),
                                      (300, 1000, 37, True), (129, 130, 17, False), (64, 4096, 32, True),
                                      (40, 513, 130, True), (1000, 256, 64, False),
                                      # rows shorter than one 32-float box of the tiled copies, and just longer
                                      (9, 4, 3, False), (50, 12, 5, True), (100, 36, 33, True), (31, 260, 65, True)])
def test_route_bit_exact(g, oracle, T, D, E, ln):
    rng = np.random.default_rng(T * 131 + D)
    x = rng.standard_normal((T, D)).astype(np.float32)
    c = (rng.standard_normal((E, D)) * 0.02).astype(np.float32)
    gamma = (1 + 0.01 * rng.standard_normal(D)).astype(np.float32) if ln else None
    gate, score, status = g.route(x, c, gamma)
    ogate, oscore = oracle.route(x, c, gamma)
    np.testing.assert_array_equal(gate, ogate)
    np.testing.assert_array_equal(score.view(np.uint32), oscore.view(np.uint32))
    assert status == 0


def test_route_ties_and_nan(g, oracle):
    x = np.ones((5, 16), np.float32)
    c = np.ones((6, 16), np.float32)
    c[4] = 2.0
    c[5] = 2.0                                   # experts 4 and 5 tie at the maximum: 4 wins
    gate, score, status = g.route(x, c)
    np.testing.assert_array_equal(gate, 4)
    np.testing.assert_array_equal(score, 32.0)
    x[2, 3] = np.nan                             # NaN scores select nothing: status bit, gate -1
    gate, score, status = g.route(x, c)
    assert status & 1 and gate[2] == -1 and np.all(gate[[0, 1, 3, 4]] == 4)


def test_expert_select(g, oracle):
    import torch
    from infmoe_b200 import capi
    rng = np.random.default_rng(0)
    for T, E in [(1, 1), (50, 7), (300, 64), (10, 200)]:
        aff = rng.integers(-4, 5, size=(T, E)).astype(np.float32)    # many exact ties
        da = g.dev(aff)
        gate = torch.empty(T, dtype=torch.int32, device="cuda")
        wt = torch.empty(T, dtype=torch.float32, device="cuda")
        st = torch.zeros(1, dtype=torch.int32, device="cuda")
        capi.check(capi.lib().infmoe_expert_select(T, E, da.data_ptr(), gate.data_ptr(), wt.data_ptr(),
                                                   st.data_ptr(), g.stream()))
        og, os_ = oracle.select_top1(aff)
        np.testing.assert_array_equal(gate.cpu().numpy(), og)
        np.testing.assert_array_equal(wt.cpu().numpy(), os_)


def test_dispatch_known_answer(g, kat):
    count, offset, pos, status = g.expert_count(kat["disp_gate"], 6)
    np.testing.assert_array_equal(count, kat["disp_count"])
    np.testing.assert_array_equal(offset, kat["disp_offset"])
    np.testing.assert_array_equal(pos, kat["disp_pos"])
    assert status == 0


@pytest.mark.parametrize("T,E,skew", [(0, 3, 0), (1, 1, 0), (31, 4, 0), (1024, 32, 0), (1025, 32, 0), (4096, 32, 0),
                                      (5000, 130, 0), (16384, 64, 1.1), (65536, 128, 0), (70001, 1000, 1.5),
                                      (3000, 5, 0)])
def test_dispatch_bit_exact(g, oracle, T, E, skew):
    rng = np.random.default_rng(T + E)
    if skew:
        p = np.arange(1, E + 1, dtype=np.float64) ** -skew
        gate = rng.choice(E, size=T, p=p / p.sum()).astype(np.int32)
    else:
        gate = rng.integers(0, E, size=T).astype(np.int32)
    count, offset, pos, status = g.expert_count(gate, E)
    oc, oo, op = oracle.dispatch(gate, E)
    np.testing.assert_array_equal(count, oc)
    np.testing.assert_array_equal(offset, oo)
    np.testing.assert_array_equal(pos, op)
    assert status == 0


def test_dispatch_all_to_one_and_bad_gate(g, oracle):
    gate = np.full(2500, 3, np.int32)
    count, offset, pos, _ = g.expert_count(gate, 6)
    np.testing.assert_array_equal(pos, np.arange(2500))
    np.testing.assert_array_equal(count, [0, 0, 0, 2500, 0, 0])
    gate[7] = -1
    _, _, _, status = g.expert_count(gate, 6)
    assert status & 2


@pytest.mark.parametrize("T,E,bad_every", [(10, 3, 2), (2500, 6, 7), (9000, 40, 3), (70001, 130, 1000)])
def test_dispatch_defines_everything_when_gates_are_invalid(g, T, E, bad_every):
    """Tokens without an expert (gate -1 from a NaN row, or any index outside [0, E)) must not leave a hole in
    what dispatch hands on: pos[] stays a permutation, the valid tokens keep the reference's stable order, the
    others follow in ascending order, offset[E] counts the valid ones, and the status word says so."""
    import torch
    from infmoe_b200 import capi
    rng = np.random.default_rng(T)
    gate = rng.integers(0, E, size=T).astype(np.int32)
    bad = np.arange(0, T, bad_every)
    gate[bad] = np.where(np.arange(bad.size) % 2 == 0, -1, E + 5)
    dg = g.dev(gate)
    SENTINEL = -123456
    pos = torch.full((T,), SENTINEL, dtype=torch.int32, device="cuda")     # what a reused workspace looks like
    count = torch.full((E,), SENTINEL, dtype=torch.int32, device="cuda")
    offset = torch.full((E + 1,), SENTINEL, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    capi.check(capi.lib().infmoe_expert_count(T, E, dg.data_ptr(), pos.data_ptr(), count.data_ptr(),
                                              offset.data_ptr(), status.data_ptr(), g.stream()))
    torch.cuda.synchronize()
    pos, count, offset = pos.cpu().numpy(), count.cpu().numpy(), offset.cpu().numpy()
    valid = (gate >= 0) & (gate < E)
    assert int(status.item()) & 2
    assert not np.any(pos == SENTINEL)
    np.testing.assert_array_equal(np.sort(pos), np.arange(T))
    assert offset[E] == valid.sum()
    np.testing.assert_array_equal(count, np.bincount(gate[valid], minlength=E))
    np.testing.assert_array_equal(offset[:E], np.concatenate(([0], np.cumsum(count)[:-1])))
    order = np.argsort(np.where(valid, gate, E), kind="stable")       # stable: ascending token index per bucket
    np.testing.assert_array_equal(pos, order)


@pytest.mark.parametrize("T,D", [(1, 4), (50, 12), (33, 130), (512, 1024), (100, 4096)])
def test_scatter_gather_mix(g, oracle, T, D):
    import torch
    from infmoe_b200 import capi
    rng = np.random.default_rng(T + D)
    x = rng.standard_normal((T, D)).astype(np.float32)
    score = rng.standard_normal(T).astype(np.float32)
    _, _, pos = oracle.dispatch(rng.integers(0, 5, T).astype(np.int32), 5)
    dx, ds, dp = g.dev(x), g.dev(score), g.dev(pos)
    routed = torch.empty_like(dx)
    rs = torch.empty_like(ds)
    capi.check(capi.lib().infmoe_expert_scatter(T, D, dx.data_ptr(), ds.data_ptr(), dp.data_ptr(), routed.data_ptr(),
                                                rs.data_ptr(), g.stream()))
    o_routed, o_rs = oracle.scatter(x, score, pos)
    np.testing.assert_array_equal(routed.cpu().numpy(), o_routed)
    np.testing.assert_array_equal(rs.cpu().numpy(), o_rs)
    out = torch.zeros_like(dx)
    capi.check(capi.lib().infmoe_expert_gather(T, D, routed.data_ptr(), dp.data_ptr(), out.data_ptr(), g.stream()))
    np.testing.assert_array_equal(out.cpu().numpy(), x)          # scatter then gather is the identity
    post = rng.standard_normal((T, D)).astype(np.float32)
    dpost = g.dev(post)
    capi.check(capi.lib().infmoe_expert_mix_gather(T, D, dp.data_ptr(), routed.data_ptr(), dpost.data_ptr(),
                                                   rs.data_ptr(), out.data_ptr(), g.stream()))
    np.testing.assert_allclose(out.cpu().numpy(), oracle.mix_gather(post, o_routed, o_rs, pos), rtol=2e-6, atol=1e-6)


def test_mix_gather_known_answer(g, kat):
    import torch
    from infmoe_b200 import capi
    post, routed, pos = g.dev(kat["mix_post"]), g.dev(kat["mix_routed"]), g.dev(kat["mix_pos"])
    coeff = torch.zeros(4, device="cuda")
    out = torch.empty_like(post)
    capi.check(capi.lib().infmoe_expert_mix_gather(4, 8, pos.data_ptr(), routed.data_ptr(), post.data_ptr(),
                                                   coeff.data_ptr(), out.data_ptr(), g.stream()))
    np.testing.assert_array_equal(out.cpu().numpy(), kat["mix_out"])


@pytest.mark.parametrize("n,D", [(3, 64), (16, 1000), (9, 4096), (5, 7)])
def test_layernorm_bit_exact(g, oracle, kat, n, D):
    import torch
    from infmoe_b200 import capi
    rng = np.random.default_rng(n * D)
    x = (rng.standard_normal((n, D)) * 2 + 0.5).astype(np.float32)
    gamma = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    dx, dg = g.dev(x), g.dev(gamma)
    out = torch.empty_like(dx)
    capi.check(capi.lib().infmoe_layernorm(out.data_ptr(), dx.data_ptr(), n, D, dg.data_ptr(), g.stream()))
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), oracle.layernorm(x, gamma).view(np.uint32))
    if D == 64:
        dx, dg = g.dev(kat["ln_x"]), g.dev(kat["ln_gamma"])
        out = torch.empty_like(dx)
        capi.check(capi.lib().infmoe_layernorm(out.data_ptr(), dx.data_ptr(), 3, 64, dg.data_ptr(), g.stream()))
        np.testing.assert_array_equal(out.cpu().numpy(), kat["ln_out"])


def test_gelu_dot(g, oracle):
    import torch
    from infmoe_b200 import capi
    rng = np.random.default_rng(11)
    a = (rng.standard_normal(100003) * 3).astype(np.float32)
    b = rng.standard_normal(100003).astype(np.float32)
    da, db = g.dev(a), g.dev(b)
    capi.check(capi.lib().infmoe_gelu_dot(da.data_ptr(), db.data_ptr(), a.size, g.stream()))
    np.testing.assert_allclose(db.cpu().numpy(), oracle.gelu_dot(a, b), rtol=1e-5, atol=1e-6)


def _ffn_case(rng, n, D, F):
    x = rng.standard_normal((n, D)).astype(np.float32)
    ln = (1 + 0.01 * rng.standard_normal(D)).astype(np.float32)
    wi0 = (rng.standard_normal((F, D)) / np.sqrt(D)).astype(np.float32)
    wi1 = (rng.standard_normal((F, D)) / np.sqrt(D)).astype(np.float32)
    wo = (rng.standard_normal((D, F)) / np.sqrt(F)).astype(np.float32)
    return x, ln, wi0, wi1, wo


# token counts on both sides of the 16-row MMA granule and of the 192-token chunk; K tails; weight-row tails
@pytest.mark.parametrize("n,D,F", [(5, 64, 256), (1, 128, 128), (16, 64, 128), (17, 64, 128), (139, 256, 512),
                                   (192, 128, 256), (193, 128, 256), (400, 256, 384), (33, 72, 200),
                                   (64, 1024, 2048)])
def test_t5ff_tensor_core_path(g, oracle, n, D, F):
    x, ln, wi0, wi1, wo = _ffn_case(np.random.default_rng(n + D + F), n, D, F)
    y = g.t5ff_run(x, ln, wi0, wi1, wo)
    y64 = oracle.expert_ffn_f64(x, ln, wi0, wi1, wo)
    err = oracle.rel_l2(y, y64)
    assert err <= FFN_TOL, err
    # the expert contribution alone (output minus residual) must also be accurate, not hidden by x
    assert oracle.rel_l2(y - x, y64 - x) <= 5 * FFN_TOL


@pytest.mark.parametrize("n,D,F", [(5, 66, 130), (20, 30, 50), (3, 7, 9)])
def test_t5ff_unaligned_shapes_exact_path(g, oracle, n, D, F):
    x, ln, wi0, wi1, wo = _ffn_case(np.random.default_rng(n * D * F), n, D, F)
    y = g.t5ff_run(x, ln, wi0, wi1, wo)
    assert oracle.rel_l2(y, oracle.expert_ffn_f64(x, ln, wi0, wi1, wo)) <= FFN_TOL


def test_t5ff_known_answer(g, oracle, kat):
    x, eye = kat["ffn_x"], kat["ffn_eye"]
    y = g.t5ff_run(x, np.ones(x.shape[1], np.float32), eye, eye, np.ascontiguousarray(eye.T))
    assert oracle.rel_l2(y, kat["ffn_y64"]) <= FFN_TOL
