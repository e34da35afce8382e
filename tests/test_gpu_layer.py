"""GPU parity of the whole layer (MoELayerPlugin::enqueue) through the C ABI."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-5   # relative L2 against the FP64-accumulated oracle


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available(), "these tests need a GPU"
    return torch


def _build(w, synth, tmp_path=None, residency=-1, from_npz=True, mc=None):
    from infmoe_b200 import MoELayer
    x, c, ln = synth.gen_inputs(w)
    experts = [synth.gen_expert_numpy(w, e) for e in range(w.expert_count)]
    path = synth.write_npz(w, str(tmp_path / f"{w.name}.npz")) if from_npz else None
    layer = MoELayer.create(w.expert_count, w.embedding_size, w.hidden_size, mc or w.max_concurrency, c, path, "T5_FF",
                            w.variant, ln)
    if from_npz:
        layer.initialize()
    else:
        for e, ex in enumerate(experts):
            layer.set_expert(e, *ex)
    layer.set_residency(residency)
    return layer, x, c, ln, experts


def _routing(layer, T, E, torch):
    from tests.gpu_util import read_device as rd
    gate, score, pos, count, offset = layer.last_routing()
    return (rd(gate, T, np.int32), rd(score, T, np.float32), rd(pos, T, np.int32), rd(count, E, np.int32),
            rd(offset, E + 1, np.int32))


def _check(layer, w, x, c, ln, experts, oracle, torch, tol=TOL):
    out = layer.forward_host(x)
    ref = oracle.layer_forward_f32(x, w.variant, c, ln, experts)
    gate, score, pos, count, offset = _routing(layer, w.tokens, w.expert_count, torch)
    np.testing.assert_array_equal(gate, ref["gate"])
    np.testing.assert_array_equal(score.view(np.uint32), ref["score"].view(np.uint32))
    np.testing.assert_array_equal(count, ref["count"])
    np.testing.assert_array_equal(offset, ref["offset"])
    np.testing.assert_array_equal(pos, ref["pos"])
    o64 = oracle.layer_forward_f64(x, w.variant, ref["gate"], ref["score"], experts)
    err = oracle.rel_l2(out, o64)
    assert err <= tol, err
    assert oracle.rel_l2(out - x, o64 - x) <= 10 * tol      # the expert contribution itself
    return out


@pytest.mark.parametrize("variant", ["default", "cpm_2", "base_layer"])
def test_tiny_layer_from_npz(torch_cuda, oracle, tmp_path, variant):
    from infmoe_b200 import synth
    w = synth.scaled(synth.WORKLOADS["tiny_default"], variant=variant)
    layer, x, c, ln, experts = _build(w, synth, tmp_path)
    out = _check(layer, w, x, c, ln, experts, oracle, torch_cuda)
    assert layer.kernel_launches > 0
    # determinism: a second call gives the same bits
    np.testing.assert_array_equal(layer.forward_host(x), out)
    layer.terminate()


def test_compressed_weight_file_loads_to_the_same_layer(torch_cuda, oracle, tmp_path):
    """initialize() reads the members of the npz with several threads into one page-locked arena; a deflated file
    (np.savez_compressed) and a stored one must give the same layer."""
    from infmoe_b200 import MoELayer, synth
    w = synth.scaled(synth.WORKLOADS["cpm2"], expert_count=12, embedding_size=128, hidden_size=384, batch=1, seq_len=200)
    x, c, ln = synth.gen_inputs(w)
    experts = [synth.gen_expert_numpy(w, e) for e in range(w.expert_count)]
    outs = []
    for compressed in (False, True):
        path = synth.write_npz(w, str(tmp_path / f"w{int(compressed)}.npz"), compressed=compressed)
        layer = MoELayer.create(w.expert_count, w.embedding_size, w.hidden_size, 2, c, path, "T5_FF", w.variant, ln)
        layer.initialize()
        outs.append(_check(layer, w, x, c, ln, experts, oracle, torch_cuda))
        layer.terminate()
    np.testing.assert_array_equal(outs[0], outs[1])


@pytest.mark.parametrize("name,kw", [
    ("cpm2", dict(expert_count=8, embedding_size=512, hidden_size=1024, batch=2, seq_len=300)),
    ("base_layer_zipf", dict(expert_count=16, embedding_size=256, hidden_size=512, batch=4, seq_len=256)),
    ("cpm2", dict(expert_count=40, embedding_size=128, hidden_size=256, batch=1, seq_len=64)),   # empty experts
    ("tiny_default", dict(expert_count=3, embedding_size=64, hidden_size=128, batch=1, seq_len=1)),   # one token
])
def test_scaled_workloads(torch_cuda, oracle, name, kw):
    from infmoe_b200 import synth
    w = synth.scaled(synth.WORKLOADS[name], **kw)
    layer, x, c, ln, experts = _build(w, synth, from_npz=False)
    _check(layer, w, x, c, ln, experts, oracle, torch_cuda)
    layer.terminate()


def test_all_tokens_to_one_expert(torch_cuda, oracle):
    from infmoe_b200 import synth
    w = synth.scaled(synth.WORKLOADS["tiny_default"], expert_count=5, embedding_size=128, hidden_size=256, batch=1,
                     seq_len=450)
    layer, x, c, ln, experts = _build(w, synth, from_npz=False)
    layer.terminate()
    from infmoe_b200 import MoELayer
    c = np.zeros_like(c)
    c[3] = 1.0
    x = np.abs(x)
    layer = MoELayer.create(5, 128, 256, 2, c, None, "T5_FF", "default", None)
    for e, ex in enumerate(experts):
        layer.set_expert(e, *ex)
    _check(layer, w, x, c, None, experts, oracle, torch_cuda)
    layer.terminate()


@pytest.mark.parametrize("mc", [1, 2, 3])
def test_streamed_experts_match_resident(torch_cuda, oracle, tmp_path, mc):
    """max_concurrency slots fed from pinned host memory give the same bits as resident weights
    (mc = 1 is broken in the reference, plugin/MoELayerPlugin.cc:375-393; here it is just serial)."""
    from infmoe_b200 import synth
    w = synth.scaled(synth.WORKLOADS["cpm2"], expert_count=6, embedding_size=128, hidden_size=256, batch=1, seq_len=90)
    res, x, c, ln, experts = _build(w, synth, tmp_path, residency=1)
    st, *_ = _build(w, synth, tmp_path, residency=0, mc=mc)
    a = _check(res, w, x, c, ln, experts, oracle, torch_cuda)
    b = _check(st, w, x, c, ln, experts, oracle, torch_cuda)
    np.testing.assert_array_equal(a, b)
    np.testing.assert_array_equal(st.forward_host(x), b)     # slots are reusable across calls
    res.terminate()
    st.terminate()


@pytest.mark.parametrize("slots", [2, 3, 6])
def test_expert_cache_keeps_experts_across_calls(torch_cuda, oracle, tmp_path, slots):
    """Streamed mode with the layer's expert cache: same bits as resident weights whatever the cache size; with
    room for every expert the second call copies nothing; replaced weights are not served from the cache."""
    from infmoe_b200 import synth
    w = synth.scaled(synth.WORKLOADS["cpm2"], expert_count=6, embedding_size=128, hidden_size=256, batch=1, seq_len=90)
    res, x, c, ln, experts = _build(w, synth, tmp_path, residency=1)
    st, *_ = _build(w, synth, tmp_path, residency=0, mc=2)
    st.set_expert_cache(slots)
    want = _check(res, w, x, c, ln, experts, oracle, torch_cuda)
    per_expert = 3 * 4 * w.embedding_size * w.hidden_size
    got = st.forward_host(x)
    np.testing.assert_array_equal(got, want)
    first = st.weight_h2d_bytes()
    assert first == w.expert_count * per_expert            # every expert is routed to in this workload
    np.testing.assert_array_equal(st.forward_host(x), want)
    second = st.weight_h2d_bytes() - first
    if slots >= w.expert_count:
        assert second == 0
    else:
        assert 0 < second <= w.expert_count * per_expert
    # a permuted batch routes to the same experts: still nothing to copy when they all fit
    perm = np.random.default_rng(0).permutation(w.tokens)
    np.testing.assert_array_equal(st.forward_host(x[perm]), want[perm])
    if slots >= w.expert_count:
        assert st.weight_h2d_bytes() == first
    # new weights for expert 0 (those of expert 1): the cached copy must not be used
    st.set_expert(0, *experts[1])
    res.set_expert(0, *experts[1])
    before = st.weight_h2d_bytes()
    np.testing.assert_array_equal(st.forward_host(x), res.forward_host(x))
    assert st.weight_h2d_bytes() - before >= per_expert
    res.terminate()
    st.terminate()


@pytest.mark.parametrize("variant", ["cpm_2", "base_layer"])
def test_forward_host_into_page_locked_output(torch_cuda, oracle, variant):
    """A page-locked output buffer is written by the layer's last kernel directly; same bits as the copied path."""
    from infmoe_b200 import synth
    torch = torch_cuda
    w = synth.scaled(synth.WORKLOADS["cpm2"], variant=variant, expert_count=6, embedding_size=128, hidden_size=256,
                     batch=1, seq_len=200)
    layer, x, c, ln, experts = _build(w, synth, from_npz=False)
    want = _check(layer, w, x, c, ln, experts, oracle, torch)          # pageable numpy output
    hx = torch.from_numpy(x).pin_memory()
    hout = torch.full_like(hx, float("nan")).pin_memory()
    layer.forward_host_ptr(hx.data_ptr(), hout.data_ptr(), w.tokens)
    np.testing.assert_array_equal(hout.numpy(), want)
    layer.terminate()


@pytest.mark.parametrize("pinned,resident", [(True, True), (False, True), (True, False)])
def test_two_host_steps_in_flight_give_the_bits_of_the_blocking_call(torch_cuda, oracle, pinned, resident):
    """infmoe_layer_submit_host / _wait_host: step k brings the rows rolled by k, two steps in flight; page-locked
    buffers are written by the pass itself, pageable ones through a device buffer and a copy stream.  A NaN row is
    reported by the wait of its own step only."""
    from infmoe_b200 import capi, synth
    torch = torch_cuda
    w = synth.scaled(synth.WORKLOADS["cpm2"], variant="cpm_2", expert_count=6, embedding_size=128, hidden_size=256,
                     batch=1, seq_len=200)
    layer, x, c, ln, experts = _build(w, synth, from_npz=False)
    layer.set_residency(1 if resident else 0)          # streamed experts: every pass waits for its weight copies
    want = torch.from_numpy(_check(layer, w, x, c, ln, experts, oracle, torch))
    hx = torch.from_numpy(x)
    mem = (lambda t: t.pin_memory()) if pinned else (lambda t: t.clone())
    steps = 5
    ins = [mem(torch.roll(hx, k, 0).contiguous()) for k in range(steps)]
    if resident:    # (a streamed pass waits for its weight copies on the host and reports such a token from submit)
        ins[3][7, :] = float("nan")                               # step 3 has a token without an expert
    outs = [mem(torch.full_like(hx, float("nan"))) for _ in range(steps)]
    status = []
    for k in range(steps):
        layer.submit_host_ptr(ins[k].data_ptr(), outs[k].data_ptr(), w.tokens)
        if k >= 1:
            try:
                layer.wait_host()
                status.append(0)
            except capi.InfMoEError as e:
                status.append(e.status)
    with pytest.raises(capi.InfMoEError):                         # the blocking call is refused while a step is in flight
        layer.forward_host_ptr(ins[0].data_ptr(), outs[0].data_ptr(), w.tokens)
    layer.wait_host()
    status.append(0)
    with pytest.raises(capi.InfMoEError):                         # nothing left to wait for
        layer.wait_host()
    assert status == ([0, 0, 0, 3, 0] if resident else [0] * 5)
    for k in range(steps):
        got, exp = outs[k], torch.roll(want, k, 0)
        if k == 3 and resident:                                   # the NaN token's row is left alone
            keep = torch.ones(w.tokens, dtype=torch.bool)
            keep[7] = False
            got, exp = got[keep], exp[keep]
        assert torch.equal(got, exp), k
    layer.terminate()


def test_bounded_wait_runs_out_and_leaves_the_context_usable(torch_cuda, oracle, tmp_path):
    """The wait every role of the expert GEMM uses, pointed at a barrier nothing completes, with a 50 ms limit:
    it gives up, raises the status bit and returns; the next layer call on the same context works."""
    import ctypes

    from infmoe_b200 import capi, synth
    timed_out, waited = ctypes.c_int32(0), ctypes.c_float(0)
    capi.check(capi.lib().infmoe_wait_timeout_probe(50, ctypes.byref(timed_out), ctypes.byref(waited)))
    assert timed_out.value == 1
    assert 50.0 <= waited.value < 200.0
    w = synth.scaled(synth.WORKLOADS["tiny_default"], variant="cpm_2")
    layer, x, c, ln, experts = _build(w, synth, tmp_path)
    _check(layer, w, x, c, ln, experts, oracle, torch_cuda)
    layer.terminate()


@pytest.mark.parametrize("variant,path", [("cpm_2", ""), ("base_layer", ""), ("base_layer", "simt")])
def test_expert_forward_scatter_writes_rows_to_given_addresses(torch_cuda, oracle, monkeypatch, variant, path):
    """The expert-parallel building block: rows with known experts, each result written to its own address
    (here: a permutation of the rows of a local tensor), optionally with the base_layer mix."""
    from infmoe_b200 import synth
    torch = torch_cuda
    if path:
        monkeypatch.setenv("INFMOE_FFN", path)
    w = synth.scaled(synth.WORKLOADS["cpm2"], variant=variant, expert_count=6, embedding_size=128, hidden_size=256,
                     batch=1, seq_len=300)
    layer, x, c, ln, experts = _build(w, synth, from_npz=False)
    rng = np.random.default_rng(5)
    n, D = w.tokens, w.embedding_size
    expert_of_row = torch.from_numpy(rng.integers(0, w.expert_count, n).astype(np.int32)).cuda()
    rows = torch.from_numpy(x).cuda()
    want = layer.expert_forward(rows, expert_of_row)            # rows in, rows out, same order
    perm = torch.from_numpy(rng.permutation(n)).cuda()
    out = torch.full((n, D), float("nan"), device="cuda")
    dst = out.data_ptr() + perm.to(torch.int64) * (D * 4)
    score = None
    if variant == "base_layer":
        score = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda()
        alpha = torch.sigmoid(score.double())[:, None]
        want = (alpha * want.double() + (1 - alpha) * rows.double()).float()
    layer.expert_forward_scatter(rows, expert_of_row, dst.contiguous(), score)
    layer.sync_status()
    got = out[perm]
    if variant == "base_layer":
        torch.testing.assert_close(got, want, rtol=2e-6, atol=2e-6)
    else:
        assert torch.equal(got, want)
    layer.terminate()


def test_exact_path_matches_tensor_core_path(torch_cuda, oracle, monkeypatch):
    from infmoe_b200 import synth
    w = synth.scaled(synth.WORKLOADS["base_layer_zipf"], expert_count=8, embedding_size=128, hidden_size=256, batch=2,
                     seq_len=200)
    layer, x, c, ln, experts = _build(w, synth, from_npz=False)
    a = layer.forward_host(x)
    layer.terminate()
    monkeypatch.setenv("INFMOE_FFN", "simt")
    layer, *_ = _build(w, synth, from_npz=False)
    b = layer.forward_host(x)
    layer.terminate()
    assert oracle.rel_l2(a, b) < 2e-6


def test_identity_sublayer_returns_input(torch_cuda):
    from infmoe_b200 import MoELayer
    rng = np.random.default_rng(0)
    x = rng.standard_normal((70, 32)).astype(np.float32)
    c = rng.standard_normal((4, 32)).astype(np.float32)
    layer = MoELayer.create(4, 32, 64, 2, c, None, "Identity", "default", None)
    np.testing.assert_array_equal(layer.forward_host(x), x)
    layer.terminate()


@pytest.mark.parametrize("variant", ["default", "base_layer"])
def test_registered_sublayer_is_driven_like_the_built_in_ones(torch_cuda, oracle, variant):
    """A sublayer type registered through the C ABI (the reference's extension point is a class derived from
    MoESubLayer, plugin/sublayers/SubLayer.h:18-48): expert e scales its rows by a weight that the layer fetches
    into one of max_concurrency device slots before every run.  Routing, dispatch and combine are the layer's."""
    import ctypes
    from infmoe_b200 import MoELayer, capi
    torch = torch_cuda
    E, D, T, mc = 7, 96, 333, 2
    rng = np.random.default_rng(9)
    x = rng.standard_normal((T, D)).astype(np.float32)
    c = (rng.standard_normal((E, D)) * 0.1).astype(np.float32)
    scales = np.arange(E, dtype=np.float32) + 2.0
    # The fetch goes through the CUDA runtime directly: a torch copy from page-locked memory would make torch's host
    # allocator remember the layer's copy stream, which no longer exists when the test's tensors are freed.
    cudart = ctypes.CDLL("libcudart.so.12")
    cudart.cudaMemcpyAsync.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    calls = {"init": 0, "copy": [], "run": []}

    def tensor_at(ptr, n):
        class V:
            __cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (int(ptr), False), "version": 2}
        return torch.as_tensor(V(), device="cuda")

    def initialize(user, e, d, f, path):
        calls["init"] += 1
        return 0 if (e, d) == (E, D) else 1

    def copy_weights(user, dst, expert, stream):
        calls["copy"].append(int(expert))
        return cudart.cudaMemcpyAsync(dst, scales[expert:expert + 1].ctypes.data, 4, 1, stream)   # 1: host to device

    def run(user, expert, n, weights, src, dst, ws, stream):
        calls["run"].append((int(expert), int(n)))
        with torch.cuda.stream(torch.cuda.ExternalStream(int(stream or 0))):
            torch.mul(tensor_at(src, n * D), tensor_at(weights, 1), out=tensor_at(dst, n * D))
        return 0

    vt = capi.SublayerVtable(None, capi.SUB_INIT_FN(initialize), capi.SUB_WEIGHT_SIZE_FN(lambda user: 4),
                             capi.SUB_WS_SIZE_FN(lambda user, n: 0), capi.SUB_COPY_FN(copy_weights), capi.SUB_RUN_FN(run))
    capi.check(capi.lib().infmoe_register_sublayer(b"ScaleByExpert", ctypes.byref(vt)))
    layer = MoELayer.create(E, D, 4 * D, mc, c, None, "ScaleByExpert", variant, None)
    with pytest.raises(capi.InfMoEError):
        layer.forward_host(x)                       # not initialized yet
    layer.initialize()
    out = layer.forward_host(x)
    gate, score = oracle.route(x, c, None)
    want = x * (gate[:, None].astype(np.float32) + 2.0)
    if variant == "base_layer":
        alpha = (1.0 / (1.0 + np.exp(-score.astype(np.float64))))[:, None]
        want = alpha * want + (1 - alpha) * x
    np.testing.assert_allclose(out, want, rtol=2e-6, atol=1e-6)
    active = sorted(set(int(e) for e in gate))
    assert calls["init"] == 1 and calls["copy"] == active
    assert calls["run"] == [(e, int(np.count_nonzero(gate == e))) for e in active]
    layer.terminate()
    with pytest.raises(capi.InfMoEError):
        MoELayer.create(E, D, 4 * D, mc, c, None, "NoSuchSublayer", variant, None)


def test_nan_input_is_reported_not_trapped(torch_cuda):
    from infmoe_b200 import MoELayer, capi, synth
    w = synth.scaled(synth.WORKLOADS["tiny_default"])
    layer, x, c, ln, experts = _build(w, synth, from_npz=False)
    bad = x.copy()
    bad[3, :] = np.nan
    with pytest.raises(capi.InfMoEError) as e:
        layer.forward_host(bad)
    assert e.value.status == 3
    layer.forward_host(x)            # the context is still usable and the status was cleared
    layer.terminate()


@pytest.mark.parametrize("variant", ["cpm_2", "base_layer"])
def test_nan_tokens_touch_nothing_outside_their_own_rows(torch_cuda, oracle, variant):
    """A workspace is not zeroed between calls (TensorRT hands out the same block again and again).  With a few
    NaN rows in the input the call must report them, leave their output rows alone, and still give every other
    token its expert's result: no stage may index anything with what a previous call left in the workspace."""
    from infmoe_b200 import capi, synth
    torch = torch_cuda
    w = synth.scaled(synth.WORKLOADS["cpm2"], variant=variant, expert_count=6, embedding_size=128, hidden_size=256,
                     batch=1, seq_len=500)
    layer, x, c, ln, experts = _build(w, synth, from_npz=False)
    layer.set_residency(1)
    T, D = w.tokens, w.embedding_size
    need = layer.get_workspace_size(T)
    ws = torch.full((need,), 0x7f, dtype=torch.uint8, device="cuda")      # garbage indices everywhere
    bad_rows = np.array([0, 17, 255, 256, 499])
    bad = x.copy()
    bad[bad_rows, 5] = np.nan
    dx = torch.from_numpy(bad).cuda()
    out = torch.full((T, D), -7.0, device="cuda")
    layer.enqueue(dx.data_ptr(), out.data_ptr(), ws.data_ptr(), need, T, torch.cuda.current_stream().cuda_stream)
    with pytest.raises(capi.InfMoEError) as e:
        layer.sync_status(torch.cuda.current_stream().cuda_stream)
    assert e.value.status == 3
    got = out.cpu().numpy()
    assert np.all(got[bad_rows] == -7.0)                                  # untouched
    good = np.setdiff1d(np.arange(T), bad_rows)
    ref = oracle.layer_forward_f32(x[good], w.variant, c, ln, experts)
    o64 = oracle.layer_forward_f64(x[good], w.variant, ref["gate"], ref["score"], experts)
    assert oracle.rel_l2(got[good], o64) <= TOL
    gate, _, pos, count, offset = _routing(layer, T, w.expert_count, torch)
    assert np.all(gate[bad_rows] == -1) and offset[-1] == T - bad_rows.size
    np.testing.assert_array_equal(pos[offset[-1]:], bad_rows)
    layer.terminate()


@pytest.mark.parametrize("variant", ["cpm_2", "base_layer"])
def test_deserialised_layer_gives_the_same_bits(torch_cuda, oracle, tmp_path, variant):
    """serialize -> deserialize -> initialize -> enqueue (the deserialising constructor of the reference,
    plugin/MoELayerPlugin.cc:104-143, fed by serialize, :425-458) equals the layer the blob came from."""
    from infmoe_b200 import MoELayer, synth
    w = synth.scaled(synth.WORKLOADS["cpm2"], variant=variant, expert_count=6, embedding_size=128, hidden_size=256,
                     batch=2, seq_len=150)
    layer, x, c, ln, experts = _build(w, synth, tmp_path)
    want = _check(layer, w, x, c, ln, experts, oracle, torch_cuda)
    blob = layer.serialize()
    layer.terminate()
    twin = MoELayer.deserialize(blob)
    assert twin.moe_variant == variant and twin.expert_count == 6
    twin.initialize()                       # reads the weight file named in the blob
    got = _check(twin, w, x, c, ln, experts, oracle, torch_cuda)
    np.testing.assert_array_equal(got, want)
    clone = twin.clone()                    # TensorRT runs clones of the deserialised plugin
    np.testing.assert_array_equal(clone.forward_host(x), want)
    clone.terminate()
    twin.terminate()


def test_clones_on_two_streams_share_one_upload(torch_cuda, oracle, tmp_path):
    """Clones share the expert store; TensorRT gives each execution context its own clone and stream.  The first
    enqueue uploads the weights on its stream; a clone whose first enqueue overlaps it on another stream must
    wait for that upload instead of reading half-written planes."""
    from infmoe_b200 import synth
    torch = torch_cuda
    w = synth.scaled(synth.WORKLOADS["cpm2"], expert_count=8, embedding_size=512, hidden_size=2048, batch=1,
                     seq_len=400)
    layer, x, c, ln, experts = _build(w, synth, tmp_path, residency=1)
    clone = layer.clone()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    dx = torch.from_numpy(x).cuda()
    o1, o2 = torch.empty_like(dx), torch.empty_like(dx)
    torch.cuda.synchronize()
    layer.forward(dx, o1, stream=s1.cuda_stream)      # queues 8 x (3 copies + 2 retile kernels) and returns at once
    clone.forward(dx, o2, stream=s2.cuda_stream)      # sees the experts marked resident
    torch.cuda.synchronize()
    ref = oracle.layer_forward_f32(x, w.variant, c, ln, experts)
    o64 = oracle.layer_forward_f64(x, w.variant, ref["gate"], ref["score"], experts)
    assert oracle.rel_l2(o1.cpu().numpy(), o64) <= TOL
    assert torch.equal(o1, o2)
    clone.terminate()
    layer.terminate()


def test_enqueue_argument_checks(torch_cuda):
    from infmoe_b200 import MoELayer, capi, synth
    torch = torch_cuda
    w = synth.WORKLOADS["tiny_default"]
    layer, x, c, ln, experts = _build(w, synth, from_npz=False)
    dx = torch.from_numpy(x).cuda()
    ws = torch.empty(1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(capi.InfMoEError) as e:
        layer.enqueue(dx.data_ptr(), dx.data_ptr(), ws.data_ptr(), 1024, w.tokens)
    assert "alias" in str(e.value)
    out = torch.empty_like(dx)
    with pytest.raises(capi.InfMoEError) as e:
        layer.enqueue(dx.data_ptr(), out.data_ptr(), ws.data_ptr(), 1024, w.tokens)
    assert "workspace" in str(e.value)
    y = layer.forward(dx)
    layer.sync_status()
    np.testing.assert_array_equal(y.cpu().numpy(), layer.forward_host(x))
    layer.terminate()
    empty = MoELayer.create(2, 8, 16, 2, np.zeros((2, 8), np.float32), None, "T5_FF", "default", None)
    with pytest.raises(capi.InfMoEError) as e:
        empty.forward_host(np.zeros((2, 8), np.float32))
    assert e.value.status == 8
