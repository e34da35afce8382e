"""Host-side logic of the C ABI that needs no GPU: the library loads, exports what the header
declares, validates attributes like the reference's creator, serialises, and reads npz files."""
import ctypes
import os
import re

import numpy as np
import pytest

from infmoe_b200 import MoELayer, MoELayerConfig, MoELayerPlugin, capi, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "infmoe_c.h")).read()
    declared = set(re.findall(r"INFMOE_API\s+[\w\s\*]+?\b(infmoe_\w+)\s*\(", header))
    assert len(declared) >= 25
    lib = ctypes.CDLL(capi.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in infmoe_c.h but not exported"
    assert declared == set(capi.SIGNATURES), "python binding and header disagree"


def _layer(**kw):
    args = dict(expert_count=3, embedding_size=8, hidden_size=16, max_concurrency=2,
                expert_centroids=np.arange(24, dtype=np.float32).reshape(3, 8), expert_weight_file=None,
                expert_sublayer_type="T5_FF", moe_variant="default", layernorm_weight=None)
    args.update(kw)
    return MoELayer.create(**args)


def test_create_validates_like_the_reference_creator(tmp_path):
    with pytest.raises(capi.InfMoEError) as e:
        _layer(moe_variant="nonsense")
    assert e.value.status == 1 and "unsupported moe variant" in str(e.value)
    with pytest.raises(capi.InfMoEError) as e:
        _layer(expert_sublayer_type="Conv")
    assert "unsupported sublayer type" in str(e.value)
    with pytest.raises(capi.InfMoEError) as e:
        _layer(moe_variant="cpm_2")                       # layernorm_weight missing
    assert "layernorm_weight" in str(e.value)
    with pytest.raises(capi.InfMoEError) as e:
        _layer(expert_weight_file=str(tmp_path / "missing.npz"))
    assert e.value.status == 4
    with pytest.raises(capi.InfMoEError):
        _layer(max_concurrency=0)
    with pytest.raises(ValueError):
        _layer(expert_centroids=np.zeros(5, np.float32))
    layer = _layer(moe_variant="cpm_2", layernorm_weight=np.ones(8, np.float32))
    assert layer.get_plugin_type() == "MoELayerPlugin" and layer.get_plugin_version() == "1"
    assert layer.get_nb_outputs() == 1 and layer.get_output_dimensions((2, 4, 8)) == (2, 4, 8)
    with pytest.raises(ValueError):
        layer.configure_plugin((2, 4, 9))
    layer.terminate()


def test_serialize_roundtrip_and_clone():
    ln = np.linspace(0.5, 1.5, 8, dtype=np.float32)
    layer = _layer(moe_variant="cpm_2", layernorm_weight=ln, max_concurrency=3)
    blob = layer.serialize()
    assert len(blob) % 4 == 0
    for other in (MoELayer.deserialize(blob), layer.clone()):
        assert (other.expert_count, other.embedding_size, other.hidden_size, other.max_concurrency) == (3, 8, 16, 3)
        assert other.moe_variant == "cpm_2" and other.expert_sublayer_type == "T5_FF"
        np.testing.assert_array_equal(other.expert_centroids, layer.expert_centroids)
        np.testing.assert_array_equal(other.layernorm_weight, ln)
    assert MoELayer.deserialize(blob).serialize() == blob
    with pytest.raises(capi.InfMoEError) as e:
        MoELayer.deserialize(blob[:-8])
    assert e.value.status == 5
    with pytest.raises(capi.InfMoEError):
        MoELayer.deserialize(b"\0" * 64)


def test_workspace_size_formula():
    layer = _layer()
    small, big = layer.get_workspace_size(1), layer.get_workspace_size(100)
    assert 0 < small < big
    # activations: routed, post, h_hi, h_lo [T][D] and g_hi, g_lo [T][F]; slots: mc x 3 matrices of D x F
    assert big >= 4 * 100 * (4 * 8 + 2 * 16) + 3 * 2 * 8 * 16 * 4


def test_python_binding_surface(tmp_path):
    cfg = MoELayerConfig(seq_len=4, expert_count=2, embedding_size=8, hidden_size=16, max_concurrency=2,
                         moe_variant="default", sublayer_type="T5_FF", max_batch_size=1, expert_centroids=None,
                         layernorm_weight=None, weight_file_path="")
    cfg.generate_random_centroids(seed=1)
    cfg.generate_random_layernorm_weight(seed=2)
    cfg.generate_random_weight_file(str(tmp_path / "w.npz"), overwrite=True, seed=3)
    assert cfg.expert_centroids.shape == (2, 8) and cfg.layernorm_weight.shape == (8,)
    z = np.load(cfg.weight_file_path)
    assert z["1/wo_weight"].shape == (8, 16) and z["1/wo_weight"].flags["C_CONTIGUOUS"]
    plugin = MoELayerPlugin(cfg)
    assert plugin.config is cfg
    layer = plugin.create_plugin("layer0")
    assert layer.name == "layer0" and layer.expert_weight_file == cfg.weight_file_path
    layer.terminate()


def _check_file(path, E, D, F):
    sums = np.zeros((E, 4))
    rc = capi.lib().infmoe_weight_file_check(path.encode(), E, D, F, sums.ctypes.data)
    capi.check(rc)
    return sums


@pytest.mark.parametrize("compressed", [False, True])
def test_npz_reader_matches_numpy(tmp_path, compressed):
    w = synth.scaled(synth.WORKLOADS["tiny_default"], expert_count=3, embedding_size=12, hidden_size=20)
    path = synth.write_npz(w, str(tmp_path / "w.npz"), compressed=compressed)
    sums = _check_file(path, 3, 12, 20)
    z = np.load(path)
    for e in range(3):
        for k, key in enumerate(["layer_norm_weight", "wi_0_weight", "wi_1_weight", "wo_weight"]):
            assert sums[e, k] == pytest.approx(z[f"{e}/{key}"].astype(np.float64).sum(), rel=1e-12)


def test_npz_reader_rejects_bad_files(tmp_path):
    w = synth.scaled(synth.WORKLOADS["tiny_default"], expert_count=2, embedding_size=8, hidden_size=16)
    path = synth.write_npz(w, str(tmp_path / "w.npz"))
    with pytest.raises(capi.InfMoEError) as e:      # wrong hidden size -> element count mismatch
        _check_file(path, 2, 8, 32)
    assert e.value.status == 5 and "elements" in str(e.value)
    with pytest.raises(capi.InfMoEError) as e:      # an expert is missing
        _check_file(path, 3, 8, 16)
    assert "missing tensors" in str(e.value)
    z = dict(np.load(path))
    z["0/wi_0_weight"] = z["0/wi_0_weight"].astype(np.float64)
    np.savez(str(tmp_path / "f64.npz"), **z)
    with pytest.raises(capi.InfMoEError) as e:
        _check_file(str(tmp_path / "f64.npz"), 2, 8, 16)
    assert "float32" in str(e.value)
    (tmp_path / "junk.npz").write_bytes(b"this is not a zip file at all, not even close.....")
    with pytest.raises(capi.InfMoEError):
        _check_file(str(tmp_path / "junk.npz"), 2, 8, 16)
    open(str(tmp_path / "trunc.npz"), "wb").write(open(path, "rb").read()[:3000])
    with pytest.raises(capi.InfMoEError):
        _check_file(str(tmp_path / "trunc.npz"), 2, 8, 16)
    with pytest.raises(capi.InfMoEError) as e:
        _check_file(str(tmp_path / "nope.npz"), 2, 8, 16)
    assert e.value.status == 4


def _npy_member(header: str, payload: bytes = b"") -> bytes:
    h = header.encode("latin1")
    return b"\x93NUMPY\x01\x00" + len(h).to_bytes(2, "little") + h + payload


@pytest.mark.parametrize("header", [
    "{'descr': '<f4', 'fortran_order':     ",                                  # nothing after the colon
    "{'descr': '<f4', 'fortran_order': False, 'shape': (8,  ",                  # shape never closed
    "{'descr': '<f4'",                                                          # keys missing
    "{'descr': '<f4', 'fortran_order': False, 'shape': (4611686018427387904, 16), }",   # element count overflows
    "",
])
def test_npz_reader_survives_garbled_npy_headers(tmp_path, header):
    """A malformed member header is a format error, not an exception through the C boundary."""
    import zipfile
    path = str(tmp_path / "bad.npz")
    with zipfile.ZipFile(path, "w", zipfile.ZIP_STORED) as z:
        z.writestr("0/layer_norm_weight.npy", _npy_member(header, b"\0" * 32))
    with pytest.raises(capi.InfMoEError) as e:
        _check_file(path, 1, 8, 16)
    assert e.value.status == 5


def test_reference_generated_weight_file(golden_dir, capfd):
    """A file written by the reference's own MoELayerConfig.generate_random_weight_file: its wo_weight is
    flagged fortran_order and must be taken as raw C-order bytes, as the reference's reader does."""
    path = os.path.join(golden_dir, "ref_generated_weights.npz")
    sums = _check_file(path, 2, 8, 16)
    np.testing.assert_allclose(sums, np.load(os.path.join(golden_dir, "ref_generated_sums.npy")), rtol=1e-12)
    assert "fortran_order" in capfd.readouterr().err


def test_enqueue_without_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    layer = _layer()
    with pytest.raises(capi.InfMoEError) as e:
        layer.forward_host(np.zeros((4, 8), np.float32))
    assert e.value.status in (2, 6, 8)
    layer.terminate()


def _simulate(slots, E, calls):
    import ctypes

    import numpy as np
    from infmoe_b200 import capi
    flat = np.asarray([e for c in calls for e in c], np.int32)
    sizes = np.asarray([len(c) for c in calls], np.int32)
    loads = np.zeros(len(calls), np.int32)
    capi.check(capi.lib().infmoe_expert_cache_simulate(slots, E, flat.ctypes.data, sizes.ctypes.data, len(calls),
                                                       loads.ctypes.data))
    return loads.tolist()


def test_expert_cache_policy_on_the_host():
    """The replacement policy of the streamed mode's expert cache, replayed without a GPU."""
    # everything fits: each expert is copied once
    assert _simulate(4, 8, [[0, 1, 2], [1, 2, 3], [0, 3], [0, 1, 2, 3]]) == [3, 1, 0, 0]
    # least recently used goes first: after [0,1] [2,3] [0], expert 1 is the oldest and is replaced by 4
    assert _simulate(4, 8, [[0, 1], [2, 3], [0], [4], [0, 2, 3, 4], [1]]) == [2, 2, 0, 1, 0, 1]
    # a repeating call larger than the cache: plain LRU would never hit; keeping the slots that later experts of
    # the same call are about to use saves one copy per call
    assert _simulate(2, 8, [[0, 1, 2]] * 3) == [3, 2, 2]
    # a call larger than the cache keeps what it can: slots reserved by later hits are not taken by earlier misses
    assert _simulate(3, 8, [[5, 6, 7], [0, 5, 6, 7]]) == [3, 2]   # expert 7, needed last, gives its slot to 0 and is reloaded
    # one slot more and only the new expert is copied
    assert _simulate(4, 8, [[5, 6, 7], [0, 5, 6, 7]]) == [3, 1]


def test_expert_cache_simulate_rejects_bad_input():
    import pytest
    from infmoe_b200 import capi
    with pytest.raises(capi.InfMoEError):
        _simulate(2, 4, [[1, 0]])        # not ascending
    with pytest.raises(capi.InfMoEError):
        _simulate(2, 4, [[0, 4]])        # out of range
