"""MoELayerPlugin / MoELayerPluginCreator (C++, libtrtmoelayer.so) driven the way TensorRT drives them: registry
lookup, attribute parsing, configure, workspace size, serialise/deserialise, clone.  No GPU needed."""
import ctypes

import numpy as np
import pytest

from tests import plugin_util as pu

CENT = np.arange(24, dtype=np.float32).reshape(3, 8)


def _creator():
    c = pu.lib().trtmoe_get_creator(b"MoELayerPlugin", b"1")
    assert c, "the creator did not register itself when the library was loaded"
    return c


def _create(**attrs):
    arr, n, keep = pu.make_fields(**attrs)
    return pu.lib().trtmoe_create_plugin(_creator(), b"moe_layer_plugin", arr, n)


def test_creator_is_registered_with_the_nine_attributes():
    assert not pu.lib().trtmoe_get_creator(b"MoELayerPlugin", b"2")
    names = (ctypes.c_char_p * 16)()
    n = pu.lib().trtmoe_creator_field_names(_creator(), names, 16)
    assert [names[i].decode() for i in range(n)] == [
        "expert_count", "embedding_size", "hidden_size", "max_concurrency", "expert_centroids", "expert_weight_file",
        "expert_sublayer_type", "moe_variant", "layernorm_weight"]


def test_create_plugin_defaults_and_surface():
    ln = np.linspace(1, 2, 8, dtype=np.float32)
    p = _create(expert_count=3, embedding_size=8, hidden_size=16, expert_centroids=CENT, layernorm_weight=ln)
    assert p
    L = pu.lib()
    assert L.trtmoe_plugin_type(p) == b"MoELayerPlugin" and L.trtmoe_plugin_version(p) == b"1"
    assert L.trtmoe_plugin_nb_outputs(p) == 1
    cfg = pu.layer_config(p)
    # defaults of the reference's creator: T5_FF experts, cpm_2 variant, two weight slots
    assert (cfg.max_concurrency, cfg.expert_sublayer_type, cfg.moe_variant) == (2, b"T5_FF", b"cpm_2")
    assert L.trtmoe_plugin_supports(p, 0, 0, 0) == 1 and L.trtmoe_plugin_supports(p, 1, 0, 0) == 1
    assert L.trtmoe_plugin_supports(p, 0, 1, 0) == 0          # FP16 is not offered
    assert L.trtmoe_plugin_supports(p, 0, 0, 1) == 0          # nor a non-linear layout
    assert L.trtmoe_plugin_workspace(p, 2, 4, 8) == 0          # not configured yet
    L.trtmoe_plugin_configure(p, 2, 4, 8)
    from infmoe_b200 import capi
    want = ctypes.c_size_t()
    capi.check(capi.lib().infmoe_layer_workspace_bytes(L.trtmoe_plugin_layer(p), 8, ctypes.byref(want)))
    assert L.trtmoe_plugin_workspace(p, 2, 4, 8) == want.value
    L.trtmoe_plugin_set_namespace(p, b"ns")
    assert L.trtmoe_plugin_namespace(p) == b"ns"
    L.trtmoe_plugin_delete(p)


def test_create_plugin_rejects_bad_attributes(capfd):
    ok = dict(expert_count=3, embedding_size=8, hidden_size=16, expert_centroids=CENT, moe_variant="default")
    assert not _create(**ok, bogus_field=1)
    assert "unknown plugin field bogus_field" in capfd.readouterr().err
    assert not _create(**{**ok, "moe_variant": "cpm_2"})                       # layernorm_weight missing
    assert "layernorm_weight" in capfd.readouterr().err
    assert not _create(**{**ok, "expert_centroids": CENT[:2]})
    assert "expert_centroids" in capfd.readouterr().err
    assert not _create(**{**ok, "moe_variant": "sparse"})
    assert "unsupported moe variant" in capfd.readouterr().err
    assert not _create(**ok, expert_sublayer_type="Conv")
    assert "unsupported sublayer type" in capfd.readouterr().err
    assert not _create(**ok, expert_weight_file="/nonexistent/weights.npz")
    assert "not a regular file" in capfd.readouterr().err
    assert not _create(embedding_size=8, hidden_size=16, expert_centroids=CENT)
    p = _create(**ok)
    assert p
    pu.lib().trtmoe_plugin_delete(p)


def test_serialize_deserialize_and_clone(tmp_path):
    from infmoe_b200 import synth
    w = synth.scaled(synth.WORKLOADS["tiny_default"], expert_count=3, embedding_size=8, hidden_size=16)
    path = synth.write_npz(w, str(tmp_path / "w.npz"))
    p = _create(expert_count=3, embedding_size=8, hidden_size=16, max_concurrency=3, expert_centroids=CENT,
                expert_weight_file=path, expert_sublayer_type="T5_FF", moe_variant="base_layer")
    L = pu.lib()
    n = L.trtmoe_plugin_serialization_size(p)
    buf = ctypes.create_string_buffer(n)
    L.trtmoe_plugin_serialize(p, buf)
    q = L.trtmoe_deserialize_plugin(_creator(), b"restored", buf, n)
    c = L.trtmoe_plugin_clone(p)
    assert q and c
    for other in (q, c):
        cfg = pu.layer_config(other)
        assert (cfg.expert_count, cfg.embedding_size, cfg.hidden_size, cfg.max_concurrency) == (3, 8, 16, 3)
        assert cfg.moe_variant == b"base_layer" and cfg.expert_weight_file.decode() == path
        np.testing.assert_array_equal(np.ctypeslib.as_array(cfg.expert_centroids, (3, 8)), CENT)
        assert L.trtmoe_plugin_serialization_size(other) == n
    buf2 = ctypes.create_string_buffer(n)
    L.trtmoe_plugin_serialize(q, buf2)
    assert buf.raw == buf2.raw
    assert not L.trtmoe_deserialize_plugin(_creator(), b"bad", buf, n - 4)
    for x in (p, q, c):
        L.trtmoe_plugin_delete(x)
