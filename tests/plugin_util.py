"""ctypes access to libtrtmoelayer.so's host driver (the entry points that play TensorRT's part)."""
import ctypes
import os

import numpy as np

from infmoe_b200 import capi

PKG = os.path.dirname(os.path.abspath(capi.__file__))
LIB_PATH = os.path.join(PKG, "libtrtmoelayer.so")

INT32, FLOAT32, UNKNOWN = 5, 1, 8     # nvinfer1::PluginFieldType


class Field(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("data", ctypes.c_void_p), ("type", ctypes.c_int32),
                ("length", ctypes.c_int32)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        capi.lib()
        h = ctypes.CDLL(LIB_PATH)
        for name, res, args in [
            ("trtmoe_get_creator", ctypes.c_void_p, [ctypes.c_char_p, ctypes.c_char_p]),
            ("trtmoe_creator_field_names", ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_char_p), ctypes.c_int32]),
            ("trtmoe_create_plugin", ctypes.c_void_p, [ctypes.c_void_p, ctypes.c_char_p, ctypes.POINTER(Field), ctypes.c_int32]),
            ("trtmoe_deserialize_plugin", ctypes.c_void_p, [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_size_t]),
            ("trtmoe_plugin_type", ctypes.c_char_p, [ctypes.c_void_p]),
            ("trtmoe_plugin_version", ctypes.c_char_p, [ctypes.c_void_p]),
            ("trtmoe_plugin_nb_outputs", ctypes.c_int, [ctypes.c_void_p]),
            ("trtmoe_plugin_supports", ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int32, ctypes.c_int32]),
            ("trtmoe_plugin_configure", None, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]),
            ("trtmoe_plugin_workspace", ctypes.c_size_t, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]),
            ("trtmoe_plugin_initialize", ctypes.c_int, [ctypes.c_void_p]),
            ("trtmoe_plugin_enqueue", ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                                     ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
            ("trtmoe_plugin_serialization_size", ctypes.c_size_t, [ctypes.c_void_p]),
            ("trtmoe_plugin_serialize", None, [ctypes.c_void_p, ctypes.c_void_p]),
            ("trtmoe_plugin_clone", ctypes.c_void_p, [ctypes.c_void_p]),
            ("trtmoe_plugin_set_namespace", None, [ctypes.c_void_p, ctypes.c_char_p]),
            ("trtmoe_plugin_namespace", ctypes.c_char_p, [ctypes.c_void_p]),
            ("trtmoe_plugin_layer", ctypes.c_void_p, [ctypes.c_void_p]),
            ("trtmoe_plugin_delete", None, [ctypes.c_void_p]),
        ]:
            f = getattr(h, name)
            f.restype, f.argtypes = res, args
        _lib = h
    return _lib


def make_fields(**attrs):
    """The PluginFieldCollection python/infmoe/plugin.py:92-119 builds: ints as INT32, arrays as FLOAT32,
    strings as raw bytes with type UNKNOWN."""
    keep, fields = [], []
    for name, v in attrs.items():
        if isinstance(v, (int, np.integer)):
            a = np.array([v], np.int32)
            keep.append(a)
            fields.append(Field(name.encode(), a.ctypes.data, INT32, 1))
        elif isinstance(v, np.ndarray):
            a = np.ascontiguousarray(v, np.float32)
            keep.append(a)
            fields.append(Field(name.encode(), a.ctypes.data, FLOAT32, a.size))
        else:
            b = ctypes.create_string_buffer(v.encode() if isinstance(v, str) else v)
            keep.append(b)
            fields.append(Field(name.encode(), ctypes.cast(b, ctypes.c_void_p).value, UNKNOWN, len(b.raw) - 1))
    arr = (Field * len(fields))(*fields)
    return arr, len(fields), keep


def layer_config(plugin):
    cfg = capi.LayerConfig()
    capi.check(capi.lib().infmoe_layer_get_config(lib().trtmoe_plugin_layer(plugin), ctypes.byref(cfg)))
    return cfg
