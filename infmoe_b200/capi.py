"""ctypes binding of the C ABI declared in include/infmoe_c.h.

The library is loaded from the package directory; there is no fallback: if
libinfmoe_b200.so is missing or fails to load, importing the symbols raises.
Device pointers are passed as plain integers (e.g. ``tensor.data_ptr()``).
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libinfmoe_b200.so")

STATUS_NAMES = {
    0: "INFMOE_OK",
    1: "INFMOE_ERR_INVALID_ARGUMENT",
    2: "INFMOE_ERR_CUDA",
    3: "INFMOE_ERR_NAN",
    4: "INFMOE_ERR_IO",
    5: "INFMOE_ERR_FORMAT",
    6: "INFMOE_ERR_UNSUPPORTED",
    7: "INFMOE_ERR_DEVICE_TIMEOUT",
    8: "INFMOE_ERR_STATE",
}


class InfMoEError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


class LayerConfig(ctypes.Structure):
    """struct infmoe_layer_config"""

    _fields_ = [
        ("expert_count", ctypes.c_int32),
        ("embedding_size", ctypes.c_int32),
        ("hidden_size", ctypes.c_int32),
        ("max_concurrency", ctypes.c_int32),
        ("expert_centroids", ctypes.POINTER(ctypes.c_float)),
        ("layernorm_weight", ctypes.POINTER(ctypes.c_float)),
        ("expert_weight_file", ctypes.c_char_p),
        ("expert_sublayer_type", ctypes.c_char_p),
        ("moe_variant", ctypes.c_char_p),
    ]


class EpConfig(ctypes.Structure):
    """struct infmoe_ep_config"""

    _fields_ = [
        ("rank", ctypes.c_int32),
        ("world", ctypes.c_int32),
        ("unique_id", ctypes.c_void_p),
        ("expert_count", ctypes.c_int32),
        ("embedding_size", ctypes.c_int32),
        ("hidden_size", ctypes.c_int32),
        ("max_tokens", ctypes.c_int64),
        ("expert_centroids", ctypes.POINTER(ctypes.c_float)),
        ("layernorm_weight", ctypes.POINTER(ctypes.c_float)),
        ("moe_variant", ctypes.c_char_p),
        ("local_experts", ctypes.c_void_p),
    ]


EP_ID_BYTES = 128

SUB_INIT_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_char_p)
SUB_WEIGHT_SIZE_FN = ctypes.CFUNCTYPE(ctypes.c_size_t, ctypes.c_void_p)
SUB_WS_SIZE_FN = ctypes.CFUNCTYPE(ctypes.c_size_t, ctypes.c_void_p, ctypes.c_int32)
SUB_COPY_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p)
SUB_RUN_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                              ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p)


class SublayerVtable(ctypes.Structure):
    """struct infmoe_sublayer_vtable"""

    _fields_ = [
        ("user", ctypes.c_void_p),
        ("initialize", SUB_INIT_FN),
        ("weight_size", SUB_WEIGHT_SIZE_FN),
        ("workspace_size", SUB_WS_SIZE_FN),
        ("copy_weights", SUB_COPY_FN),
        ("run", SUB_RUN_FN),
    ]


_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_i32 = ctypes.c_int32
_sz = ctypes.c_size_t

# name -> argument types (every function returns int unless listed in _RESTYPES)
SIGNATURES = {
    "infmoe_layer_create": [ctypes.POINTER(LayerConfig), ctypes.POINTER(_vp)],
    "infmoe_layer_clone": [_vp, ctypes.POINTER(_vp)],
    "infmoe_layer_initialize": [_vp],
    "infmoe_layer_set_expert": [_vp, _i32, _vp, _vp, _vp, _vp, ctypes.c_int],
    "infmoe_layer_set_residency": [_vp, ctypes.c_int],
    "infmoe_layer_set_file_expert_offset": [_vp, _i32],
    "infmoe_layer_set_expert_cache": [_vp, _i32],
    "infmoe_layer_weight_h2d_bytes": [_vp, ctypes.POINTER(ctypes.c_uint64)],
    "infmoe_expert_cache_simulate": [_i32, _i32, _vp, _vp, _i32, _vp],
    "infmoe_wait_timeout_probe": [ctypes.c_uint32, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_float)],
    "infmoe_layer_workspace_bytes": [_vp, _i64, ctypes.POINTER(_sz)],
    "infmoe_layer_enqueue": [_vp, _vp, _vp, _vp, _sz, _i64, _vp],
    "infmoe_layer_expert_forward": [_vp, _vp, _vp, _vp, _vp, _sz, _i64, _vp],
    "infmoe_layer_expert_forward_scatter": [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _i64, _vp],
    "infmoe_layer_sync_status": [_vp, _vp],
    "infmoe_layer_forward_host": [_vp, _vp, _vp, _i64],
    "infmoe_layer_submit_host": [_vp, _vp, _vp, _i64],
    "infmoe_layer_wait_host": [_vp],
    "infmoe_layer_last_routing": [_vp] + [ctypes.POINTER(_vp)] * 5,
    "infmoe_layer_kernel_launches": [_vp],
    "infmoe_layer_set_profiling": [_vp, ctypes.c_int],
    "infmoe_layer_stage_ms": [_vp, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(_i32)],
    "infmoe_layer_destroy": [_vp],
    "infmoe_layer_serialization_size": [_vp, ctypes.POINTER(_sz)],
    "infmoe_layer_serialize": [_vp, _vp, _sz],
    "infmoe_layer_deserialize": [_vp, _sz, ctypes.POINTER(_vp)],
    "infmoe_layer_get_config": [_vp, ctypes.POINTER(LayerConfig)],
    "infmoe_weight_file_check": [ctypes.c_char_p, _i32, _i32, _i32, _vp],
    "infmoe_route": [_vp, _vp, _vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp],
    "infmoe_expert_select": [_i64, _i32, _vp, _vp, _vp, _vp, _vp],
    "infmoe_expert_count": [_i64, _i32, _vp, _vp, _vp, _vp, _vp, _vp],
    "infmoe_expert_scatter": [_i64, _i32, _vp, _vp, _vp, _vp, _vp, _vp],
    "infmoe_expert_gather": [_i64, _i32, _vp, _vp, _vp, _vp],
    "infmoe_expert_mix_gather": [_i64, _i32, _vp, _vp, _vp, _vp, _vp, _vp],
    "infmoe_layernorm": [_vp, _vp, _i64, _i32, _vp, _vp],
    "infmoe_gelu_dot": [_vp, _vp, _sz, _vp],
    "infmoe_t5ff_workspace_bytes": [_i64, _i32, _i32, ctypes.POINTER(_sz)],
    "infmoe_t5ff_run": [_i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp],
    "infmoe_t5ff_static_limit": [_i64, _i32, _i32, ctypes.POINTER(_sz), ctypes.POINTER(_sz)],
    "infmoe_t5ff_run_static": [_i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "infmoe_register_sublayer": [ctypes.c_char_p, ctypes.POINTER(SublayerVtable)],
    "infmoe_ep_unique_id": [_vp],
    "infmoe_ep_create": [ctypes.POINTER(EpConfig), ctypes.POINTER(_vp)],
    "infmoe_ep_create_sharded": [ctypes.POINTER(LayerConfig), _i32, _i32, _vp, _i64, ctypes.POINTER(_vp),
                                 ctypes.POINTER(_vp)],
    "infmoe_ep_create_loopback": [ctypes.POINTER(EpConfig), _i32, ctypes.POINTER(_vp)],
    "infmoe_ep_forward": [_vp, _vp, _vp, _i64, _vp],
    "infmoe_ep_forward_begin": [_vp, _vp, _i64, _vp],
    "infmoe_ep_forward_experts": [_vp, _vp],
    "infmoe_ep_forward_end": [_vp, _vp, _vp],
    "infmoe_ep_output": [_vp, ctypes.POINTER(_vp)],
    "infmoe_ep_forward_host": [_vp, _vp, _vp, _i64],
    "infmoe_ep_submit_host": [_vp, _vp, _vp, _i64],
    "infmoe_ep_wait_host": [_vp],
    "infmoe_ep_sync_status": [_vp, _vp],
    "infmoe_ep_last_routing": [_vp] + [ctypes.POINTER(_vp)] * 5,
    "infmoe_ep_received": [_vp, ctypes.POINTER(_vp), ctypes.POINTER(_vp), ctypes.POINTER(_vp), ctypes.POINTER(_i64)],
    "infmoe_ep_set_profiling": [_vp, ctypes.c_int],
    "infmoe_ep_phase_ms": [_vp, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(_i32)],
    "infmoe_ep_destroy": [_vp],
    "infmoe_last_error": [],
}
_RESTYPES = {"infmoe_last_error": ctypes.c_char_p, "infmoe_layer_kernel_launches": ctypes.c_int64}

_lib = None


def lib() -> ctypes.CDLL:
    """Loads libinfmoe_b200.so and declares every entry point of infmoe_c.h."""
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m infmoe_b200.build` (there is no CPU fallback)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(handle, name)  # raises AttributeError if a declared symbol is not exported
            fn.argtypes = args
            fn.restype = _RESTYPES.get(name, ctypes.c_int)
        _lib = handle
    return _lib


def last_error() -> str:
    msg = lib().infmoe_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(status: int) -> None:
    if status != 0:
        raise InfMoEError(status, last_error())
