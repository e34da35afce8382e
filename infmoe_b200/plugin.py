"""Python mirror of the reference binding (python/infmoe/plugin.py).

`MoELayerPlugin(config, namespace='')` keeps the reference's surface: the
`config` property and `create_plugin(plugin_name)`.  In the reference
create_plugin asks TensorRT's registry for the C++ plugin; here it returns a
`MoELayer`, a thin object over the C ABI that exposes the same life cycle as the
C++ class `MoELayerPlugin` (plugin/MoELayerPlugin.h:91-133): initialize,
configure_plugin, get_workspace_size, enqueue, serialize, clone, terminate.
"""
from __future__ import annotations

import ctypes
import os
import sys
from typing import Optional, Sequence

import numpy as np

from . import capi
from .config import MoELayerConfig

try:  # optional: the reference imports TensorRT unconditionally (python/infmoe/plugin.py:6)
    import tensorrt as trt  # type: ignore
except ImportError:  # pragma: no cover - depends on the installation
    trt = None

PLUGIN_NAME = "MoELayerPlugin"
PLUGIN_VERSION = "1"


def search_library(lib_name: str = "libtrtmoelayer.so") -> str:
    """The TensorRT plugin library, looked for where the reference looks (python/infmoe/plugin.py:14-29): the
    plugin's build directory first, then ./build beside this package, then the package directory itself."""
    here = os.path.dirname(os.path.realpath(__file__))
    for d in (os.path.join(here, "../../plugin/builddir"), os.path.join(here, "build"), here):
        path = os.path.join(d, lib_name)
        if os.path.isfile(path):
            print(f"Loaded library {path}", file=sys.stderr)
            sys.stderr.flush()
            return path
    raise Exception(f"Cannot find {lib_name}, have you run python -m infmoe_b200.build?")


_TRT_STATE = {}


def _trt_creator(namespace: str):
    """Loads libtrtmoelayer.so (its static registration runs on dlopen) and asks TensorRT's registry for the
    creator, like the reference's module-level code (python/infmoe/plugin.py:32-58)."""
    if "lib" not in _TRT_STATE:
        _TRT_STATE["lib"] = ctypes.CDLL(search_library())
        _TRT_STATE["logger"] = trt.Logger(trt.Logger.WARNING)
        trt.init_libnvinfer_plugins(_TRT_STATE["logger"], "")
    creator = trt.get_plugin_registry().get_plugin_creator(PLUGIN_NAME, PLUGIN_VERSION, namespace)
    if creator is None:
        raise Exception("Cannot initialize creator for MoELayerPlugin: check that libtrtmoelayer.so was loaded and "
                        "that it was built against the TensorRT version of the tensorrt Python package")
    return creator


def _fptr(a: Optional[np.ndarray]):
    if a is None:
        return ctypes.cast(None, ctypes.POINTER(ctypes.c_float))
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


class MoELayer:
    """One MoE layer instance (the role of the C++ MoELayerPlugin object)."""

    def __init__(self, handle: int, name: str = "moe_layer_plugin"):
        self._h = ctypes.c_void_p(handle)
        self.name = name
        self._seq_len = -1
        self._ws = None  # torch workspace tensor owned for forward()

    # -- construction ---------------------------------------------------------------------------
    @classmethod
    def create(cls, expert_count: int, embedding_size: int, hidden_size: int, max_concurrency: int,
               expert_centroids: np.ndarray, expert_weight_file: Optional[str], expert_sublayer_type: str = "T5_FF",
               moe_variant: str = "cpm_2", layernorm_weight: Optional[np.ndarray] = None,
               name: str = "moe_layer_plugin") -> "MoELayer":
        """The nine attributes of MoELayerPluginCreator (plugin/MoELayerPluginCreator.cc:15-47)."""
        cent = np.ascontiguousarray(expert_centroids, dtype=np.float32)
        if cent.size != expert_count * embedding_size:
            raise ValueError("expert_centroids must hold expert_count * embedding_size floats")
        ln = None
        if layernorm_weight is not None:
            ln = np.ascontiguousarray(layernorm_weight, dtype=np.float32)
            if ln.size != embedding_size:
                raise ValueError("layernorm_weight must hold embedding_size floats")
        cfg = capi.LayerConfig(
            expert_count, embedding_size, hidden_size, max_concurrency, _fptr(cent), _fptr(ln),
            expert_weight_file.encode("utf-8") if expert_weight_file else None,
            expert_sublayer_type.encode("utf-8"), moe_variant.encode("utf-8"))
        h = ctypes.c_void_p()
        capi.check(capi.lib().infmoe_layer_create(ctypes.byref(cfg), ctypes.byref(h)))
        return cls(h.value, name)

    @classmethod
    def deserialize(cls, blob: bytes, name: str = "moe_layer_plugin") -> "MoELayer":
        h = ctypes.c_void_p()
        buf = ctypes.create_string_buffer(blob, len(blob))
        capi.check(capi.lib().infmoe_layer_deserialize(buf, len(blob), ctypes.byref(h)))
        return cls(h.value, name)

    def clone(self) -> "MoELayer":
        h = ctypes.c_void_p()
        capi.check(capi.lib().infmoe_layer_clone(self._h, ctypes.byref(h)))
        c = MoELayer(h.value, self.name)
        c._seq_len = self._seq_len
        return c

    # -- plugin life cycle ----------------------------------------------------------------------
    def get_plugin_type(self) -> str:
        return PLUGIN_NAME

    def get_plugin_version(self) -> str:
        return PLUGIN_VERSION

    def get_nb_outputs(self) -> int:
        return 1

    def initialize(self) -> int:
        capi.check(capi.lib().infmoe_layer_initialize(self._h))
        return 0

    def configure_plugin(self, input_dims: Sequence[int]) -> None:
        """input [B, S, D] with D == embedding_size (plugin/MoELayerPlugin.cc:170-180)."""
        if len(input_dims) != 3 or input_dims[2] != self.embedding_size:
            raise ValueError("input must be [batch, seq_len, embedding_size]")
        self._seq_len = int(input_dims[1])

    def get_output_dimensions(self, input_dims: Sequence[int]):
        return tuple(input_dims)

    def get_workspace_size(self, token_num: int) -> int:
        n = ctypes.c_size_t()
        capi.check(capi.lib().infmoe_layer_workspace_bytes(self._h, int(token_num), ctypes.byref(n)))
        return int(n.value)

    def set_residency(self, mode: int) -> None:
        capi.check(capi.lib().infmoe_layer_set_residency(self._h, int(mode)))

    def set_expert_cache(self, slots: int) -> None:
        """Streamed mode: keep `slots` experts in device memory across calls (least recently used replaced); 0 = off."""
        capi.check(capi.lib().infmoe_layer_set_expert_cache(self._h, int(slots)))

    def weight_h2d_bytes(self) -> int:
        """Expert weight bytes copied host -> device by enqueue so far."""
        n = ctypes.c_uint64()
        capi.check(capi.lib().infmoe_layer_weight_h2d_bytes(self._h, ctypes.byref(n)))
        return int(n.value)

    def set_expert(self, expert: int, ln_w, wi0, wi1, wo) -> None:
        """Weights by pointer: numpy arrays (host) or CUDA torch tensors (device)."""
        arrs = [ln_w, wi0, wi1, wo]
        if all(isinstance(a, np.ndarray) for a in arrs):
            arrs = [np.ascontiguousarray(a, dtype=np.float32) for a in arrs]
            ptrs = [a.ctypes.data for a in arrs]
            dev = 0
        else:
            arrs = [a.contiguous().float() for a in arrs]
            if not all(a.is_cuda for a in arrs):
                raise ValueError("tensors must all be CUDA tensors")
            ptrs = [a.data_ptr() for a in arrs]
            dev = 1
        D, F = self.embedding_size, self.hidden_size
        sizes = [D, D * F, D * F, D * F]
        for a, n in zip(arrs, sizes):
            got = a.size if isinstance(a, np.ndarray) else a.numel()
            if got != n:
                raise ValueError(f"expert tensor has {got} elements, expected {n}")
        capi.check(capi.lib().infmoe_layer_set_expert(self._h, int(expert), *ptrs, dev))

    def enqueue(self, d_input: int, d_output: int, d_workspace: int, workspace_bytes: int, token_num: int,
                stream: int = 0) -> int:
        capi.check(capi.lib().infmoe_layer_enqueue(self._h, d_input, d_output, d_workspace, workspace_bytes,
                                                   int(token_num), stream))
        return 0

    def expert_forward(self, rows, expert_of_row, out=None, stream: Optional[int] = None):
        """Runs only the experts on CUDA tensor `rows` [n][D] whose expert indices (int32 [n]) are known."""
        import torch

        n = rows.shape[0]
        if out is None:
            out = torch.empty_like(rows)
        if n == 0:
            return out
        need = self.get_workspace_size(n)
        if self._ws is None or self._ws.numel() < need or self._ws.device != rows.device:
            self._ws = torch.empty(need, dtype=torch.uint8, device=rows.device)
        s = torch.cuda.current_stream(rows.device).cuda_stream if stream is None else stream
        capi.check(capi.lib().infmoe_layer_expert_forward(self._h, rows.data_ptr(), expert_of_row.data_ptr(),
                                                          out.data_ptr(), self._ws.data_ptr(), self._ws.numel(), n, s))
        return out

    def expert_forward_scatter(self, rows, expert_of_row, row_dst, row_score=None, stream: Optional[int] = None):
        """Experts on `rows`; the result of row i goes to the address row_dst[i] (int64/uint64 CUDA tensor)."""
        import torch

        n = rows.shape[0]
        if n == 0:
            return
        need = self.get_workspace_size(n)
        if self._ws is None or self._ws.numel() < need or self._ws.device != rows.device:
            self._ws = torch.empty(need, dtype=torch.uint8, device=rows.device)
        s = torch.cuda.current_stream(rows.device).cuda_stream if stream is None else stream
        capi.check(capi.lib().infmoe_layer_expert_forward_scatter(
            self._h, rows.data_ptr(), expert_of_row.data_ptr(), row_score.data_ptr() if row_score is not None else None,
            row_dst.data_ptr(), self._ws.data_ptr(), self._ws.numel(), n, s))

    def sync_status(self, stream: int = 0) -> None:
        capi.check(capi.lib().infmoe_layer_sync_status(self._h, stream))

    def serialize(self) -> bytes:
        n = ctypes.c_size_t()
        capi.check(capi.lib().infmoe_layer_serialization_size(self._h, ctypes.byref(n)))
        buf = ctypes.create_string_buffer(n.value)
        capi.check(capi.lib().infmoe_layer_serialize(self._h, buf, n.value))
        return buf.raw

    def terminate(self) -> None:
        if self._h:
            capi.lib().infmoe_layer_destroy(self._h)
            self._h = None
            self._ws = None

    destroy = terminate

    def __del__(self):
        try:
            self.terminate()
        except Exception:
            pass

    # -- attributes -----------------------------------------------------------------------------
    def _cfg(self) -> capi.LayerConfig:
        cfg = capi.LayerConfig()
        capi.check(capi.lib().infmoe_layer_get_config(self._h, ctypes.byref(cfg)))
        return cfg

    @property
    def expert_count(self) -> int:
        return self._cfg().expert_count

    @property
    def embedding_size(self) -> int:
        return self._cfg().embedding_size

    @property
    def hidden_size(self) -> int:
        return self._cfg().hidden_size

    @property
    def max_concurrency(self) -> int:
        return self._cfg().max_concurrency

    @property
    def moe_variant(self) -> str:
        return self._cfg().moe_variant.decode()

    @property
    def expert_sublayer_type(self) -> str:
        return self._cfg().expert_sublayer_type.decode()

    @property
    def expert_weight_file(self) -> str:
        f = self._cfg().expert_weight_file
        return f.decode() if f else ""

    @property
    def expert_centroids(self) -> np.ndarray:
        c = self._cfg()
        return np.ctypeslib.as_array(c.expert_centroids, (c.expert_count, c.embedding_size)).copy()

    @property
    def layernorm_weight(self) -> Optional[np.ndarray]:
        c = self._cfg()
        if not c.layernorm_weight:
            return None
        return np.ctypeslib.as_array(c.layernorm_weight, (c.embedding_size,)).copy()

    @property
    def kernel_launches(self) -> int:
        return int(capi.lib().infmoe_layer_kernel_launches(self._h))

    # -- conveniences ---------------------------------------------------------------------------
    def forward(self, x, out=None, stream: Optional[int] = None):
        """x: CUDA float32 torch tensor [..., D]; returns a tensor of the same shape (stream ordered)."""
        import torch

        if not (x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()):
            raise ValueError("x must be a contiguous float32 CUDA tensor")
        T = x.numel() // self.embedding_size
        if out is None:
            out = torch.empty_like(x)
        need = self.get_workspace_size(T)
        if self._ws is None or self._ws.numel() < need or self._ws.device != x.device:
            self._ws = torch.empty(need, dtype=torch.uint8, device=x.device)
        s = torch.cuda.current_stream(x.device).cuda_stream if stream is None else stream
        self.enqueue(x.data_ptr(), out.data_ptr(), self._ws.data_ptr(), self._ws.numel(), T, s)
        return out

    def forward_host(self, x: np.ndarray, out: Optional[np.ndarray] = None) -> np.ndarray:
        """Host buffers in and out (copies inside); blocks until the result is there."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        T = x.size // self.embedding_size
        if out is None:
            out = np.empty_like(x)
        capi.check(capi.lib().infmoe_layer_forward_host(self._h, x.ctypes.data, out.ctypes.data, T))
        return out

    def forward_host_ptr(self, h_in: int, h_out: int, token_num: int) -> None:
        capi.check(capi.lib().infmoe_layer_forward_host(self._h, h_in, h_out, int(token_num)))

    def submit_host_ptr(self, h_in: int, h_out: int, token_num: int) -> None:
        """Enqueues a step with host buffers and returns; at most two steps in flight (see wait_host)."""
        capi.check(capi.lib().infmoe_layer_submit_host(self._h, h_in, h_out, int(token_num)))

    def wait_host(self) -> None:
        """Blocks until the oldest submitted step's result is in its output buffer; raises on its status."""
        capi.check(capi.lib().infmoe_layer_wait_host(self._h))

    def set_profiling(self, enable: bool) -> None:
        capi.check(capi.lib().infmoe_layer_set_profiling(self._h, 1 if enable else 0))

    STAGES = ("route", "dispatch", "scatter", "ffn_gemm1", "ffn_gemm2", "combine")

    def stage_ms(self):
        """Average device milliseconds per stage over the calls since the last read -> (dict, calls)."""
        ms = (ctypes.c_float * 6)()
        n = ctypes.c_int32()
        capi.check(capi.lib().infmoe_layer_stage_ms(self._h, ms, ctypes.byref(n)))
        return dict(zip(self.STAGES, [float(v) for v in ms])), int(n.value)

    def last_routing(self):
        """Device pointers (gate, score, pos, count, offset) of the last enqueue."""
        ptrs = [ctypes.c_void_p() for _ in range(5)]
        capi.check(capi.lib().infmoe_layer_last_routing(self._h, *[ctypes.byref(p) for p in ptrs]))
        return tuple(p.value for p in ptrs)


class MoELayerPlugin:
    r"""
    Python binding of MoELayerPlugin
    """

    def __init__(self, config: MoELayerConfig, namespace: str = '') -> None:
        capi.lib()  # fails loudly when the native library is absent
        self.__check_config(config)
        self.__config = config
        self.namespace = namespace

    @property
    def config(self) -> MoELayerConfig:
        return self.__config

    @config.setter
    def config(self, config: MoELayerConfig):
        self.__check_config(config)
        self.__config = config

    # name kept from the reference (python/infmoe/plugin.py:68-71)
    def set_config(self, config: MoELayerConfig):
        self.config = config

    def create_trt_plugin(self, plugin_name='moe_layer_plugin'):
        """The TensorRT IPluginV2 object, created through TensorRT's plugin registry from the nine attributes
        (python/infmoe/plugin.py:92-119 and :73-75 of the reference).  Needs the tensorrt package."""
        if trt is None:
            raise ImportError("the tensorrt Python package is not installed; create_plugin() gives the same layer "
                              "through the C ABI")
        c = self.__config
        if c is None:
            raise Exception('No MoE config provided')
        self._encoded = [c.weight_file_path.encode('utf-8'), c.sublayer_type.encode('utf-8'),
                         c.moe_variant.encode('utf-8')]
        fields = [
            trt.PluginField("expert_count", np.int32(c.expert_count), trt.PluginFieldType.INT32),
            trt.PluginField("embedding_size", np.int32(c.embedding_size), trt.PluginFieldType.INT32),
            trt.PluginField("hidden_size", np.int32(c.hidden_size), trt.PluginFieldType.INT32),
            trt.PluginField("max_concurrency", np.int32(c.max_concurrency), trt.PluginFieldType.INT32),
            trt.PluginField("expert_centroids", c.expert_centroids, trt.PluginFieldType.FLOAT32),
            trt.PluginField("expert_weight_file", self._encoded[0], trt.PluginFieldType.UNKNOWN),
            trt.PluginField("expert_sublayer_type", self._encoded[1], trt.PluginFieldType.UNKNOWN),
            trt.PluginField("moe_variant", self._encoded[2], trt.PluginFieldType.UNKNOWN),
        ]
        if c.layernorm_weight is not None:
            fields.append(trt.PluginField("layernorm_weight", c.layernorm_weight, trt.PluginFieldType.FLOAT32))
        return _trt_creator(self.namespace).create_plugin(plugin_name, trt.PluginFieldCollection(fields))

    def create_plugin(self, plugin_name='moe_layer_plugin'):
        """The plugin object for `config`.  With INFMOE_USE_TENSORRT=1 and the tensorrt package installed this is
        the TensorRT plugin from the registry, as in the reference; otherwise a `MoELayer` over the C ABI with
        the same life cycle, which needs no TensorRT."""
        if trt is not None and os.environ.get("INFMOE_USE_TENSORRT", "0") == "1":
            return self.create_trt_plugin(plugin_name)
        c = self.__config
        if c is None:
            raise Exception('No MoE config provided')
        layer = MoELayer.create(
            expert_count=c.expert_count, embedding_size=c.embedding_size, hidden_size=c.hidden_size,
            max_concurrency=c.max_concurrency, expert_centroids=c.expert_centroids,
            expert_weight_file=c.weight_file_path, expert_sublayer_type=c.sublayer_type,
            moe_variant=c.moe_variant, layernorm_weight=c.layernorm_weight, name=plugin_name)
        if c.seq_len and c.seq_len > 0:
            layer._seq_len = c.seq_len
        return layer

    @staticmethod
    def __check_config(config: MoELayerConfig):
        assert config.expert_count > 0
        assert config.seq_len > 0
        assert config.embedding_size > 0
        assert config.hidden_size > 0
        assert config.max_concurrency > 0
        assert config.max_batch_size > 0
        assert config.sublayer_type != ''
        assert config.expert_centroids is not None and config.expert_centroids.size > 0
        assert config.weight_file_path != '' or config.sublayer_type == 'Identity'
        assert config.moe_variant != ''
