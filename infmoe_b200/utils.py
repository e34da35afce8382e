"""The helper functions of the reference's python/infmoe/utils.py, same names and call pattern.

    inputs, outputs, bindings, stream = allocate_buffers(engine)
    out_host, = do_inference(context, bindings, inputs, outputs, stream, batch_size)
    layer = create_layer_from_plugin(network, plugin, [input_tensor], name)

With a real TensorRT engine / network these do what the reference's do (python/infmoe/utils.py:21-65), on torch
tensors instead of pycuda allocations.  Without TensorRT (it is not installed where this library is developed)
the same calls work on the small stand-ins below, which play TensorRT's part for a network that consists of MoE
layers only: `LayerNetwork` collects plugins, `LayerEngine` fixes the input shape and owns the workspace,
`LayerContext.execute_async` enqueues the layers on the caller's stream.  That keeps the reference's demo flow
(python/examples/stacked_moe.py) runnable end to end through the C ABI.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np

try:  # the reference imports these at module level; here they are optional
    import tensorrt as trt  # type: ignore
except ImportError:  # pragma: no cover - depends on the installation
    trt = None

__all__ = ["HostDeviceMem", "allocate_buffers", "do_inference", "create_layer_from_plugin", "LayerNetwork",
           "LayerEngine", "LayerContext"]


class HostDeviceMem(object):
    r"""
    Represent corresponding CPU & GPU buffer: `host` is a numpy view of page-locked memory, `device` a CUDA tensor
    """

    def __init__(self, host_mem, device_mem):
        self.host = host_mem
        self.device = device_mem

    def __str__(self):
        return "Host:\n" + str(self.host) + "\nDevice:\n" + str(self.device)

    def __repr__(self):
        return self.__str__()


class _Output:
    def __init__(self, name):
        self.name = name


class _NetworkLayer:
    """What add_plugin_v2 returns, as far as the reference's helper uses it."""

    def __init__(self, plugin, inputs):
        self.plugin = plugin
        self.inputs = list(inputs)
        self._out = _Output("")

    def get_output(self, index: int):
        assert index == 0
        return self._out


class LayerNetwork:
    """A network of MoE layers applied one after the other to one [B, S, D] input (TensorRT stand-in)."""

    def __init__(self, input_name: str = "input"):
        self.input_name = input_name
        self.layers: List[_NetworkLayer] = []

    def add_plugin_v2(self, inputs, plugin):
        layer = _NetworkLayer(plugin, inputs)
        self.layers.append(layer)
        return layer

    def build_engine(self, input_shape: Sequence[int], max_batch_size: int = 1) -> "LayerEngine":
        return LayerEngine(self, tuple(int(v) for v in input_shape), int(max_batch_size))


class LayerEngine:
    """Fixed input shape [S, D] per batch item, max_batch_size items: the part of ICudaEngine the helpers touch."""

    def __init__(self, network: LayerNetwork, input_shape, max_batch_size: int):
        if not network.layers:
            raise ValueError("the network has no layers")
        self.network = network
        self.shape = input_shape            # per batch item, e.g. (seq_len, d_model)
        self.max_batch_size = max_batch_size
        self.bindings = [network.input_name, network.layers[-1].get_output(0).name or "output"]
        for layer in network.layers:
            layer.plugin.configure_plugin((max_batch_size,) + tuple(input_shape))
            layer.plugin.initialize()

    def __iter__(self):
        return iter(self.bindings)

    def get_binding_shape(self, binding):
        return self.shape

    def binding_is_input(self, binding):
        return binding == self.bindings[0]

    def create_execution_context(self) -> "LayerContext":
        return LayerContext(self)


class LayerContext:
    def __init__(self, engine: LayerEngine):
        self.engine = engine
        # TensorRT runs clones of the plugins, one set per execution context; the weights are shared
        self.layers = [l.plugin.clone() for l in engine.network.layers]
        self._mid = None

    def execute_async(self, batch_size=1, bindings=None, stream_handle=0):
        import torch

        S, D = self.engine.shape
        T = int(batch_size) * S
        src, dst = int(bindings[0]), int(bindings[1])
        n = len(self.layers)
        if n > 1 and (self._mid is None or self._mid[0].numel() < T * D):
            self._mid = [torch.empty(T * D, dtype=torch.float32, device="cuda") for _ in range(2)]
        for i, layer in enumerate(self.layers):
            out = dst if i == n - 1 else self._mid[i % 2].data_ptr()
            need = layer.get_workspace_size(T)
            if layer._ws is None or layer._ws.numel() < need:
                layer._ws = torch.empty(need, dtype=torch.uint8, device="cuda")
            layer.enqueue(src, out, layer._ws.data_ptr(), layer._ws.numel(), T, int(stream_handle))
            src = out
        return True


def allocate_buffers(engine):
    r"""
    Allocate page-locked host and GPU buffers for every binding of the engine
    """
    import torch

    inputs, outputs, bindings = [], [], []
    stream = torch.cuda.Stream()
    for binding in engine:
        if trt is not None and not isinstance(engine, LayerEngine):
            size = trt.volume(engine.get_binding_shape(binding)) * engine.max_batch_size
            dtype = trt.nptype(engine.get_binding_dtype(binding))
        else:
            size = int(np.prod(engine.get_binding_shape(binding))) * engine.max_batch_size
            dtype = np.float32
        host = torch.empty(size, dtype=torch.from_numpy(np.empty(0, dtype)).dtype).pin_memory()
        device = torch.empty(size, dtype=host.dtype, device="cuda")
        bindings.append(int(device.data_ptr()))
        mem = HostDeviceMem(host.numpy(), device)
        mem._host_tensor = host        # keeps the pinned allocation alive
        (inputs if engine.binding_is_input(binding) else outputs).append(mem)
    return inputs, outputs, bindings, stream


def do_inference(context, bindings, inputs, outputs, stream, batch_size=1):
    r"""
    Run inference (inputs & outputs are CPU buffers)
    """
    import torch

    with torch.cuda.stream(stream):
        for inp in inputs:
            inp.device.copy_(inp._host_tensor, non_blocking=True)
        context.execute_async(batch_size=batch_size, bindings=bindings, stream_handle=stream.cuda_stream)
        for out in outputs:
            out._host_tensor.copy_(out.device, non_blocking=True)
    stream.synchronize()
    return [out.host for out in outputs]


def create_layer_from_plugin(network, plugin, inputs, name='moe_output'):
    moe_layer = network.add_plugin_v2(inputs=inputs, plugin=plugin)
    moe_layer.get_output(0).name = name
    return moe_layer
