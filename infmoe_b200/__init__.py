"""B200-native MoE layer behind InfMoE's plugin interface.

Public surface (same names as the reference's python/infmoe/__init__.py:6-10):
MoELayerConfig, MoELayerPlugin and the helpers of utils; plus MoELayer, the object create_plugin returns.
"""
from .config import MoELayerConfig
from .plugin import MoELayer, MoELayerPlugin
from .utils import HostDeviceMem, allocate_buffers, create_layer_from_plugin, do_inference

__version__ = '0.0.1'
__all__ = ["MoELayerConfig", "MoELayerPlugin", "MoELayer", "HostDeviceMem", "allocate_buffers", "do_inference",
           "create_layer_from_plugin"]
