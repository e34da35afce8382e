"""B200-native MoE layer behind InfMoE's plugin interface.

Public surface (same names as the reference's python/infmoe/__init__.py:6-10):
MoELayerConfig, MoELayerPlugin; plus MoELayer, the object create_plugin returns.
"""
from .config import MoELayerConfig
from .plugin import MoELayer, MoELayerPlugin

__version__ = '0.0.1'
__all__ = ["MoELayerConfig", "MoELayerPlugin", "MoELayer"]
