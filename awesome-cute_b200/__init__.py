"""B200 (sm_100a) W4A16 GEMM: drop-in for the Marlin path of CalebDu/Awesome-Cute (gemm/marlin_gemm).

The directory name carries a hyphen, so load it through ``__graft_entry__.load_package()`` (or
importlib) under the module name ``awesome_cute_b200``.
"""
from . import _lib  # raises if libw4a16.so is not built: there is no fallback
from ._lib import plan
from .marlin import (HostGemm, Layer, load_packed, quantize_pack_device, save_packed, device_status, mul, mul_gather, mul_host, mul_simt, pack_weights, permute_scales, quantize_pack,
                     shard_columns, unpack_weights, unpermute_scales)

from .sharded import ColumnShardedLayer, GatherBuffers, all_gather_columns

__all__ = ["plan", "ColumnShardedLayer", "GatherBuffers", "all_gather_columns", "mul_gather", "Layer", "mul", "mul_simt", "mul_host", "HostGemm", "quantize_pack_device", "save_packed", "load_packed", "device_status", "pack_weights", "unpack_weights", "permute_scales",
           "unpermute_scales", "quantize_pack", "shard_columns"]
