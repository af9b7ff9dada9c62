"""relux_b200 -- B200-native KV-cache append and cached-attention decode for relux.

The product is the C-ABI library `librelux_cuda.so` (sources in relux_b200/csrc, interface in
include/relux_cuda.h).  This package is the thin host-side mirror of relux's cache / attention
interface used by the tests and the benchmark.
"""
from . import lib  # noqa: F401
from .api import Device, DeviceBuffer, Pool, KVCache, MLACache, BFloat16  # noqa: F401
