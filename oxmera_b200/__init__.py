"""oxmera_b200: the matmul path of oxmera on B200 (sm_100a).

The product is the C-ABI library `liboxmera_b200.so` (include/oxmera_b200.h,
built from oxmera_b200/csrc).  This package is the host-side mirror of the
oxmera vocabulary (DType, Device, Layout, Tensor, Backend, registry) over that
ABI, used by the tests and the benchmark.
"""
from .core import (BackendFault, BackendUnavailable, BroadcastIncompatible, DType, Device, DeviceMismatch,
                   DivisionByZero, DTypeMismatch, IndexOutOfBounds, Layout, NotImplementedOp, OxmeraError, RankMismatch,
                   ShapeMismatch, UnsupportedDType, broadcast_shapes, contiguous_strides, numel)
from .tensor import Storage, Tensor, bf16_bits_to_f32, f32_to_bf16_bits
from .backend import (B200Backend, backend_for, register_backend, shard_plan, shard_ranges, sharded_matmul_host,
                      unregister_all)

__all__ = [
    "B200Backend", "BackendFault", "BackendUnavailable", "BroadcastIncompatible", "DType", "Device",
    "DeviceMismatch", "DivisionByZero", "DTypeMismatch", "IndexOutOfBounds", "Layout", "NotImplementedOp", "OxmeraError",
    "RankMismatch", "ShapeMismatch", "Storage", "Tensor", "UnsupportedDType", "backend_for",
    "bf16_bits_to_f32", "broadcast_shapes", "contiguous_strides", "f32_to_bf16_bits", "numel",
    "register_backend", "shard_plan", "shard_ranges", "sharded_matmul_host", "unregister_all",
]
