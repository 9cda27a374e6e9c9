"""quant_ops_b200: the W4A4 hot path of libarry/quant_ops, rebuilt for B200 (sm_100a).

Drop-in surface (reference: src/quant_ops/__init__.py:39-45):
    flatquant_dynamic_quantize, dequantize_int4, int4_matmul, get_decompose_dim, CUDA_AVAILABLE
plus the fused layer (w4a4_linear, W4A4Linear) and the weight-side helpers.

    import quant_ops_b200 as quant_ops
"""
from __future__ import annotations

from . import _native
from .decompose import get_decompose_dim
from .ops import (dequantize_int4, device_status, flatquant_cuda, flatquant_dynamic_quantize, int4_matmul, int4_matmul_cuda,
                  int4_matmul_ex, pack_int4_to_int32, prepare_weights, quantize_weights_int4, unpack_int32_to_int4, w4a4_linear,
                  w4a4_linear_prepared)
from . import meta as _meta  # noqa: F401  (registers the fake kernels)
from . import sharding
from .linear import W4A4Linear

__version__ = "1.0.0"


def _cuda_available() -> bool:
    import torch

    return bool(torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10)


CUDA_AVAILABLE = _cuda_available()

__all__ = [
    "flatquant_dynamic_quantize", "flatquant_cuda", "dequantize_int4", "int4_matmul", "int4_matmul_cuda",
    "int4_matmul_ex", "w4a4_linear", "w4a4_linear_prepared", "prepare_weights", "get_decompose_dim", "pack_int4_to_int32", "unpack_int32_to_int4",
    "quantize_weights_int4", "device_status", "W4A4Linear", "sharding", "CUDA_AVAILABLE", "__version__",
]
