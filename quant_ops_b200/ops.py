"""Python operator layer: the reference's public functions, backed by the sm_100a kernels only.

Names, argument order, defaults and output shapes follow the reference
(src/quant_ops/ops/quantization/flatquant/ops.py:133-178, src/quant_ops/ops/quantization/int4_matmul/ops.py:140-157).
Two deliberate differences: there is no fallback chain (a failed check raises, CPU tensors raise) and the
per-token scales are float32 [tokens] whose values are the reference's dtype-rounded scales, which is what the
reference's own CUDA op and fake kernel return and what int4_matmul requires.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _native

_native.load_torch_binding()
_ops = torch.ops.quant_ops


def flatquant_dynamic_quantize(input_tensor: torch.Tensor, left_trans: torch.Tensor, right_trans: torch.Tensor,
                               clip_ratio: float = 1.0, pack_int32: bool = False, *,
                               scale_dtype: Optional[torch.dtype] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Kronecker transform L^T.X.R per token, clip-scaled absmax scale, int4 codes (int8 or 8 per int32).

    The positional arguments are the reference's.  `scale_dtype` (keyword only, an addition) stores the per-token
    scales as float16 / bfloat16 instead of float32; the value is the same, the reference's scale being a value of
    the input dtype already (float16 scales of bfloat16 inputs are rounded once more).
    """
    if scale_dtype is None:
        return _ops.flatquant_dynamic_quantize(input_tensor, left_trans, right_trans, float(clip_ratio), bool(pack_int32))
    return _ops.flatquant_dynamic_quantize_ex(input_tensor, left_trans, right_trans, float(clip_ratio), bool(pack_int32), scale_dtype)


def device_status(stream: Optional[torch.cuda.Stream] = None) -> None:
    """Waits for `stream` (default: the current stream) and raises RuntimeError if a kernel of this library gave up
    on one of its bounded device-side waits since the last check; outputs written since then are not valid.

    The reference checks cudaGetLastError after a blocking synchronise inside every call
    (src/quant_ops/ops/quantization/flatquant/kernels/cuda_quant_kernel.cu:380-387); here calls never block, so the
    check is a call of its own, to be made wherever the caller synchronises anyway.
    """
    import ctypes

    st = stream if stream is not None else torch.cuda.current_stream()
    _native.check(_native.lib.qo_device_status(ctypes.c_void_p(st.cuda_stream)))


def flatquant_cuda(input_tensor, left_trans, right_trans, clip_ratio: float = 1.0, pack_int32: bool = False):
    """Reference alias (flatquant/ops.py:54-75): moves the three tensors to the current GPU first."""
    return flatquant_dynamic_quantize(input_tensor.cuda(), left_trans.cuda(), right_trans.cuda(), clip_ratio, pack_int32)


def dequantize_int4(quantized: torch.Tensor, scales: torch.Tensor, packed_int32: bool = False) -> torch.Tensor:
    """codes * per-token scale as float32 [tokens, features]."""
    return _ops.dequantize_int4(quantized, scales, bool(packed_int32))


def int4_matmul(a_packed: torch.Tensor, b_packed: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor) -> torch.Tensor:
    """[T, K/8] x [K/8, N] packed int4 -> float16 [T, N] = (int32 acc * scale_a[row]) * scale_b[col]."""
    return _ops.int4_matmul(a_packed, b_packed, scale_a, scale_b)


def int4_matmul_cuda(a_packed, b_packed, scale_a, scale_b):
    """Reference alias (int4_matmul/ops.py:106-137): moves operands to the GPU; strided operands are accepted."""
    return int4_matmul(a_packed.cuda(), b_packed.cuda(), scale_a.cuda(), scale_b.cuda())


def int4_matmul_ex(a_packed, b_packed, scale_a, scale_b, out_dtype: torch.dtype = torch.float16,
                   return_accumulators: bool = False):
    """int4_matmul with a choice of output dtype (float16 / bfloat16) and optional raw int32 accumulators."""
    out, acc = _ops.int4_matmul_ex(a_packed, b_packed, scale_a, scale_b, out_dtype, bool(return_accumulators))
    return (out, acc) if return_accumulators else out


def w4a4_linear(x: torch.Tensor, left_trans: torch.Tensor, right_trans: torch.Tensor, w_packed: torch.Tensor,
                w_scale: torch.Tensor, bias: Optional[torch.Tensor] = None, clip_ratio: float = 1.0,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Fused quantize -> int4 GEMM.  w_packed is [n_out, K/8] (K contiguous), w_scale float32 [n_out]."""
    return _ops.w4a4_linear(x, left_trans, right_trans, w_packed, w_scale, bias, float(clip_ratio), out_dtype)


def prepare_weights(w_packed: torch.Tensor) -> torch.Tensor:
    """Packed weights [n_out, K/8] -> the int8 operand of the tensor-core GEMM (a byte tensor in the kernel's blocked
    layout: 256 output channels x 128 values per 32 KB block), made once at load time for w4a4_linear_prepared."""
    return _ops.prepare_weights(w_packed)


def w4a4_linear_prepared(x: torch.Tensor, left_trans: torch.Tensor, right_trans: torch.Tensor, w_packed: torch.Tensor,
                         w_prepared: torch.Tensor, w_scale: torch.Tensor, bias: Optional[torch.Tensor] = None,
                         clip_ratio: float = 1.0, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """w4a4_linear with the weights also given as the int8 copy made by prepare_weights: same results, no per-call
    rewriting of either operand (the activations are quantized straight to int8 codes)."""
    return _ops.w4a4_linear_prepared(x, left_trans, right_trans, w_packed, w_prepared, w_scale, bias, float(clip_ratio), out_dtype)


def pack_int4_to_int32(tensor: torch.Tensor) -> torch.Tensor:
    """int8 codes [rows, F] in [-8, 7] -> int32 [rows, F/8], nibble i of a word = code[8p+i] + 8."""
    return _ops.pack_int4(tensor)


def unpack_int32_to_int4(packed: torch.Tensor) -> torch.Tensor:
    return _ops.unpack_int4(packed)


def quantize_weights_int4(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-output-channel symmetric int4 (absmax/7): returns (packed [rows, K/8] int32, scale [rows] float32)."""
    return _ops.quantize_weights_int4(w)
