"""Fake (meta) kernels so the ops can be traced by FakeTensor / torch.compile / CUDA-graph capture tooling.

Shape and dtype contract of the reference's fake kernels (src/quant_ops/meta_ops.py:22-37).
"""
from __future__ import annotations

import torch
from torch.library import register_fake

from . import _native

_native.load_torch_binding()


@register_fake("quant_ops::int4_matmul")
def _int4_matmul_fake(a, b, scale_a, scale_b):
    return a.new_empty((a.size(0), b.size(1)), dtype=torch.float16)


@register_fake("quant_ops::int4_matmul_ex")
def _int4_matmul_ex_fake(a, b, scale_a, scale_b, out_dtype, return_acc=False):
    out = a.new_empty((a.size(0), b.size(1)), dtype=out_dtype)
    acc = a.new_empty((a.size(0), b.size(1)) if return_acc else (0,), dtype=torch.int32)
    return out, acc


@register_fake("quant_ops::flatquant_dynamic_quantize")
def _flatquant_fake(input, left_trans, right_trans, clip_ratio=1.0, pack_int32=False):
    tokens = input.size(0)
    features = left_trans.size(0) * right_trans.size(0)
    if pack_int32:
        out = input.new_empty((tokens, features // 8), dtype=torch.int32)
    else:
        out = input.new_empty((tokens, features), dtype=torch.int8)
    return out, input.new_empty((tokens,), dtype=torch.float32)


@register_fake("quant_ops::flatquant_dynamic_quantize_ex")
def _flatquant_ex_fake(input, left_trans, right_trans, clip_ratio=1.0, pack_int32=False, scale_dtype=None):
    out, _ = _flatquant_fake(input, left_trans, right_trans, clip_ratio, pack_int32)
    return out, input.new_empty((input.size(0),), dtype=scale_dtype or torch.float32)


@register_fake("quant_ops::dequantize_int4")
def _dequant_fake(quantized, scales, packed_int32=False):
    feats = quantized.size(1) * (8 if packed_int32 else 1)
    return quantized.new_empty((quantized.size(0), feats), dtype=torch.float32)


@register_fake("quant_ops::w4a4_linear")
def _linear_fake(x, left_trans, right_trans, w_packed, w_scale, bias=None, clip_ratio=1.0, out_dtype=None):
    if out_dtype is None:
        out_dtype = torch.bfloat16 if x.dtype == torch.bfloat16 else torch.float16
    return x.new_empty((x.size(0), w_packed.size(0)), dtype=out_dtype)


@register_fake("quant_ops::prepare_weights")
def _prepare_fake(w_packed):
    blocks = ((w_packed.size(0) + 255) // 256) * ((w_packed.size(1) * 8 + 127) // 128)
    return w_packed.new_empty((blocks * 256 * 128,), dtype=torch.uint8)


@register_fake("quant_ops::w4a4_linear_prepared")
def _linear_prepared_fake(x, left_trans, right_trans, w_packed, w_prepared, w_scale, bias=None, clip_ratio=1.0, out_dtype=None):
    if out_dtype is None:
        out_dtype = torch.bfloat16 if x.dtype == torch.bfloat16 else torch.float16
    return x.new_empty((x.size(0), w_packed.size(0)), dtype=out_dtype)


@register_fake("quant_ops::pack_int4")
def _pack_fake(codes):
    return codes.new_empty((codes.size(0), codes.size(1) // 8), dtype=torch.int32)


@register_fake("quant_ops::unpack_int4")
def _unpack_fake(packed):
    return packed.new_empty((packed.size(0), packed.size(1) * 8), dtype=torch.int8)


@register_fake("quant_ops::quantize_weights_int4")
def _wq_fake(w):
    return (w.new_empty((w.size(0), w.size(1) // 8), dtype=torch.int32), w.new_empty((w.size(0),), dtype=torch.float32))
