"""W4A4 linear layer on top of the fused op: the caller-side object of the path.

Mirrors the parameter layout and `apply` flow of the reference's layer method
(AscendW4A4FlatQuantDynamicLinearMethod, w4a4_flatquant_dynamic.py:98-165 parameters, :168-266 apply, :268-304
load-time weight preparation): int8 weight [out, in] packed to int32 [out, in/8] at load time, float32
per-output-channel scale, left/right transforms, clip ratio; apply accepts any leading dimensions, returns the input's
dtype and adds an optional bias.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops
from .decompose import get_decompose_dim


class W4A4Linear(torch.nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, clip_ratio: float = 1.0,
                 dtype: torch.dtype = torch.bfloat16, device=None, keep_int8_weights: bool = False):
        """keep_int8_weights: also hold the weights widened to int8 in the GEMM's blocked layout (a byte tensor, about
        twice the packed size); forward then rewrites no operand per call.  The copy is made by load_quantized / load_float / prepare()."""
        super().__init__()
        self.keep_int8_weights = bool(keep_int8_weights)
        self.weight_int8 = None  # derived from weight_packed, not part of the state dict
        if in_features % 8:
            raise ValueError("in_features must be a multiple of 8 (eight int4 values per packed word)")
        self.in_features, self.out_features, self.clip_ratio = in_features, out_features, float(clip_ratio)
        m, n = get_decompose_dim(in_features)
        self.register_buffer("weight_packed", torch.zeros(out_features, in_features // 8, dtype=torch.int32, device=device))
        self.register_buffer("weight_scale", torch.ones(out_features, dtype=torch.float32, device=device))
        self.register_buffer("left_trans", torch.eye(m, dtype=dtype, device=device))
        self.register_buffer("right_trans", torch.eye(n, dtype=dtype, device=device))
        self.register_buffer("bias", torch.zeros(out_features, dtype=dtype, device=device) if bias else None)

    @torch.no_grad()
    def load_quantized(self, weight_int8: torch.Tensor, weight_scale: torch.Tensor, left_trans: torch.Tensor,
                       right_trans: torch.Tensor, bias: Optional[torch.Tensor] = None) -> "W4A4Linear":
        """Load-time preparation: int8 codes [out, in] in [-8, 7] are packed along `in`; scales become float32."""
        if weight_int8.shape != (self.out_features, self.in_features):
            raise ValueError("weight shape mismatch")
        self.weight_packed.copy_(ops.pack_int4_to_int32(weight_int8.to(self.weight_packed.device, torch.int8)))
        self.weight_scale.copy_(weight_scale.reshape(-1).to(torch.float32))
        self.left_trans.copy_(left_trans)
        self.right_trans.copy_(right_trans)
        if bias is not None and self.bias is not None:
            self.bias.copy_(bias)
        return self.prepare()

    @torch.no_grad()
    def prepare(self) -> "W4A4Linear":
        """(Re)builds the int8 copy of the weights after weight_packed changed; a no-op without keep_int8_weights."""
        self.weight_int8 = ops.prepare_weights(self.weight_packed) if self.keep_int8_weights else None
        return self

    @torch.no_grad()
    def load_float(self, weight: torch.Tensor, left_trans: torch.Tensor, right_trans: torch.Tensor,
                   bias: Optional[torch.Tensor] = None) -> "W4A4Linear":
        """Quantizes a float weight per output channel (absmax / 7) on the GPU, then loads it."""
        packed, scale = ops.quantize_weights_int4(weight.to(self.weight_packed.device))
        self.weight_packed.copy_(packed)
        self.weight_scale.copy_(scale)
        self.left_trans.copy_(left_trans)
        self.right_trans.copy_(right_trans)
        if bias is not None and self.bias is not None:
            self.bias.copy_(bias)
        return self.prepare()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if x2.dtype != self.left_trans.dtype:
            raise RuntimeError(f"input dtype {x2.dtype} does not match the transforms' dtype {self.left_trans.dtype}")
        out_dtype = x2.dtype if x2.dtype in (torch.float16, torch.bfloat16) else torch.float16
        if self.weight_int8 is not None:
            y = ops.w4a4_linear_prepared(x2, self.left_trans, self.right_trans, self.weight_packed, self.weight_int8,
                                         self.weight_scale, self.bias, self.clip_ratio, out_dtype)
        else:
            y = ops.w4a4_linear(x2, self.left_trans, self.right_trans, self.weight_packed, self.weight_scale, self.bias,
                                self.clip_ratio, out_dtype)
        return y.reshape(*lead, self.out_features)
