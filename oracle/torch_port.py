"""CPU restatement of the reference's path with torch CPU tensor ops -- TEST / BASELINE INFRASTRUCTURE.

The reference's own CPU implementation is a chain of torch tensor ops; it cannot travel with this repository, so
this module restates the same chain (same library calls in the same order, hence the same CPU cost) for two uses
only: the `--impl reference` arm / `cpu_baseline` leg of the benchmark, and a cross-check of the numpy oracle.
It is pinned by tests/test_oracle_golden.py against fixtures produced by the reference itself.

Follows (paths inside the reference project):
  quantize   src/quant_ops/ops/quantization/flatquant/ops.py:99-130
  matmul     src/quant_ops/ops/quantization/int4_matmul/ops.py:88-103
"""
from __future__ import annotations

import torch


def _pack_rows(codes: torch.Tensor) -> torch.Tensor:
    rows, feat = codes.shape
    nib = (codes + 8).to(torch.uint8).view(rows, feat // 8, 8)
    words = torch.zeros(rows, feat // 8, dtype=torch.int32, device=codes.device)
    for slot in range(8):
        words += nib[:, :, slot].to(torch.int32) << (4 * slot)
    return words


def _unpack_rows(words: torch.Tensor) -> torch.Tensor:
    rows, wcount = words.shape
    codes = torch.zeros(rows, wcount * 8, dtype=torch.int8, device=words.device)
    for slot in range(8):
        codes[:, slot::8] = (((words >> (4 * slot)) & 0xF) - 8).to(torch.int8)
    return codes


def quantize(x: torch.Tensor, left: torch.Tensor, right: torch.Tensor, clip_ratio: float = 1.0, pack_int32: bool = False):
    tokens, feat = x.shape
    z = torch.matmul(left.T, torch.matmul(x.reshape(-1, left.shape[0], right.shape[0]), right)).reshape(tokens, feat)
    hi = z.amax(1, keepdim=True)
    lo = z.amin(1, keepdim=True)
    top = torch.maximum(torch.abs(lo * clip_ratio), hi * clip_ratio)
    scale = (top / 7.0).clamp(min=1e-8).squeeze(1)
    q = torch.round(z / scale.view(-1, 1)).clamp(-8, 7)
    if pack_int32:
        return _pack_rows(q), scale
    return q.to(torch.int8), scale


def matmul(a_packed: torch.Tensor, b_packed: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor) -> torch.Tensor:
    a = _unpack_rows(a_packed)
    b = _unpack_rows(b_packed.T).T
    acc = torch.matmul(a.float(), b.float())
    return (acc * scale_a.view(-1, 1) * scale_b.view(1, -1)).half()


def linear(x, left, right, clip_ratio, w_packed, w_scale):
    a, s = quantize(x, left, right, clip_ratio, True)
    return matmul(a, w_packed.t(), s.float(), w_scale)
