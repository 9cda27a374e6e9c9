"""CPU oracle for the W4A4 hot path -- TEST INFRASTRUCTURE, not product code.

This file restates, in plain numpy, the arithmetic of the reference's PyTorch
implementation of the path (libarry/quant_ops).  It exists so that the CUDA
kernels can be checked against an independent statement of the same algorithm.
Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import it; the shipped package never does.

Parity pin: every function here is checked (tests/test_oracle_golden.py)
against fixtures under tests/golden/ that were produced by running the
reference's own Python functions on CPU tensors (tests/golden/make_golden.py).

Reference functions restated (paths inside the reference project):
  get_decompose_dim      src/quant_ops/utils/decompose.py:11-38
  flatquant_quantize     src/quant_ops/ops/quantization/flatquant/ops.py:78-130
  dequantize_int4        src/quant_ops/ops/quantization/flatquant/ops.py:156-178
  pack_int4_to_int32     src/quant_ops/ops/quantization/int4_matmul/ops.py:23-45
  unpack_int32_to_int4   src/quant_ops/ops/quantization/int4_matmul/ops.py:48-66
  int4_matmul            src/quant_ops/ops/quantization/int4_matmul/ops.py:69-103

Number formats.  Activations are carried as float32 arrays whose values are
exactly representable in the working dtype ("bf16", "fp16" or "fp32").  The
reference evaluates every step in the working dtype, which for the 16-bit
types means: compute in float32, round the result to the 16-bit type.  The
rounding points reproduced here are: each of the two transform products, the
two clip products, the division by 7, the quotient x/scale.
"""
from __future__ import annotations

import math

import numpy as np

DTYPES = ("bf16", "fp16", "fp32")


# --------------------------------------------------------------------------- rounding helpers
def round_to(a: np.ndarray, dtype: str) -> np.ndarray:
    """Round float32 values to `dtype` (nearest-even) and return them as float32."""
    a = np.asarray(a, dtype=np.float32)
    if dtype == "fp32":
        return a
    if dtype == "fp16":
        with np.errstate(over="ignore"):
            return a.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        u = np.ascontiguousarray(a).view(np.uint32)
        bias = np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
        r = ((u + bias) & np.uint32(0xFFFF0000)).view(np.float32)
        nan = np.isnan(a)
        if nan.any():
            r = np.where(nan, a, r)
        return r
    raise ValueError(f"unknown dtype {dtype!r}")


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    return (round_to(a, "bf16").view(np.uint32) >> np.uint32(16)).astype(np.uint16)


# --------------------------------------------------------------------------- get_decompose_dim
def get_decompose_dim(n: int) -> tuple[int, int]:
    """Smallest a >= ceil(sqrt(n)) with a*a - n a perfect square b*b; returns (a-b, a+b).

    The reference loops forever when no such a exists (n = 2 mod 4); this
    restatement raises instead, which is also what the product does.
    """
    n = int(n)
    if n <= 0:
        raise ValueError("n must be positive")
    if n % 4 == 2:
        raise ValueError(f"{n} has no factorisation (a-b)(a+b): n = 2 (mod 4)")
    a = math.isqrt(n)
    if a * a < n:
        a += 1
    while True:
        d = a * a - n
        b = math.isqrt(d)
        if b * b == d:
            return a - b, a + b
        a += 1


# --------------------------------------------------------------------------- packing
def pack_int4_to_int32(codes: np.ndarray) -> np.ndarray:
    """codes int8 [rows, F] in [-8, 7]  ->  int32 [rows, F/8]; nibble i of a word is code[8p+i] + 8."""
    codes = np.asarray(codes)
    rows, feat = codes.shape
    if feat % 8:
        raise ValueError("feature count must be a multiple of 8")
    u = (codes.astype(np.int16) + 8).astype(np.uint32).reshape(rows, feat // 8, 8)
    w = np.zeros((rows, feat // 8), dtype=np.uint32)
    for i in range(8):
        w |= u[:, :, i] << np.uint32(4 * i)
    return w.view(np.int32)


def unpack_int32_to_int4(words: np.ndarray) -> np.ndarray:
    """Inverse of pack_int4_to_int32: int32 [rows, P] -> int8 [rows, 8P]."""
    w = np.ascontiguousarray(words).astype(np.int32).view(np.uint32)
    rows, p = w.shape
    out = np.empty((rows, p, 8), dtype=np.int8)
    for i in range(8):
        out[:, :, i] = (((w >> np.uint32(4 * i)) & np.uint32(0xF)).astype(np.int16) - 8).astype(np.int8)
    return out.reshape(rows, p * 8)


# --------------------------------------------------------------------------- FlatQuant quantizer
def kronecker_transform(x: np.ndarray, left: np.ndarray, right: np.ndarray, dtype: str) -> np.ndarray:
    """Per token: view the row as an M x N matrix X and return L^T . (X . R), each product rounded to dtype."""
    m, n = left.shape[0], right.shape[0]
    t = x.shape[0]
    x3 = np.asarray(x, dtype=np.float32).reshape(t, m, n)
    y = round_to(np.matmul(x3, np.asarray(right, dtype=np.float32)), dtype)
    z = round_to(np.matmul(np.asarray(left, dtype=np.float32).T, y), dtype)
    return z.reshape(t, m * n)


def token_scales(z: np.ndarray, clip_ratio: float, dtype: str) -> np.ndarray:
    """scale = max(|min*c|, max*c) / 7 clamped below at 1e-8, every step rounded to dtype."""
    c = np.float32(clip_ratio)
    zmax = z.max(axis=1)
    zmin = z.min(axis=1)
    hi = round_to(zmax * c, dtype)
    lo = np.abs(round_to(zmin * c, dtype))
    top = np.maximum(lo, hi)
    s = round_to(top / np.float32(7.0), dtype)
    floor = round_to(np.float32(1e-8), dtype)  # 0 in fp16: the clamp does nothing there
    return np.maximum(s, floor).astype(np.float32)


def quantize_rows(z: np.ndarray, scales: np.ndarray, dtype: str) -> np.ndarray:
    """codes = clamp(round_half_even(round_to(z / scale)), -8, 7) as int8.

    A zero scale (possible only in fp16, all-zero row) gives 0/0 in the
    reference; the agreed behaviour is code 0, which is what comes out here
    because the quotient is replaced by 0 wherever it is not finite and z is 0.
    """
    with np.errstate(divide="ignore", invalid="ignore"):
        q = round_to(z / scales[:, None].astype(np.float32), dtype)
    q = np.where(np.isnan(q), np.float32(0), q)
    r = np.clip(np.rint(q), -8, 7)
    return r.astype(np.int8)


def flatquant_quantize(x, left, right, clip_ratio=1.0, pack_int32=False, dtype="bf16"):
    """Full quantizer. Returns (codes int8 [T,F] or int32 [T,F/8], scales float32 [T] holding dtype-rounded values)."""
    if dtype not in DTYPES:
        raise ValueError(dtype)
    x = np.asarray(x, dtype=np.float32)
    if x.ndim != 2:
        raise ValueError("input must be [tokens, features]")
    m, n = left.shape[0], right.shape[0]
    if x.shape[1] != m * n:
        raise ValueError("feature count must equal M*N")
    if x.shape[0] == 0:
        width = x.shape[1] // 8 if pack_int32 else x.shape[1]
        return (np.zeros((0, width), np.int32 if pack_int32 else np.int8), np.zeros((0,), np.float32))
    z = kronecker_transform(x, left, right, dtype)
    s = token_scales(z, clip_ratio, dtype)
    codes = quantize_rows(z, s, dtype)
    if pack_int32:
        return pack_int4_to_int32(codes), s
    return codes, s


# --------------------------------------------------------------------------- dequantize
def dequantize_int4(quantized: np.ndarray, scales: np.ndarray, packed_int32: bool = False) -> np.ndarray:
    """float32 [T,F] = code * scale[token]."""
    codes = unpack_int32_to_int4(quantized) if packed_int32 else np.asarray(quantized, dtype=np.int8)
    return codes.astype(np.float32) * np.asarray(scales, dtype=np.float32).reshape(-1, 1)


# --------------------------------------------------------------------------- int4 GEMM
def int4_accumulators(a_packed: np.ndarray, b_packed: np.ndarray) -> np.ndarray:
    """Exact int32 accumulators of A[T,K] . B[K,N] for packed operands.

    a_packed is [T, K/8]; b_packed is [K/8, N] with the nibbles of a word
    running along K.  The products are summed in float32, which is exact
    because |acc| <= 64*K < 2**24 for every K the path uses (K <= 262143).
    """
    a = unpack_int32_to_int4(a_packed).astype(np.float32)  # [T, K]
    b = unpack_int32_to_int4(np.ascontiguousarray(np.asarray(b_packed).T)).T.astype(np.float32)  # [K, N]
    if a.shape[1] * 64 >= 2 ** 24:
        raise ValueError("K too large for exact float32 accumulation")
    acc = a @ b
    return acc.astype(np.int32)


def int4_matmul(a_packed, b_packed, scale_a, scale_b, out_dtype="fp16") -> np.ndarray:
    """out = round_to((acc * scale_a[row]) * scale_b[col]); returned as float32 holding out_dtype values."""
    acc = int4_accumulators(a_packed, b_packed).astype(np.float32)
    sa = np.asarray(scale_a, dtype=np.float32).reshape(-1, 1)
    sb = np.asarray(scale_b, dtype=np.float32).reshape(1, -1)
    return round_to((acc * sa) * sb, out_dtype)


# --------------------------------------------------------------------------- fused layer
def w4a4_linear(x, left, right, clip_ratio, w_packed_nk, w_scale, dtype="bf16", out_dtype="fp16"):
    """Quantize activations, multiply by packed weights [Nout, K/8] (passed transposed to the GEMM)."""
    a, s = flatquant_quantize(x, left, right, clip_ratio, True, dtype)
    return int4_matmul(a, np.asarray(w_packed_nk).T, s, w_scale, out_dtype)


# --------------------------------------------------------------------------- harness-side weight quantizer
def quantize_weights(w: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Per-output-channel symmetric int4 (absmax/7).  Not part of the reference: input generation only."""
    w = np.asarray(w, dtype=np.float32)
    s = np.maximum(np.abs(w).max(axis=1) / np.float32(7.0), np.float32(1e-8)).astype(np.float32)
    q = np.clip(np.rint(w / s[:, None]), -8, 7).astype(np.int8)
    return q, s


# --------------------------------------------------------------------------- float simulation of the layer
def fake_quant_linear(x, left, right, clip_ratio, w_int8, w_scale, dtype="bf16", bias=None) -> np.ndarray:
    """Float simulation of the W4A4 layer: a second, independent statement of its intended numerics.

    Restates AscendW4A4FlatQuantDynamicFakeLinearMethod.apply (w4a4_flatquant_dynamic.py:440-507) with its own
    scale rule (get_scale_zero, :401-423): the row extremes are first widened to include 0 (xmax >= 0, xmin <= 0),
    multiplied by clip_ratio, scale = max(|xmin|, xmax) / 7 clamped below at 1e-8; activations are quantized and
    de-quantized in the activation dtype, the int8 weights are de-quantized with their per-channel scale and cast
    to the activation dtype, and the product is an ordinary linear layer in that dtype.  It differs from the
    integer path by the dtype roundings of the de-quantized operands, so it is compared with a tolerance.
    Returns float32 holding `dtype` values, shape [tokens, n_out].
    """
    z = kronecker_transform(x, left, right, dtype)
    c = np.float32(clip_ratio)
    zmax = np.maximum(z.max(axis=1, keepdims=True), np.float32(0))
    zmin = np.minimum(z.min(axis=1, keepdims=True), np.float32(0))
    zmax = round_to(zmax * c, dtype)
    zmin = round_to(zmin * c, dtype)
    top = np.maximum(np.abs(zmin), zmax)
    scale = np.maximum(round_to(top / np.float32(7.0), dtype), round_to(np.float32(1e-8), dtype)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = round_to(z / scale, dtype)
    q = np.clip(np.rint(np.where(np.isnan(q), np.float32(0), q)), -8, 7).astype(np.float32)
    x_deq = round_to(q * scale, dtype)
    w_deq = round_to(np.asarray(w_int8, dtype=np.float32) * np.asarray(w_scale, dtype=np.float32).reshape(-1, 1), dtype)
    out = round_to(x_deq @ w_deq.T, dtype)
    if bias is not None:
        out = round_to(out + np.asarray(bias, dtype=np.float32).reshape(1, -1), dtype)
    return out
