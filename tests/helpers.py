"""Shared test helpers: seeded inputs, torch<->numpy conversion, thin callers of the C ABI.

The parity tests call the C ABI directly (ctypes) with torch tensors providing the device memory, compare with
the numpy oracle (oracle/w4a4_oracle.py) and with the golden fixtures made from the reference (tests/golden/).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np
import torch

from oracle import w4a4_oracle as O
from quant_ops_b200 import _native as N

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TD = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
QD = {"bf16": N.QO_BF16, "fp16": N.QO_F16, "fp32": N.QO_F32}
lib = N.lib


def golden(name: str):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def bits_to_f32(arr: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "bf16":
        return O.bf16_bits_to_f32(arr)
    if dtype == "fp16":
        return arr.view(np.float16).astype(np.float32)
    return arr.astype(np.float32)


def bits_to_torch(arr: np.ndarray, dtype: str) -> torch.Tensor:
    if dtype == "fp32":
        return torch.from_numpy(arr.copy())
    return torch.from_numpy(arr.view(np.int16).copy()).view(TD[dtype])


def t2f(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def make_inputs(tokens, feat, dtype, seed, outliers=True, ortho=True, mn=None):
    """Seeded activations [tokens, feat] (optionally 1% of the channels x50) and random-orthogonal L, R."""
    g = torch.Generator().manual_seed(seed)
    m, n = mn if mn is not None else O.get_decompose_dim(feat)
    x = torch.randn(tokens, feat, generator=g)
    if outliers and feat >= 100:
        idx = torch.randperm(feat, generator=g)[: feat // 100]
        x[:, idx] *= 50
    if ortho:
        left = torch.linalg.qr(torch.randn(m, m, dtype=torch.float64, generator=g)).Q
        right = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, generator=g)).Q
    else:
        left = torch.randn(m, m, generator=g)
        right = torch.randn(n, n, generator=g)
    # QR hands back column-major factors: the C ABI wants plain row-major buffers
    return x.to(TD[dtype]).contiguous(), left.to(TD[dtype]).contiguous(), right.to(TD[dtype]).contiguous()


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None and t.numel() > 0 else C.c_void_p(0)


def stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def abi_quantize(x, left, right, clip, pack, dtype, scale_dtype="fp32", policy=0, ldx=None):
    """qo_flatquant_quantize on CUDA tensors; returns (codes, scales) tensors."""
    tokens, feat = x.shape
    m, n = left.shape[0], right.shape[0]
    codes = torch.empty((tokens, feat // 8 if pack else feat), dtype=torch.int32 if pack else torch.int8, device=x.device)
    scales = torch.empty((tokens,), dtype=TD[scale_dtype], device=x.device)
    N.check(lib.qo_set_kernel_policy(policy))
    try:
        N.check(lib.qo_flatquant_quantize(ptr(x), ldx if ldx is not None else (x.stride(0) if tokens > 1 else feat),
                                          ptr(left), ptr(right), ptr(codes), ptr(scales), tokens, m, n, float(clip),
                                          QD[dtype], int(pack), QD[scale_dtype], stream_ptr()))
    finally:
        lib.qo_set_kernel_policy(0)
    torch.cuda.synchronize()
    return codes, scales


def abi_int4_matmul(a, b, sa, sb, out_dtype="fp16", want_acc=False, policy=0, use_workspace=True):
    t, kp = a.shape
    n = b.shape[1]
    out = torch.empty((t, n), dtype=TD[out_dtype], device=a.device)
    acc = torch.empty((t, n), dtype=torch.int32, device=a.device) if want_acc else None
    need = lib.qo_int4_matmul_workspace_bytes(t, kp * 8, n)
    ws = torch.empty((need,), dtype=torch.uint8, device=a.device) if (use_workspace and need) else None
    N.check(lib.qo_set_kernel_policy(policy))
    try:
        N.check(lib.qo_int4_matmul(ptr(a), a.stride(0) if t > 1 else kp, ptr(b), b.stride(0), b.stride(1), ptr(sa), ptr(sb),
                                   ptr(out), QD[out_dtype], t, kp * 8, n, ptr(acc), ptr(ws), need if ws is not None else 0,
                                   stream_ptr()))
    finally:
        lib.qo_set_kernel_policy(0)
    torch.cuda.synchronize()
    return (out, acc) if want_acc else out


def compare_codes(got: np.ndarray, ref: np.ndarray, max_frac=1e-3):
    """Codes must be identical except +-1 on at most max_frac of the elements (never more than 1 apart)."""
    d = np.abs(got.astype(np.int32) - ref.astype(np.int32))
    assert d.max(initial=0) <= 1, f"code differs by {d.max()}"
    frac = float((d != 0).mean()) if d.size else 0.0
    assert frac <= max_frac, f"{frac:.5%} of the codes differ (limit {max_frac:.3%})"
    return frac


def compare_scales(got: np.ndarray, ref: np.ndarray, rel=1e-3):
    denom = np.maximum(np.abs(ref), 1e-30)
    err = np.abs(got - ref) / denom
    assert err.max(initial=0) <= rel, f"scale relative error {err.max():.3e} > {rel}"
