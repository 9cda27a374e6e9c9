"""Regenerate the golden fixtures in this directory by running the reference's own PyTorch functions.

Usage:  python tests/golden/make_golden.py /path/to/reference_checkout

The reference package cannot be imported as a whole (its loader insists on a
prebuilt extension for another Python version), so the two `ops.py` files and
`utils/decompose.py` are loaded on their own with their `.kernels` sub-module
stubbed out.  Everything below runs on CPU tensors; the outputs are what the
reference computes, stored next to the inputs that produced them.

Fixture format (.npz, one file per case): 16-bit float tensors are stored as
their raw uint16 bit patterns (`*_bits`), everything else in its own dtype.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
TD = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def load_reference(root: str):
    src = os.path.join(root, "src", "quant_ops")
    pk = types.ModuleType("refq")
    pk.__path__ = []
    sys.modules["refq"] = pk
    for sub, attr in (("fq", "cuda_quant_ops"), ("im", "cuda_int4_matmul_ops")):
        p = types.ModuleType(f"refq.{sub}")
        p.__path__ = []
        sys.modules[f"refq.{sub}"] = p
        k = types.ModuleType(f"refq.{sub}.kernels")
        setattr(k, attr, None)
        k.CUDA_KERNELS_AVAILABLE = False
        sys.modules[f"refq.{sub}.kernels"] = k

    def imp(name, path):
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod

    fq = imp("refq.fq.ops", os.path.join(src, "ops", "quantization", "flatquant", "ops.py"))
    im = imp("refq.im.ops", os.path.join(src, "ops", "quantization", "int4_matmul", "ops.py"))
    dc = imp("refq_decompose", os.path.join(src, "utils", "decompose.py"))
    return fq, im, dc


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def make_inputs(dc, tokens, feat, dtype, seed, outliers, ortho):
    g = torch.Generator().manual_seed(seed)
    m, n = dc.get_decompose_dim(feat)
    x = torch.randn(tokens, feat, generator=g)
    if outliers:
        idx = torch.randperm(feat, generator=g)[: feat // 100]
        x[:, idx] *= 50
    if ortho:
        left = torch.linalg.qr(torch.randn(m, m, dtype=torch.float64, generator=g)).Q
        right = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, generator=g)).Q
    else:
        left = torch.randn(m, m, generator=g)
        right = torch.randn(n, n, generator=g)
    return x.to(TD[dtype]), left.to(TD[dtype]), right.to(TD[dtype])


QUANT_CASES = [
    # name, tokens, features, dtype, clip, pack, outliers, orthogonal L/R, seed
    ("quant_fp16_4096_int8", 16, 4096, "fp16", 1.0, False, False, True, 20241),
    ("quant_bf16_4096_packed", 16, 4096, "bf16", 0.9, True, True, True, 20242),
    ("quant_bf16_14336_packed", 6, 14336, "bf16", 0.9, True, True, True, 20244),
    ("quant_bf16_11008_packed", 4, 11008, "bf16", 0.9, True, True, True, 20246),
    ("quant_fp32_2048_int8", 8, 2048, "fp32", 1.0, False, False, True, 20247),
    ("quant_fp16_4096_randnLR", 8, 4096, "fp16", 1.0, False, False, False, 42),
    ("quant_fp16_256_packed", 32, 256, "fp16", 0.6, True, False, True, 20248),
    ("quant_bf16_1024_int8", 9, 1024, "bf16", 1.0, False, True, True, 20249),
]


def main(root: str) -> None:
    fq, im, dc = load_reference(root)
    torch.set_num_threads(1)

    dims = [16, 64, 100, 256, 1024, 2048, 4096, 5120, 8192, 11008, 13824, 14336, 28672, 15, 21, 9991]
    np.savez(os.path.join(HERE, "decompose.npz"), n=np.array(dims),
             mn=np.array([dc.get_decompose_dim(d) for d in dims]))

    for name, tokens, feat, dtype, clip, pack, outl, ortho, seed in QUANT_CASES:
        x, left, right = make_inputs(dc, tokens, feat, dtype, seed, outl, ortho)
        codes, scales = fq.flatquant_pytorch(x, left, right, clip, pack)
        deq = fq.dequantize_int4(codes, scales, pack)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            dtype=dtype, clip=np.float64(clip), pack=np.bool_(pack),
            x=bits(x), left=bits(left), right=bits(right),
            codes=codes.numpy(), scales=scales.float().numpy(),
            dequant_head=deq.numpy()[:2].copy(),  # first two rows keep the file small
        )

    # Known-answer rows with identity transforms: rounding ties, clipping, packing layout, zero row.
    for dtype in ("bf16", "fp16", "fp32"):
        m = n = 4
        x = torch.zeros(5, 16)
        x[0, :8] = torch.tensor([7, 3.5, 2.5, 1.5, 0.5, -0.5, -2.5, -3.5])
        x[1, :4] = torch.tensor([-10.0, 10.0, 9.0, -9.0])
        x[2, :2] = torch.tensor([-10.0, 2.0])
        x[3, 7] = 7.0
        eye = torch.eye(4)
        out = {}
        for clip, pack in ((1.0, False), (1.0, True), (0.5, False), (0.5, True)):
            c, s = fq.flatquant_pytorch(x.to(TD[dtype]), eye.to(TD[dtype]), eye.to(TD[dtype]), clip, pack)
            key = f"c{int(clip * 10)}_{'p' if pack else 'i'}"
            # a zero row divides 0 by 0 in fp16 (the clamp at 1e-8 rounds to 0 there); the cast of NaN to an
            # integer is not defined, so row 4's codes are not part of the fixture for fp16.
            out["codes_" + key] = c.numpy()
            out["scales_" + key] = s.float().numpy()
        np.savez(os.path.join(HERE, f"kat_identity_{dtype}.npz"), x=x.numpy(), **out)

    # int4 GEMM in the layout of the reference's own benchmark script (B packed along K, N contiguous).
    for name, t, k, nout, seed in (("gemm_64x512x96", 64, 512, 96, 7), ("gemm_33x256x40", 33, 256, 40, 8)):
        g = torch.Generator().manual_seed(seed)
        a = torch.randint(-8, 8, (t, k), generator=g, dtype=torch.int8)
        b = torch.randint(-8, 8, (k, nout), generator=g, dtype=torch.int8)
        ap = im.pack_int4_to_int32(a)
        bp = im.pack_int4_to_int32(b.T.contiguous()).T.contiguous()
        sa = torch.rand(t, generator=g) * 0.1 + 0.01
        sb = torch.rand(nout, generator=g) * 0.1 + 0.01
        out = im.int4_matmul_pytorch(ap, bp, sa, sb)
        acc = a.to(torch.int32) @ b.to(torch.int32)
        assert torch.equal(im.unpack_int32_to_int4(ap), a)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), a_codes=a.numpy(), b_codes=b.numpy(),
                            a_packed=ap.numpy(), b_packed=bp.numpy(), scale_a=sa.numpy(), scale_b=sb.numpy(),
                            out_bits=bits(out), acc=acc.numpy())

    # fused layer = the composition a user of the reference writes by hand
    x, left, right = make_inputs(dc, 12, 1024, "bf16", 20250, True, True)
    g = torch.Generator().manual_seed(99)
    w = torch.randn(48, 1024, generator=g) * 0.02
    sw = (w.abs().amax(1) / 7.0).clamp(min=1e-8)
    wq = torch.round(w / sw[:, None]).clamp(-8, 7).to(torch.int8)
    wp = im.pack_int4_to_int32(wq)
    aq, sa = fq.flatquant_pytorch(x, left, right, 0.9, True)
    out = im.int4_matmul_pytorch(aq, wp.t(), sa.float(), sw)
    np.savez_compressed(os.path.join(HERE, "linear_bf16_1024x48.npz"), x=bits(x), left=bits(left), right=bits(right),
                        clip=np.float64(0.9), w_packed=wp.numpy(), w_scale=sw.numpy(), a_packed=aq.numpy(),
                        a_scale=sa.float().numpy(), out_bits=bits(out))
    print("fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference repository>")
    main(sys.argv[1])
