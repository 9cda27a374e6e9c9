"""Times the reference project's own CUDA extensions (built unmodified by baseline/build_ref_cuda.py) on this GPU.

    python baseline/time_ref_cuda.py [--steps K]

Prints one JSON line: the reference's quantizer op (cuBLAS batched matmul x2 + its scale/quantize kernel) on
x [8192, 4096] bf16 with packing, and its dp4a GEMM on 4096 x 4096 x n_out packed int4, both through the dispatcher ops
the extensions register (quant_ops::flatquant_dynamic_quantize, quant_ops::int4_matmul).  It is the kernel-to-beat
figure on the same box.  Runs in a process of its own: the product's binding registers the same dispatcher
namespace, so the two cannot be loaded together.  Prints {"unavailable": reason} when the objects are missing.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--gemm-steps", type=int, default=5)
    args = ap.parse_args()
    libs = [os.path.join(HERE, "_ref", n) for n in ("ref_cuda_quant_ops.so", "ref_cuda_int4_matmul_ops.so")]
    if not all(os.path.exists(p) for p in libs):
        print(json.dumps({"unavailable": "baseline/_ref/*.so not built (python baseline/build_ref_cuda.py <reference checkout>)"}))
        return
    import torch

    if "quant_ops_b200" in sys.modules:
        raise SystemExit("time_ref_cuda.py must not share a process with quant_ops_b200 (same dispatcher namespace)")
    if not torch.cuda.is_available():
        print(json.dumps({"unavailable": "no CUDA device"}))
        return
    try:
        for p in libs:
            torch.ops.load_library(p)
    except Exception as exc:
        print(json.dumps({"unavailable": f"load failed: {str(exc)[:300]}"}))
        return
    dev = "cuda:0"
    g = torch.Generator().manual_seed(20242)
    tokens, feat, m, n = 8192, 4096, 64, 64
    x = torch.randn(tokens, feat, generator=g)
    x[:, torch.randperm(feat, generator=g)[: feat // 100]] *= 50
    left = torch.linalg.qr(torch.randn(m, m, dtype=torch.float64, generator=g)).Q.bfloat16().contiguous().to(dev)
    right = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, generator=g)).Q.bfloat16().contiguous().to(dev)
    xs = [torch.roll(x, i, 0).bfloat16().to(dev) for i in range(4)]  # 4 x 67 MB of inputs > L2
    out = {"impl": "reference CUDA extensions, unmodified, sm_100a", "gpu": torch.cuda.get_device_name(0)}

    def timed(fn, steps):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    try:
        q = torch.ops.quant_ops.flatquant_dynamic_quantize
        ms = timed(lambda i: q(xs[i % 4], left, right, 0.9, True), args.steps)
        algo = tokens * (feat * 2 + feat // 2 + 4) + (m * m + n * n) * 2
        out["quantize"] = {"workload": "x [8192, 4096] bf16, pack_int32", "ms_per_step": ms, "value": algo / (ms / 1e3) / 1e9, "unit": "GB/s",
                           "steps": args.steps}
        codes, scales = q(xs[0], left, right, 0.9, True)
    except Exception as exc:
        out["quantize"] = {"unavailable": str(exc)[:300]}
        codes = torch.randint(-2**31, 2**31 - 1, (tokens, feat // 8), dtype=torch.int32, device=dev)
        scales = torch.rand(tokens, device=dev)
    out["gemm"] = []
    for n_out in (4096, 11008, 14336):
        try:
            a = codes[:4096].contiguous()
            sa = scales[:4096].float().contiguous()
            b = torch.randint(-2**31, 2**31 - 1, (feat // 8, n_out), generator=g, dtype=torch.int32).to(dev)  # reference layout [K/8, N]
            sb = (torch.rand(n_out, generator=g) * 0.01 + 0.001).to(dev)
            mm = torch.ops.quant_ops.int4_matmul
            ms = timed(lambda i: mm(a, b, sa, sb), args.gemm_steps)
            ops = 2.0 * 4096 * feat * n_out
            out["gemm"].append({"workload": f"4096 x 4096 x {n_out} packed int4, fp16 out", "ms_per_step": ms, "value": ops / (ms / 1e3) / 1e12,
                                "unit": "TOP/s", "steps": args.gemm_steps})
        except Exception as exc:
            out["gemm"].append({"workload": f"n_out={n_out}", "unavailable": str(exc)[:300]})
    print(json.dumps(out))


if __name__ == "__main__":
    main()
