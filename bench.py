#!/usr/bin/env python
"""Benchmark of the W4A4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (N = 1): the FlatQuant quantizer at activation scale -- x [8192, 4096] bf16 ~ N(0,1) with 1 % of
the channels x50, L and R 64x64 random orthogonal, clip 0.9, packed int32 output plus per-token scales.  One step
= one pass of the quantizer over one batch.  Batches rotate through several buffer sets that together exceed the
L2 cache, so every step reads its input from HBM.  `value` is algorithmic GB/s with inputs resident in HBM;
`e2e` is the same metric through the host-buffer entry point (pinned host memory in, pinned host memory out).
With N > 1 every rank runs the same workload on its own GPU (rows are independent, no collective): weak scaling.

`--impl reference` times the reference's CPU implementation of the same path (its torch CPU op chain, restated in
oracle/torch_port.py) on the host cores, on a bounded sample of the workload.

`--workload` selects one of the other measured cases of the path (single GPU, one JSON line each, same keys where
they apply): `quantize_wide` (x [4096, 14336] bf16, 112 x 128 factors), `gemm` (packed int4 4096 x 4096 x 4096),
`linear` (fused quantize + GEMM, 14336 -> 4096, `--tokens` rows; weights rotate over buffers larger than L2),
`stack` (the seven W4A4 projections of a Llama-3-8B layer over 65,536 tokens, rows split over the ranks, weights kept
as int8 by `qo_prepare_weights`; tokens/s; the one secondary workload that also runs under torchrun).
The default, `quantize`, is the headline above.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOKENS, FEAT, M, N_ = 8192, 4096, 64, 64
CLIP = 0.9
SEED = 20242
ALGO_BYTES_PER_STEP = TOKENS * (FEAT * 2 + FEAT // 2 + 4) + (M * M + N_ * N_) * 2  # 83,935,232
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one quantizer launch on this workload (ncu, see profiles/)
NCU_TRAFFIC_BYTES_PER_LAUNCH = 69_641_472  # 67.16 MB read + 2.48 MB written


def make_inputs(tokens, seed):
    import torch

    g = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, FEAT, generator=g)
    idx = torch.randperm(FEAT, generator=g)[: FEAT // 100]
    x[:, idx] *= 50
    left = torch.linalg.qr(torch.randn(M, M, dtype=torch.float64, generator=g)).Q
    right = torch.linalg.qr(torch.randn(N_, N_, dtype=torch.float64, generator=g)).Q
    return x.bfloat16().contiguous(), left.bfloat16().contiguous(), right.bfloat16().contiguous()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy bandwidth)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (earlier measurement on this pool)"


class ClockSampler(threading.Thread):
    """Polls NVML for SM clock and throttle reasons while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            pass

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.0002)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def cpu_port_run(steps: int, warmup: int, sample_tokens: int):
    """Times the torch CPU restatement of the reference on `sample_tokens` rows of the workload per step."""
    import torch

    from oracle import torch_port

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x, left, right = make_inputs(sample_tokens, SEED)
    for _ in range(max(1, warmup)):
        torch_port.quantize(x, left, right, CLIP, True)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        torch_port.quantize(x, left, right, CLIP, True)
        times.append(time.perf_counter() - t0)
    total = sum(times)
    bytes_per_step = sample_tokens * (FEAT * 2 + FEAT // 2 + 4) + (M * M + N_ * N_) * 2
    return bytes_per_step * steps / total / 1e9, total / steps * 1e3, cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = 2048
    gbs, ms, cores = cpu_port_run(args.steps, args.warmup, sample)
    sample_txt = f"{sample} of the {TOKENS} tokens per step (same seed, same distribution); torch CPU ops, {cores} threads"
    print(json.dumps({
        "impl": "reference", "metric": "flatquant_quantize_GBps", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "flatquant_quantize x[8192,4096] bf16, 1% outlier channels x50, L/R 64x64 orthogonal, clip 0.9, pack_int32",
                   "sample": sample_txt},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample_txt},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ours(args):
    import ctypes as C

    import torch
    import torch.distributed as dist

    from quant_ops_b200 import _native as nat

    lib = nat.lib
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    x, left, right = make_inputs(TOKENS, SEED + rank)
    nsets = 4  # 4 x 84 MB of inputs+outputs > 126 MB of L2
    xs = [x.to(dev) if i == 0 else torch.roll(x, i, 0).to(dev) for i in range(nsets)]
    ld, rd = left.to(dev), right.to(dev)
    codes = [torch.empty(TOKENS, FEAT // 8, dtype=torch.int32, device=dev) for _ in range(nsets)]
    scales = [torch.empty(TOKENS, dtype=torch.float32, device=dev) for _ in range(nsets)]
    stream = torch.cuda.current_stream()
    sp = C.c_void_p(stream.cuda_stream)
    vp = lambda t: C.c_void_p(t.data_ptr())

    def step(i):
        s = i % nsets
        nat.check(lib.qo_flatquant_quantize(vp(xs[s]), FEAT, vp(ld), vp(rd), vp(codes[s]), vp(scales[s]), TOKENS, M, N_,
                                            CLIP, nat.QO_BF16, 1, nat.QO_F32, sp))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(3, args.warmup)):
        step(i)
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    launches0 = lib.qo_kernel_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for i in range(args.steps):
        step(i)
    ev1.record(stream)
    barrier()
    launches = lib.qo_kernel_launch_count() - launches0
    clocks = sampler.stop()
    ms_total = ev0.elapsed_time(ev1)
    path = lib.qo_last_quantizer_path()

    # end to end through the host-buffer entry point: pinned host input, pinned host outputs, copies inside the timing
    xh = x.pin_memory()
    ch = torch.empty(TOKENS, FEAT // 8, dtype=torch.int32).pin_memory()
    sh = torch.empty(TOKENS, dtype=torch.float32).pin_memory()
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_step():
        nat.check(lib.qo_flatquant_quantize_host(vp(xh), vp(left), vp(right), vp(ch), vp(sh), TOKENS, M, N_, CLIP,
                                                 nat.QO_BF16, 1, nat.QO_F32))

    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0

    tmax = torch.tensor([ms_total, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms = float(tmax[0]), float(tmax[1])

    # a few rows against the oracle, so a fast-but-wrong run cannot print a number
    from oracle import w4a4_oracle as O

    rows = [0, 1, 4097, 8191]
    rc, rs = O.flatquant_quantize(xs[0][rows].float().cpu().numpy(), left.float().numpy(), right.float().numpy(), CLIP, True, "bf16")
    got = O.unpack_int32_to_int4(codes[0][rows].cpu().numpy())
    diff = abs(got.astype(int) - O.unpack_int32_to_int4(rc).astype(int))
    parity_ok = bool(diff.max() <= 1 and (diff != 0).mean() <= 1e-3 and
                     abs(scales[0][rows].cpu().numpy() - rs).max() <= 1e-3 * abs(rs).max())

    if rank == 0:
        peak, peak_src = measured_peak()
        value = ALGO_BYTES_PER_STEP * args.steps * world / (ms_total / 1e3) / 1e9
        per_gpu = value / world
        out = {
            "metric": "flatquant_quantize_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "flatquant_quantize x[8192,4096] bf16, 1% outlier channels x50, L/R 64x64 orthogonal, clip 0.9, pack_int32",
                       "tokens_per_gpu": TOKENS, "l2": f"inputs rotate over {nsets} buffer sets (336 MB) > L2, each step reads HBM",
                       "kernel": {1: "generic SIMT", 2: "tcgen05"}.get(path, "?"), "parity_vs_oracle_sample": parity_ok},
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": ALGO_BYTES_PER_STEP},
            "e2e": {"value": ALGO_BYTES_PER_STEP * e2e_steps * world / (e2e_ms / 1e3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": TOKENS * FEAT * 2 + (M * M + N_ * N_) * 2, "d2h_bytes_per_step": TOKENS * (FEAT // 2 + 4),
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": int(launches), "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            gbs, ms, cores = cpu_port_run(5, 1, 2048)
            out["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                                   "sample": f"2048 of the {TOKENS} tokens per step, 5 steps; torch CPU ops, {cores} threads"}
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def measured_tensor_peak():
    """Dense int8 peak taken as twice the measured bf16 GEMM burst figure (int8 runs at twice the bf16 rate)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            return 2.0 * float(json.load(fh)["bf16_tflops"]), "2 x measured bf16 burst (MEASURED_PEAKS.json)"
    except Exception:
        return 2.0 * 1590.0, "2 x fallback bf16 burst (earlier measurement on this pool)"


def run_other(args):
    """Secondary workloads: device-resident inputs, CUDA events around `steps` calls through the C ABI."""
    import ctypes as C

    import torch

    from quant_ops_b200 import _native as nat

    lib = nat.lib
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and args.workload != "stack":
        raise SystemExit("bench.py: only the default workload and `stack` run on several GPUs")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    stream = torch.cuda.current_stream()
    sp = C.c_void_p(stream.cuda_stream)
    vp = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
    g = torch.Generator(device="cpu").manual_seed(SEED)
    hbm_peak, hbm_src = measured_peak()
    tc_peak, tc_src = measured_tensor_peak()

    if args.workload == "stack":
        total_tokens = 65536
        tloc = total_tokens // world
        chunk = min(tloc, 8192)
        shapes = [("q", 4096, 4096), ("k", 4096, 1024), ("v", 4096, 1024), ("o", 4096, 4096), ("gate", 4096, 14336),
                  ("up", 4096, 14336), ("down", 14336, 4096)]
        g.manual_seed(SEED + rank)
        gd = torch.Generator(device=dev).manual_seed(SEED + rank)  # activations are drawn on the device (1.2 G values)
        xin = {k: torch.randn(tloc, k, generator=gd, device=dev, dtype=torch.bfloat16) for k in (4096, 14336)}
        for k in xin:
            xin[k][:, torch.randperm(k, generator=g)[: k // 100].to(dev)] *= 50
        layers = []
        ws_need = 0
        for name, k, n_out in shapes:
            m, n = (64, 64) if k == 4096 else (112, 128)
            left = torch.linalg.qr(torch.randn(m, m, dtype=torch.float64, generator=g)).Q.bfloat16().contiguous().to(dev)
            right = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, generator=g)).Q.bfloat16().contiguous().to(dev)
            wp = torch.randint(-2**31, 2**31 - 1, (n_out, k // 8), generator=g, dtype=torch.int32).to(dev)
            sw = (torch.rand(n_out, generator=g) * 0.01 + 0.001).to(dev)
            w8 = torch.empty(lib.qo_prepared_weights_bytes(n_out, k), dtype=torch.uint8, device=dev)
            nat.check(lib.qo_prepare_weights(vp(wp), vp(w8), n_out, k, sp))
            out = torch.empty(tloc, n_out, dtype=torch.bfloat16, device=dev)
            ws_need = max(ws_need, lib.qo_w4a4_linear_prepared_workspace_bytes(chunk, k, n_out))
            layers.append((k, n_out, m, n, left, right, wp, w8, sw, out))
        ws = torch.empty(ws_need, dtype=torch.uint8, device=dev)

        def step(i):
            for k, n_out, m, n, left, right, wp, w8, sw, out in layers:
                x = xin[k]
                for r0 in range(0, tloc, chunk):
                    rows = min(chunk, tloc - r0)
                    nat.check(lib.qo_w4a4_linear_prepared(C.c_void_p(x.data_ptr() + r0 * k * 2), k, vp(left), vp(right), vp(wp), vp(w8),
                                                          vp(sw), None, C.c_void_p(out.data_ptr() + r0 * n_out * 2), rows, m, n, n_out,
                                                          CLIP, nat.QO_BF16, nat.QO_BF16, vp(ws), ws_need, sp))

        ops_per_token = 2.0 * sum(k * n_out for _, k, n_out in shapes)
        desc = {"workload": "Llama-3-8B-shaped W4A4 projection stack (q, k, v, o, gate, up, down), 65,536 bf16 tokens split by rows over the ranks, "
                            "per-layer random-orthogonal L/R, random int4 weights kept widened (qo_prepare_weights), outputs stay row-sharded",
                "tokens_per_gpu": tloc, "parallelism": f"rows x{world}, no collective", "l2": "activations and outputs of a step are 8 GB per 65,536 tokens"}
        metric, unit = "w4a4_stack_tokens_per_s", "tokens/s"
        scale_value = lambda sec: total_tokens / sec
        dtype = "bf16 -> s4 x s4 -> s32 -> bf16"

        def roof(v):
            tops = v / world * ops_per_token / 1e12
            return {"bound": "tensor", "achieved": tops, "peak": tc_peak, "unit": "TOP/s", "frac": tops / tc_peak, "traffic": None,
                    "peak_source": tc_src, "algorithmic_ops_per_token": ops_per_token}
    elif args.workload in ("quantize_wide", "quantize_tokens"):
        # quantize_tokens: the headline shape (64 x 64) at another token count, to separate the fixed cost of a
        # launch (first-tile latency of the pipeline) from the streaming rate
        tokens, m, n = (4096, 112, 128) if args.workload == "quantize_wide" else (int(args.tokens or 65536), 64, 64)
        feat = m * n
        x = torch.randn(tokens, feat, generator=g)
        x[:, torch.randperm(feat, generator=g)[: feat // 100]] *= 50
        left = torch.linalg.qr(torch.randn(m, m, dtype=torch.float64, generator=g)).Q.bfloat16().contiguous().to(dev)
        right = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, generator=g)).Q.bfloat16().contiguous().to(dev)
        nsets = max(2, int(400e6 // (tokens * feat * 2)) + 1)  # the input sets together exceed L2 (3 x 147 MB for quantize_wide)
        xs = [torch.roll(x, i, 0).bfloat16().to(dev) for i in range(nsets)]
        codes = [torch.empty(tokens, feat // 8, dtype=torch.int32, device=dev) for _ in range(nsets)]
        scales = [torch.empty(tokens, dtype=torch.float32, device=dev) for _ in range(nsets)]
        algo = tokens * (feat * 2 + feat // 2 + 4) + (m * m + n * n) * 2

        def step(i):
            s = i % nsets
            nat.check(lib.qo_flatquant_quantize(vp(xs[s]), feat, vp(left), vp(right), vp(codes[s]), vp(scales[s]), tokens, m, n,
                                                CLIP, nat.QO_BF16, 1, nat.QO_F32, sp))

        desc = {"workload": f"flatquant_quantize x[{tokens},{feat}] bf16, 1% outlier channels x50, L {m}x{m} / R {n}x{n} orthogonal, clip 0.9, pack_int32",
                "l2": f"inputs rotate over {nsets} buffer sets ({nsets * tokens * feat * 2 // 1000000} MB) > L2"}
        metric, unit, scale_value = "flatquant_quantize_GBps", "GB/s", lambda sec: algo / sec / 1e9
        roof = lambda v: {"bound": "hbm", "achieved": v, "peak": hbm_peak, "unit": "GB/s", "frac": v / hbm_peak, "traffic": None,
                          "peak_source": hbm_src, "algorithmic_bytes_per_launch": algo}
        dtype = "bf16"
    else:
        if args.workload == "gemm":
            t, k, n_out = 4096, 4096, 4096
        else:
            t, k, n_out = int(args.tokens or 16), 14336, 4096
        nw = max(2, int(200e6 // (n_out * k // 2)) + 1)  # weight buffers that together exceed L2
        wps = [torch.randint(-2**31, 2**31 - 1, (n_out, k // 8), generator=g, dtype=torch.int32).to(dev) for _ in range(nw)]
        sw = (torch.rand(n_out, generator=g) * 0.01 + 0.001).to(dev)
        out = torch.empty(t, n_out, dtype=torch.bfloat16, device=dev)
        ops = 2.0 * t * k * n_out
        if args.workload == "gemm":
            ap = torch.randint(-2**31, 2**31 - 1, (t, k // 8), generator=g, dtype=torch.int32).to(dev)
            sa = (torch.rand(t, generator=g) * 0.1 + 0.01).to(dev)
            need = lib.qo_int4_matmul_workspace_bytes(t, k, n_out)
            ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)

            def step(i):
                nat.check(lib.qo_int4_matmul(vp(ap), k // 8, vp(wps[i % nw]), 1, k // 8, vp(sa), vp(sw), vp(out), nat.QO_BF16, t, k,
                                             n_out, None, vp(ws), need, sp))

            desc = {"workload": "int4_matmul 4096 x 4096 x 4096 packed int4, bf16 out; the call widens both operands to int8, then runs the tcgen05 GEMM",
                    "l2": f"weights rotate over {nw} buffers"}
        else:
            m, n = 112, 128
            x = torch.randn(t, k, generator=g).bfloat16().to(dev)
            left = torch.linalg.qr(torch.randn(m, m, dtype=torch.float64, generator=g)).Q.bfloat16().contiguous().to(dev)
            right = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, generator=g)).Q.bfloat16().contiguous().to(dev)
            if args.prepared:
                need = lib.qo_w4a4_linear_prepared_workspace_bytes(t, k, n_out)
                w8s = [torch.empty(lib.qo_prepared_weights_bytes(n_out, k), dtype=torch.uint8, device=dev) for _ in range(nw)]
                for wp, w8 in zip(wps, w8s):
                    nat.check(lib.qo_prepare_weights(vp(wp), vp(w8), n_out, k, sp))
            else:
                need = lib.qo_w4a4_linear_workspace_bytes(t, k, n_out)
            ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)

            def step(i):
                if args.prepared:
                    nat.check(lib.qo_w4a4_linear_prepared(vp(x), k, vp(left), vp(right), vp(wps[i % nw]), vp(w8s[i % nw]), vp(sw), None,
                                                          vp(out), t, m, n, n_out, CLIP, nat.QO_BF16, nat.QO_BF16, vp(ws), need, sp))
                else:
                    nat.check(lib.qo_w4a4_linear(vp(x), k, vp(left), vp(right), vp(wps[i % nw]), vp(sw), None, vp(out), t, m, n, n_out,
                                                 CLIP, nat.QO_BF16, nat.QO_BF16, vp(ws), need, sp))

            desc = {"workload": f"w4a4_linear{' with weights kept as int8' if args.prepared else ''} (quantize + packed int4 GEMM) {t} tokens, 14336 -> 4096, bf16 in / out",
                    "l2": f"weights rotate over {nw} buffers ({nw * n_out * k // 2 // 10**6} MB) > L2"}
        metric, unit, scale_value = "int4_matmul_TOPs", "TOP/s", lambda sec: ops / sec / 1e12
        weight_bytes = n_out * k // 2

        def roof(v):
            r = {"bound": "tensor", "achieved": v, "peak": tc_peak, "unit": "TOP/s", "frac": v / tc_peak, "traffic": None,
                 "peak_source": tc_src, "algorithmic_ops_per_launch": ops}
            # few rows: the bound is reading the packed weights once
            if t <= 256:
                sec = ops / (v * 1e12)
                gbs = weight_bytes / sec / 1e9
                r = {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak, "traffic": None,
                     "peak_source": hbm_src, "algorithmic_bytes_per_launch": weight_bytes}
            return r
        dtype = "s4 x s4 -> s32"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(3, args.warmup)):
        step(i)
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    launches0 = lib.qo_kernel_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for i in range(args.steps):
        step(i)
    ev1.record(stream)
    barrier()
    launches = lib.qo_kernel_launch_count() - launches0
    clocks = sampler.stop()
    sec = ev0.elapsed_time(ev1) / 1e3 / args.steps
    if lib.qo_device_status(sp) != 0:
        raise SystemExit("bench.py: device status " + str(lib.qo_last_error()))
    if world > 1:
        tmax = torch.tensor([sec], dtype=torch.float64, device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        sec = float(tmax[0])
        dist.destroy_process_group()
        if rank != 0:
            return
    value = scale_value(sec)
    desc["gemm_kernel"] = {0: "-", 1: "generic SIMT", 2: "tcgen05", 3: "weight-streaming"}.get(lib.qo_last_gemm_path(), "?")
    print(json.dumps({
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong" if args.workload == "stack" else "weak", "vs_baseline": None,
        "dtype": dtype, "data": "synthetic", "config": desc, "roofline": roof(value), "gpu_launches": int(launches), "clocks": clocks,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="quantize", choices=["quantize", "quantize_wide", "quantize_tokens", "gemm", "linear", "stack"])
    ap.add_argument("--tokens", type=int, default=None, help="rows of the `linear` (default 16) and `quantize_tokens` (default 65536) workloads")
    ap.add_argument("--prepared", action="store_true", help="`linear`: weights also kept widened to int8 (qo_prepare_weights)")
    args = ap.parse_args()
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        # started by hand rather than by torchrun: start one rank per GPU ourselves
        import subprocess

        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.abspath(__file__), *sys.argv[1:]]
        raise SystemExit(subprocess.call(cmd))
    if args.impl == "reference":
        run_reference(args)
    elif args.workload != "quantize":
        run_other(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
