#!/usr/bin/env python
"""Benchmark of the W4A4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--repeats R]

The default run (`--workload all`) prints ONE JSON line.  Its top-level keys are the headline workload; the other
measured parts of the path hang below it as sub-records, each with its own roofline, CPU baseline and end-to-end figure:

  headline   FlatQuant quantizer at activation scale: x [8192, 4096] bf16 ~ N(0,1) with 1 % of the channels x50, L and
             R 64 x 64 random orthogonal, clip 0.9, packed int32 codes + per-token scales.  One step = one pass of the
             quantizer over one batch; `value` = algorithmic GB/s with inputs resident in HBM.  With N > 1 every rank
             quantizes its own 8192 tokens (weak scaling, no collective).
  "gemm"     packed-int4 GEMM, T = K = 4096 with A produced by the quantizer, n_out in {4096, 11008, 14336}; TOP/s.
  "linear"   fused quantize -> GEMM, 14336 -> 4096, T in {1, 16, 256, 4096}, packed weights and prepared weights.
  "stack"    the seven W4A4 projections of a Llama-3-8B layer over 65,536 tokens split by rows over the ranks (strong
             scaling; tokens/s; max over ranks), without and with the optional NCCL all-gather of the outputs.
  "quantize_wide"  the quantizer at the down-projection shape, x [4096, 14336].

Timing: W warm-up steps, then R regions of exactly K steps each, every region bracketed by barrier + device
synchronise on both sides and timed with CUDA events on the launching stream; the maximum over ranks is taken per
region and the MEDIAN region gives `ms_per_step` (min and max are reported beside it).  Operands rotate through buffer
sets that together exceed the L2 cache.  `graph_ms_per_step` is the same K steps captured once in a CUDA graph and
replayed.  SM clock and throttle reasons are sampled while the regions run.

`--impl reference` times the reference's CPU implementation of the same workloads (its torch CPU op chain, restated in
oracle/torch_port.py) on all host cores: the headline on the full 8192 tokens per step, the sub-records on the
bounded samples they name.  `--workload NAME` (quantize, quantize_wide, quantize_tokens, gemm, linear, stack)
restricts either arm to one part; single-part lines carry that part's metric at the top level.
"""
from __future__ import annotations

import argparse
import ctypes as C
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
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
NOMINAL_INT8_TOPS = 4500.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from the ncu capture summarised in the named file
NCU_TRAFFIC = {
    "quantize": (69_641_472, "profiles/flatquant_n64_8192x4096.md"),
}
STACK_SHAPES = [("q", 4096, 4096), ("k", 4096, 1024), ("v", 4096, 1024), ("o", 4096, 4096), ("gate", 4096, 14336),
                ("up", 4096, 14336), ("down", 14336, 4096)]
STACK_TOKENS = 65536


# ---------------------------------------------------------------------------------------------------------------
# shared helpers
# ---------------------------------------------------------------------------------------------------------------
def quant_bytes(tokens, m, n):
    feat = m * n
    return tokens * (feat * 2 + feat // 2 + 4) + (m * m + n * n) * 2


def make_activations(tokens, feat, seed, device=None):
    """x ~ N(0,1) with 1 % of the channels (seeded choice) multiplied by 50, bf16."""
    import torch

    g = torch.Generator().manual_seed(seed)
    if device is None:
        x = torch.randn(tokens, feat, generator=g)
        x[:, torch.randperm(feat, generator=g)[: feat // 100]] *= 50
        return x.bfloat16().contiguous()
    gd = torch.Generator(device=device).manual_seed(seed)  # large batches are drawn on the device
    x = torch.randn(tokens, feat, generator=gd, device=device, dtype=torch.bfloat16)
    x[:, torch.randperm(feat, generator=g)[: feat // 100].to(device)] *= 50
    return x


def make_transforms(m, n, seed):
    import torch

    g = torch.Generator().manual_seed(seed)
    left = torch.linalg.qr(torch.randn(m, m, dtype=torch.float64, generator=g)).Q
    right = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, generator=g)).Q
    return left.bfloat16().contiguous(), right.bfloat16().contiguous()


def make_inputs(tokens, seed):
    left, right = make_transforms(M, N_, seed + 1000)
    return make_activations(tokens, FEAT, seed), left, right


def measured_peaks():
    """(HBM GB/s, int8 TOP/s, source strings) from MEASURED_PEAKS.json; the file holds no int8 figure, so the int8
    tensor peak is taken as twice the measured bf16 GEMM burst (int8 runs at twice the bf16 rate)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            d = json.load(fh)
        return (float(d["hbm_gbs"]), 2.0 * float(d["bf16_tflops"]), "measured (MEASURED_PEAKS.json, copy bandwidth)",
                "2 x measured bf16 GEMM burst (MEASURED_PEAKS.json)")
    except Exception:
        return (FALLBACK_HBM_GBS, 2.0 * FALLBACK_BF16_TFLOPS, "fallback (6.65 TB/s, an earlier copy measurement)",
                "2 x fallback bf16 burst (1.59 PFLOP/s)")


class ClockSampler(threading.Thread):
    """Polls NVML for SM clock and throttle reasons while the timed regions run."""

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


class Env:
    """Process-wide state of one rank: device, stream, library handle, distributed group."""

    def __init__(self):
        import torch

        from quant_ops_b200 import _native as nat

        self.torch, self.nat, self.lib = torch, nat, nat.lib
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        self.stream = torch.cuda.current_stream()
        self.sp = C.c_void_p(self.stream.cuda_stream)
        self.hbm_peak, self.tc_peak, self.hbm_src, self.tc_src = measured_peaks()

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if self.dist is None:
            return list(values)
        t = self.torch.tensor(list(values), dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()


def vp(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def time_regions(env: Env, step, steps: int, warmup: int, repeats: int):
    """W warm-up steps, then `repeats` regions of exactly `steps` steps; returns per-region milliseconds (max over
    ranks), the kernel launches of one region and the clock record taken while the regions ran."""
    torch = env.torch
    it = 0
    for _ in range(warmup):
        step(it, env.sp)
        it += 1
    env.barrier()
    sampler = ClockSampler(physical_gpu_index(env.local_rank))
    sampler.start()
    regions, launches = [], 0
    for _ in range(repeats):
        env.barrier()
        l0 = env.lib.qo_kernel_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(env.stream)
        for _ in range(steps):
            step(it, env.sp)
            it += 1
        e1.record(env.stream)
        env.barrier()
        launches = env.lib.qo_kernel_launch_count() - l0
        regions.append(e0.elapsed_time(e1))
    clocks = sampler.stop()
    if env.lib.qo_device_status(env.sp) != 0:
        raise SystemExit("bench.py: device status " + env.lib.qo_last_error().decode())
    return env.max_over_ranks(regions), int(launches), clocks


def graph_replay_ms(env: Env, step, steps: int, repeats: int):
    """The same `steps` steps captured once in a CUDA graph and replayed; median milliseconds per replay (max over
    ranks), or None when the capture is refused."""
    torch = env.torch
    try:
        side = torch.cuda.Stream()
        side.wait_stream(env.stream)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            sp = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            for i in range(steps):
                step(i, sp)
        for _ in range(2):
            graph.replay()
        env.barrier()
        times = []
        for _ in range(repeats):
            env.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(env.stream)
            graph.replay()
            e1.record(env.stream)
            env.barrier()
            times.append(e0.elapsed_time(e1))
        del graph
        return statistics.median(env.max_over_ranks(times))
    except Exception as exc:  # a refused capture is reported, not hidden
        sys.stderr.write(f"bench.py: CUDA-graph replay skipped: {exc}\n")
        torch.cuda.synchronize()
        return None


def summarize(regions, steps):
    med = statistics.median(regions)
    return {"ms_per_step": med / steps, "ms_per_step_min": min(regions) / steps, "ms_per_step_max": max(regions) / steps,
            "regions": len(regions), "steps_per_region": steps}


def host_cores():
    return os.cpu_count() or 1


def cpu_time(fn, warm=1, runs=3):
    """min over `runs` of fn() on the host cores, seconds (the reference's CPU path is deterministic work)."""
    import torch

    torch.set_num_threads(host_cores())
    for _ in range(warm):
        fn()
    best = None
    for _ in range(runs):
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best


# ---------------------------------------------------------------------------------------------------------------
# quantizer workloads
# ---------------------------------------------------------------------------------------------------------------
def quantizer_record(env: Env, args, tokens, m, n, label, headline=False):
    torch, lib, nat = env.torch, env.lib, env.nat
    feat = m * n
    x = make_activations(tokens, feat, SEED + env.rank)
    left, right = make_transforms(m, n, SEED + 1000 + env.rank)
    nsets = max(4, int(400e6 // (tokens * feat * 2)) + 1)  # the input sets together exceed the 126 MB L2
    nsets = min(nsets, 64)
    xs = [x.to(env.dev) if i == 0 else torch.roll(x, i, 0).to(env.dev) for i in range(nsets)]
    ld, rd = left.to(env.dev), right.to(env.dev)
    codes = [torch.empty(tokens, feat // 8, dtype=torch.int32, device=env.dev) for _ in range(nsets)]
    scales = [torch.empty(tokens, dtype=torch.float32, device=env.dev) for _ in range(nsets)]
    algo = quant_bytes(tokens, m, n)

    def step(i, sp):
        s = i % nsets
        nat.check(lib.qo_flatquant_quantize(vp(xs[s]), feat, vp(ld), vp(rd), vp(codes[s]), vp(scales[s]), tokens, m, n,
                                            CLIP, nat.QO_BF16, 1, nat.QO_F32, sp))

    regions, launches, clocks = time_regions(env, step, args.steps, max(3, args.warmup), args.repeats)
    rec = summarize(regions, args.steps)
    path = lib.qo_last_quantizer_path()
    graph_ms = graph_replay_ms(env, step, args.steps, min(args.repeats, 15))
    # the same call on ONE buffer set every step (input and outputs of a step fit the 126 MB L2 for the benchmarked
    # shape): stated separately, never the headline
    warm_regions, _, _ = time_regions(env, lambda i, sp: step(0, sp), args.steps, 3, min(args.repeats, 9))
    warm = summarize(warm_regions, args.steps)

    # a few rows against the oracle, so a fast-but-wrong run cannot print a number
    from oracle import w4a4_oracle as O

    rows = sorted({0, 1, tokens // 2 + 1, tokens - 1})
    rc, rs = O.flatquant_quantize(xs[0][rows].float().cpu().numpy(), left.float().numpy(), right.float().numpy(), CLIP, True, "bf16")
    diff = abs(O.unpack_int32_to_int4(codes[0][rows].cpu().numpy()).astype(int) - O.unpack_int32_to_int4(rc).astype(int))
    parity_ok = bool(diff.max() <= 1 and (diff != 0).mean() <= 1e-3 and
                     abs(scales[0][rows].cpu().numpy() - rs).max() <= 1e-3 * abs(rs).max())

    sec = rec["ms_per_step"] / 1e3
    per_gpu = algo / sec / 1e9
    traffic = NCU_TRAFFIC.get(label, (None, None))
    rec.update({
        "workload": f"flatquant_quantize x[{tokens},{feat}] bf16, 1% outlier channels x50, L {m}x{m} / R {n}x{n} orthogonal, clip {CLIP}, pack_int32",
        "value": per_gpu * env.world, "unit": "GB/s",
        "graph_ms_per_step": None if graph_ms is None else graph_ms / args.steps,
        "l2_warm_ms_per_step": warm["ms_per_step"],
        "kernel": {1: "generic SIMT", 2: "tcgen05"}.get(path, "?"), "parity_vs_oracle_sample": parity_ok,
        "l2": f"inputs and outputs rotate over {nsets} buffer sets ({nsets * algo // 10**6} MB) > L2, every step reads HBM",
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": env.hbm_peak, "unit": "GB/s", "frac": per_gpu / env.hbm_peak,
                     "traffic": traffic[0], "traffic_source": traffic[1], "peak_source": env.hbm_src,
                     "algorithmic_bytes_per_launch": algo,
                     "graph_replay_frac": None if graph_ms is None else algo / (graph_ms / args.steps / 1e3) / 1e9 / env.hbm_peak},
        "gpu_launches": launches, "clocks": clocks,
    })

    if headline:
        # end to end through the host-buffer entry point: pinned host input, pinned host outputs, copies inside the timing
        xh = x.pin_memory()
        ch = torch.empty(tokens, feat // 8, dtype=torch.int32).pin_memory()
        sh = torch.empty(tokens, dtype=torch.float32).pin_memory()
        e2e_steps = max(3, min(args.steps, 20))

        def e2e_step():
            nat.check(lib.qo_flatquant_quantize_host(vp(xh), vp(left), vp(right), vp(ch), vp(sh), tokens, m, n, CLIP,
                                                     nat.QO_BF16, 1, nat.QO_F32))

        for _ in range(2):
            e2e_step()
        env.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        e2e_ms = env.max_over_ranks([(time.perf_counter() - t0) * 1e3])[0]
        rec["e2e"] = {"value": algo * e2e_steps * env.world / (e2e_ms / 1e3) / 1e9, "unit": "GB/s",
                      "h2d_bytes_per_step": tokens * feat * 2 + (m * m + n * n) * 2, "d2h_bytes_per_step": tokens * (feat // 2 + 4),
                      "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                      "call": "qo_flatquant_quantize_host: pinned host x -> device slices -> kernel -> pinned host codes and scales"}
    if env.world == 1 and env.rank == 0 and not args.no_cpu_baseline:
        rec["cpu_baseline"] = cpu_quantize(tokens, m, n, 3)
    del xs, codes, scales
    torch.cuda.empty_cache()
    return rec


def cpu_quantize(tokens, m, n, runs):
    from oracle import torch_port

    x = make_activations(tokens, m * n, SEED)
    left, right = make_transforms(m, n, SEED + 1000)
    sec = cpu_time(lambda: torch_port.quantize(x, left, right, CLIP, True), 1, runs)
    return {"value": quant_bytes(tokens, m, n) / sec / 1e9, "unit": "GB/s", "cores": host_cores(), "kind": "port", "ms_per_step": sec * 1e3,
            "sample": f"all {tokens} tokens per step, min of {runs} steps; the reference's torch CPU op chain, {host_cores()} threads"}


def dequantize_record(env: Env, args, tokens=TOKENS, feat=M * N_):
    """dequantize_int4 of packed codes: [tokens, feat / 8] int32 + float32 scales -> float32 [tokens, feat] (write-bound)."""
    torch, lib, nat = env.torch, env.lib, env.nat
    g = torch.Generator(device=env.dev).manual_seed(SEED + 7)
    nsets = 3  # 3 x (17 MB in + 134 MB out) > L2
    codes = [torch.randint(-2**31, 2**31 - 1, (tokens, feat // 8), generator=g, device=env.dev, dtype=torch.int32) for _ in range(nsets)]
    scales = [torch.rand(tokens, generator=g, device=env.dev) * 0.1 + 0.01 for _ in range(nsets)]
    outs = [torch.empty(tokens, feat, device=env.dev) for _ in range(nsets)]
    algo = tokens * (feat // 2 + 4 + 4 * feat)

    def step(i, sp):
        j = i % nsets
        nat.check(lib.qo_dequantize_int4(vp(codes[j]), vp(scales[j]), vp(outs[j]), tokens, feat, 1, nat.QO_F32, sp))

    regions, launches, clocks = time_regions(env, step, args.sub_steps, 3, args.sub_repeats)
    rec = summarize(regions, args.sub_steps)
    from oracle import w4a4_oracle as O

    step(0, env.sp)
    torch.cuda.synchronize()
    rows = [0, 1, tokens // 2, tokens - 1]
    ref = O.dequantize_int4(codes[0][rows].cpu().numpy(), scales[0][rows].cpu().numpy(), True)
    parity_ok = bool((outs[0][rows].cpu().numpy() == ref).all())
    gbps = algo / (rec["ms_per_step"] / 1e3) / 1e9
    rec.update({"workload": f"dequantize_int4: packed codes [{tokens}, {feat // 8}] + scales -> float32 [{tokens}, {feat}]",
                "value": gbps, "unit": "GB/s", "parity_vs_oracle_sample": parity_ok, "l2": f"{nsets} buffer sets ({nsets * algo // 10**6} MB) > L2",
                "roofline": {"bound": "hbm", "achieved": gbps, "peak": env.hbm_peak, "unit": "GB/s", "frac": gbps / env.hbm_peak, "traffic": None,
                             "peak_source": env.hbm_src, "algorithmic_bytes_per_launch": algo},
                "gpu_launches": launches, "clocks": clocks})
    if not args.no_cpu_baseline:
        sample = 1024
        c_cpu, s_cpu = codes[0][:sample].cpu().numpy(), scales[0][:sample].cpu().numpy()
        sec = cpu_time(lambda: O.dequantize_int4(c_cpu, s_cpu, True), 1, 3)
        rec["cpu_baseline"] = {"value": sample * (feat // 2 + 4 + 4 * feat) / sec / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                               "ms_per_step": sec * 1e3, "sample": f"{sample} of the {tokens} tokens, min of 3; numpy restatement of the reference's unpack-and-scale loop"}
    del codes, scales, outs
    torch.cuda.empty_cache()
    return rec


# ---------------------------------------------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------------------------------------------
def tensor_roofline(env, tops, ops):
    return {"bound": "tensor", "achieved": tops, "peak": env.tc_peak, "unit": "TOP/s", "frac": tops / env.tc_peak,
            "frac_of_nominal_int8_dense": tops / NOMINAL_INT8_TOPS, "nominal_int8_dense": NOMINAL_INT8_TOPS, "traffic": None,
            "peak_source": env.tc_src, "algorithmic_ops_per_launch": ops}


def quantized_weights(env, n_out, k, seed):
    """W ~ N(0, 0.02) quantized per output channel (absmax / 7) on the device: packed [n_out, k/8] + float32 scales."""
    torch, lib, nat = env.torch, env.lib, env.nat
    gd = torch.Generator(device=env.dev).manual_seed(seed)
    w = torch.randn(n_out, k, generator=gd, device=env.dev) * 0.02
    wp = torch.empty(n_out, k // 8, dtype=torch.int32, device=env.dev)
    sw = torch.empty(n_out, device=env.dev)
    nat.check(lib.qo_quantize_weights_int4(vp(w), vp(wp), vp(sw), n_out, k, env.sp))
    torch.cuda.synchronize()
    return wp, sw


def gemm_records(env: Env, args, n_outs):
    """cfg 3: A [4096, 4096] packed = the quantizer's output on the headline activations; W [n_out, 4096]."""
    torch, lib, nat = env.torch, env.lib, env.nat
    from oracle import torch_port
    from oracle import w4a4_oracle as O

    t, k = 4096, 4096
    x, left, right = make_inputs(t, SEED)
    ap = torch.empty(t, k // 8, dtype=torch.int32, device=env.dev)
    sa = torch.empty(t, dtype=torch.float32, device=env.dev)
    xd, ld, rd = x.to(env.dev), left.to(env.dev), right.to(env.dev)
    nat.check(lib.qo_flatquant_quantize(vp(xd), k, vp(ld), vp(rd), vp(ap), vp(sa), t, M, N_, CLIP, nat.QO_BF16, 1, nat.QO_F32, env.sp))
    torch.cuda.synchronize()
    out_recs = []
    for n_out in n_outs:
        wp, sw = quantized_weights(env, n_out, k, SEED + n_out)
        nw = max(2, int(200e6 // (n_out * k // 2)) + 1)  # weight buffers that together exceed L2
        wps = [wp] + [torch.roll(wp, i, 0) for i in range(1, nw)]
        sws = [sw] + [torch.roll(sw, i, 0) for i in range(1, nw)]
        out = torch.empty(t, n_out, dtype=torch.float16, device=env.dev)
        need = lib.qo_int4_matmul_workspace_bytes(t, k, n_out)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device=env.dev)
        ops = 2.0 * t * k * n_out

        def step(i, sp):
            j = i % nw
            nat.check(lib.qo_int4_matmul(vp(ap), k // 8, vp(wps[j]), 1, k // 8, vp(sa), vp(sws[j]), vp(out), nat.QO_F16, t, k, n_out,
                                         None, vp(ws) if need else None, need, sp))

        regions, launches, clocks = time_regions(env, step, args.sub_steps, 3, args.sub_repeats)
        rec = summarize(regions, args.sub_steps)
        graph_ms = graph_replay_ms(env, step, args.sub_steps, min(args.sub_repeats, 9))
        sec = rec["ms_per_step"] / 1e3
        tops = ops / sec / 1e12
        # parity: outputs of sampled rows against the oracle (exact: same integer sums, same two float32 multiplies)
        step(0, env.sp)
        torch.cuda.synchronize()
        rows = [0, 1, 2047, 4095]
        ref = O.int4_matmul(ap[rows].cpu().numpy(), wp.cpu().numpy().T, sa[rows].cpu().numpy(), sw.cpu().numpy(), "fp16")
        parity_ok = bool((out[rows].float().cpu().numpy() == ref).all())
        rec.update({"workload": f"int4_matmul T={t} K={k} n_out={n_out}: A packed by the quantizer, W ~ N(0, 0.02) per-channel int4, fp16 out",
                    "value": tops, "unit": "TOP/s", "graph_ms_per_step": None if graph_ms is None else graph_ms / args.sub_steps,
                    "kernel": {1: "generic SIMT", 2: "tcgen05", 3: "weight-streaming"}.get(lib.qo_last_gemm_path(), "?"),
                    "parity_vs_oracle_sample": parity_ok, "l2": f"weights rotate over {nw} buffers",
                    "path": ("packed operands by TMA, nibbles unpacked in the kernel (A through tensor memory, B in shared memory), no workspace use"
                             if launches == args.sub_steps else
                             "widening pass (nibbles -> int8 in the workspace) + int8 tensor-core kernel on single CTAs"),
                    "roofline": tensor_roofline(env, tops, ops), "gpu_launches": launches, "clocks": clocks})
        # the library GEMM on already widened int8 operands, for comparison in the same run (not part of the product path)
        try:
            a8 = torch.randint(-8, 8, (t, k), dtype=torch.int8, device=env.dev)
            b8 = torch.randint(-8, 8, (n_out, k), dtype=torch.int8, device=env.dev).t()
            for _ in range(3):
                torch._int_mm(a8, b8)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(args.sub_steps):
                torch._int_mm(a8, b8)
            e1.record()
            torch.cuda.synchronize()
            lib_sec = e0.elapsed_time(e1) / 1e3 / args.sub_steps
            rec["library_int8_gemm"] = {"call": "torch._int_mm (cuBLASLt) on int8 operands already in memory, int32 out, no unpack, no scale epilogue",
                                        "ms_per_step": lib_sec * 1e3, "value": ops / lib_sec / 1e12, "unit": "TOP/s"}
            del a8, b8
        except Exception as exc:
            rec["library_int8_gemm"] = {"unavailable": str(exc)[:200]}
        # end to end: packed activations + scales from pinned host memory, fp16 output back to pinned host memory
        aph, sah = ap.cpu().pin_memory(), sa.cpu().pin_memory()
        outh = torch.empty(t, n_out, dtype=torch.float16).pin_memory()
        apd2, sad2 = torch.empty_like(ap), torch.empty_like(sa)

        def e2e_step():
            apd2.copy_(aph, non_blocking=True)
            sad2.copy_(sah, non_blocking=True)
            nat.check(lib.qo_int4_matmul(vp(apd2), k // 8, vp(wp), 1, k // 8, vp(sad2), vp(sw), vp(out), nat.QO_F16, t, k, n_out,
                                         None, vp(ws) if need else None, need, env.sp))
            outh.copy_(out, non_blocking=True)
            torch.cuda.synchronize()

        e2e_step()
        t0 = time.perf_counter()
        for _ in range(3):
            e2e_step()
        e2e_sec = (time.perf_counter() - t0) / 3
        rec["e2e"] = {"value": ops / e2e_sec / 1e12, "unit": "TOP/s", "h2d_bytes_per_step": t * k // 2 + 4 * t,
                      "d2h_bytes_per_step": t * n_out * 2, "steps": 3, "ms_per_step": e2e_sec * 1e3,
                      "call": "pinned host A + scales -> device, qo_int4_matmul (weights resident), output -> pinned host"}
        if not args.no_cpu_baseline:
            a_c, w_c, sa_c, sw_c = ap.cpu(), wp.cpu(), sa.cpu(), sw.cpu()
            runs = 1 if n_out > 4096 else 2
            sec_c = cpu_time(lambda: torch_port.matmul(a_c, w_c.t(), sa_c, sw_c), 0, runs)
            rec["cpu_baseline"] = {"value": ops / sec_c / 1e12, "unit": "TOP/s", "cores": host_cores(), "kind": "port", "ms_per_step": sec_c * 1e3,
                                   "sample": f"the whole {t} x {k} x {n_out} product, min of {runs}; the reference's torch CPU op chain (unpack, float32 matmul, scales)"}
        out_recs.append(rec)
        del wps, sws, out, ws
        torch.cuda.empty_cache()
    return out_recs


# ---------------------------------------------------------------------------------------------------------------
# fused layer
# ---------------------------------------------------------------------------------------------------------------
def linear_records(env: Env, args, token_counts, variants):
    """cfg 4: x [T, 14336] bf16 with outlier channels, (112, 128) transforms, W [4096, 14336]."""
    torch, lib, nat = env.torch, env.lib, env.nat
    from oracle import torch_port
    from oracle import w4a4_oracle as O

    k, n_out, m, n = 14336, 4096, 112, 128
    left, right = make_transforms(m, n, SEED + 4)
    ld, rd = left.to(env.dev), right.to(env.dev)
    wp, sw = quantized_weights(env, n_out, k, SEED + 40)
    nw = max(2, int(200e6 // (n_out * k // 2)) + 1)
    wps = [wp] + [torch.roll(wp, i, 0) for i in range(1, nw)]
    sws = [sw] + [torch.roll(sw, i, 0) for i in range(1, nw)]
    w8s = None
    weight_bytes = n_out * k // 2
    recs = []
    for t in token_counts:
        x = make_activations(t, k, SEED + 4 + t)
        xd = x.to(env.dev)
        out = torch.empty(t, n_out, dtype=torch.bfloat16, device=env.dev)
        ops = 2.0 * t * k * n_out
        for prepared in variants:
            if prepared and w8s is None:
                w8s = [torch.empty(lib.qo_prepared_weights_bytes(n_out, k), dtype=torch.uint8, device=env.dev) for _ in range(nw)]
                for a, b in zip(wps, w8s):
                    nat.check(lib.qo_prepare_weights(vp(a), vp(b), n_out, k, env.sp))
            need = (lib.qo_w4a4_linear_prepared_workspace_bytes if prepared else lib.qo_w4a4_linear_workspace_bytes)(t, k, n_out)
            ws = torch.empty(max(need, 16), dtype=torch.uint8, device=env.dev)

            def step(i, sp, wsel=None):
                j = i % nw if wsel is None else wsel
                if prepared:
                    nat.check(lib.qo_w4a4_linear_prepared(vp(xd), k, vp(ld), vp(rd), vp(wps[j]), vp(w8s[j]), vp(sws[j]), None, vp(out), t, m, n,
                                                          n_out, CLIP, nat.QO_BF16, nat.QO_BF16, vp(ws), need, sp))
                else:
                    nat.check(lib.qo_w4a4_linear(vp(xd), k, vp(ld), vp(rd), vp(wps[j]), vp(sws[j]), None, vp(out), t, m, n, n_out, CLIP,
                                                 nat.QO_BF16, nat.QO_BF16, vp(ws), need, sp))

            regions, launches, clocks = time_regions(env, step, args.sub_steps, 3, args.sub_repeats)
            rec = summarize(regions, args.sub_steps)
            graph_ms = graph_replay_ms(env, step, args.sub_steps, min(args.sub_repeats, 9))
            sec = rec["ms_per_step"] / 1e3
            tops = ops / sec / 1e12
            step(0, env.sp, 0)
            torch.cuda.synchronize()
            rows = sorted({0, t // 2, t - 1})
            rc, rs = O.flatquant_quantize(x[rows].float().numpy(), left.float().numpy(), right.float().numpy(), CLIP, True, "bf16")
            ref = O.int4_matmul(rc, wp.cpu().numpy().T, rs, sw.cpu().numpy(), "bf16")
            got = out[rows].float().cpu().numpy()
            rng = abs(ref).max(axis=1, keepdims=True)
            parity_ok = bool((abs(got - ref) <= 1e-2 * abs(ref).clip(min=rng)).all())
            if t <= 256:  # few rows: the bound is reading the packed weights once
                gbs = weight_bytes / sec / 1e9
                roof = {"bound": "hbm", "achieved": gbs, "peak": env.hbm_peak, "unit": "GB/s", "frac": gbs / env.hbm_peak, "traffic": None,
                        "peak_source": env.hbm_src, "algorithmic_bytes_per_launch": weight_bytes + t * k * 2 + t * n_out * 2}
                if graph_ms is not None:
                    roof["graph_replay_frac"] = weight_bytes / (graph_ms / args.sub_steps / 1e3) / 1e9 / env.hbm_peak
            else:
                roof = tensor_roofline(env, tops, ops)
            rec.update({"workload": f"w4a4_linear{' with weights kept as int8' if prepared else ''}: quantize + packed int4 GEMM, {t} tokens, {k} -> {n_out}, bf16 in / out",
                        "tokens": t, "prepared": bool(prepared), "value": tops, "unit": "TOP/s",
                        "graph_ms_per_step": None if graph_ms is None else graph_ms / args.sub_steps,
                        "gemm_kernel": {1: "generic SIMT", 2: "tcgen05", 3: "weight-streaming"}.get(lib.qo_last_gemm_path(), "?"),
                        "parity_vs_oracle_sample": parity_ok, "l2": f"weights rotate over {nw} buffers ({nw * weight_bytes // 10**6} MB) > L2",
                        "roofline": roof, "gpu_launches": launches, "clocks": clocks})
            # end to end: activations from pinned host memory, outputs back to pinned host memory
            xh = x.pin_memory()
            outh = torch.empty(t, n_out, dtype=torch.bfloat16).pin_memory()

            def e2e_step():
                xd.copy_(xh, non_blocking=True)
                step(0, env.sp, 0)
                outh.copy_(out, non_blocking=True)
                torch.cuda.synchronize()

            e2e_step()
            t0 = time.perf_counter()
            for _ in range(3):
                e2e_step()
            e2e_sec = (time.perf_counter() - t0) / 3
            rec["e2e"] = {"value": ops / e2e_sec / 1e12, "unit": "TOP/s", "h2d_bytes_per_step": t * k * 2, "d2h_bytes_per_step": t * n_out * 2,
                          "steps": 3, "ms_per_step": e2e_sec * 1e3,
                          "call": "pinned host x -> device, fused layer (weights resident), output -> pinned host"}
            if not args.no_cpu_baseline and not prepared:
                w_c, sw_c = wp.cpu(), sw.cpu()
                sec_c = cpu_time(lambda: torch_port.linear(x, left, right, CLIP, w_c, sw_c), 0, 1)
                rec["cpu_baseline"] = {"value": ops / sec_c / 1e12, "unit": "TOP/s", "cores": host_cores(), "kind": "port", "ms_per_step": sec_c * 1e3,
                                       "sample": f"the whole layer on all {t} tokens, one run; the reference's torch CPU op chain"}
            elif recs and recs[-1].get("tokens") == t and "cpu_baseline" in recs[-1]:
                rec["cpu_baseline"] = recs[-1]["cpu_baseline"]  # same arithmetic, same CPU work
            recs.append(rec)
            del ws
        del xd, out
        torch.cuda.empty_cache()
    return recs


# ---------------------------------------------------------------------------------------------------------------
# projection stack
# ---------------------------------------------------------------------------------------------------------------
def stack_record(env: Env, args):
    """cfg 5: seven projections over 65,536 tokens split by rows over the ranks; weights prepared (kept as int8)."""
    torch, lib, nat = env.torch, env.lib, env.nat
    from quant_ops_b200 import sharding

    start, tloc = sharding.shard_rows(STACK_TOKENS, env.world, env.rank)
    chunk = min(tloc, 8192)
    xin = {k: make_activations(tloc, k, SEED + 50 + env.rank, device=env.dev) for k in (4096, 14336)}
    layers, ws_need = [], 0
    for idx, (name, k, n_out) in enumerate(STACK_SHAPES):
        m, n = (64, 64) if k == 4096 else (112, 128)
        left, right = make_transforms(m, n, SEED + 60 + idx)   # weights, L, R are replicated: same seeds on every rank
        wp, sw = quantized_weights(env, n_out, k, SEED + 70 + idx)
        w8 = torch.empty(lib.qo_prepared_weights_bytes(n_out, k), dtype=torch.uint8, device=env.dev)
        nat.check(lib.qo_prepare_weights(vp(wp), vp(w8), n_out, k, env.sp))
        out = torch.empty(tloc, n_out, dtype=torch.bfloat16, device=env.dev)
        ws_need = max(ws_need, lib.qo_w4a4_linear_prepared_workspace_bytes(chunk, k, n_out))
        layers.append((name, k, n_out, m, n, left.to(env.dev), right.to(env.dev), wp, w8, sw, out, left, right))
    ws = torch.empty(ws_need, dtype=torch.uint8, device=env.dev)

    def run_layer(layer, sp, out_override=None):
        name, k, n_out, m, n, left, right, wp, w8, sw, out = layer[:11]
        if out_override is not None:
            out = out_override
        x = xin[k]
        for r0 in range(0, tloc, chunk):
            rows = min(chunk, tloc - r0)
            nat.check(lib.qo_w4a4_linear_prepared(C.c_void_p(x.data_ptr() + r0 * k * 2), k, vp(left), vp(right), vp(wp), vp(w8),
                                                  vp(sw), None, C.c_void_p(out.data_ptr() + r0 * n_out * 2), rows, m, n, n_out,
                                                  CLIP, nat.QO_BF16, nat.QO_BF16, vp(ws), ws_need, sp))

    def step(i, sp):
        for layer in layers:
            run_layer(layer, sp)

    steps = max(1, min(args.sub_steps, 5))
    regions, launches, clocks = time_regions(env, step, steps, 2, max(3, min(args.sub_repeats, 7)))
    rec = summarize(regions, steps)
    sec = rec["ms_per_step"] / 1e3
    ops_per_token = 2.0 * sum(k * n_out for _, k, n_out in STACK_SHAPES)
    tokens_per_s = STACK_TOKENS / sec
    tops = tokens_per_s / env.world * ops_per_token / 1e12

    # parity: sampled rows of every projection against the oracle
    from oracle import w4a4_oracle as O

    step(0, env.sp)
    torch.cuda.synchronize()
    parity_ok = True
    rows = sorted({0, tloc // 3, tloc - 1})
    for name, k, n_out, m, n, left_d, right_d, wp, w8, sw, out, left, right in layers:
        rc, rs = O.flatquant_quantize(xin[k][rows].float().cpu().numpy(), left.float().numpy(), right.float().numpy(), CLIP, True, "bf16")
        ref = O.int4_matmul(rc, wp.cpu().numpy().T, rs, sw.cpu().numpy(), "bf16")
        got = out[rows].float().cpu().numpy()
        rng = abs(ref).max(axis=1, keepdims=True)
        parity_ok = parity_ok and bool((abs(got - ref) <= 1e-2 * abs(ref).clip(min=rng)).all())

    rec.update({
        "workload": "Llama-3-8B-shaped W4A4 projection stack (q, k, v, o, gate, up, down), 65,536 bf16 tokens with 1% outlier channels split by rows "
                    "over the ranks, per-layer random-orthogonal L/R, weights ~ N(0, 0.02) int4 per channel kept widened (qo_prepare_weights), "
                    "outputs stay row-sharded",
        "value": tokens_per_s, "unit": "tokens/s", "scaling": "strong", "tokens_per_gpu": tloc, "parallelism": f"rows x{env.world}, no data-path collective",
        "parity_vs_oracle_sample": parity_ok, "l2": "activations and outputs of a step are 8 GB per 65,536 tokens",
        "roofline": {**tensor_roofline(env, tops, ops_per_token * tloc), "algorithmic_ops_per_token": ops_per_token},
        "gpu_launches": launches, "clocks": clocks,
    })

    # optional all-gather of the outputs: projection i is gathered on a second stream under projection i+1's compute
    if env.dist is not None:
        comm = torch.cuda.Stream()
        fulls = [torch.empty(STACK_TOKENS, layer[2], dtype=torch.bfloat16, device=env.dev) for layer in layers]

        def step_gather(i, sp):
            for layer, full in zip(layers, fulls):
                run_layer(layer, sp)
                done = torch.cuda.Event()
                done.record(env.stream)
                comm.wait_event(done)
                with torch.cuda.stream(comm):
                    sharding.all_gather_rows(layer[10], STACK_TOKENS, out=full)
            env.stream.wait_stream(comm)

        gregions, glaunches, gclocks = time_regions(env, step_gather, steps, 2, max(3, min(args.sub_repeats, 5)))
        g = summarize(gregions, steps)
        gsec = g["ms_per_step"] / 1e3
        # every rank's slice of the gathered tensor must equal that rank's local output (checked through checksums)
        torch.cuda.synchronize()
        loc = torch.stack([layer[10].view(torch.int16).to(torch.int64).sum() for layer in layers])
        all_loc = [torch.empty_like(loc) for _ in range(env.world)]
        env.dist.all_gather(all_loc, loc)
        gathered_ok = True
        for r in range(env.world):
            s0, cnt = sharding.shard_rows(STACK_TOKENS, env.world, r)
            mine = torch.stack([full[s0:s0 + cnt].view(torch.int16).to(torch.int64).sum() for full in fulls])
            gathered_ok = gathered_ok and bool(torch.equal(mine, all_loc[r]))
        gathered_ok = gathered_ok and bool(torch.equal(fulls[0][start:start + tloc], layers[0][10]))
        gathered_bytes = sum(STACK_TOKENS * layer[2] * 2 for layer in layers)
        recv = gathered_bytes * (env.world - 1) / env.world
        g.update({"value": STACK_TOKENS / gsec, "unit": "tokens/s", "gathered_equals_local_slices": gathered_ok,
                  "bytes_received_per_gpu": recv, "nvlink_GBps_per_gpu": recv / gsec / 1e9,
                  "bound": "NVLink: every GPU receives (N-1)/N of the 5.64 GB of outputs per step; the compute of the next projection hides under it",
                  "gpu_launches": glaunches, "clocks": gclocks})
        rec["with_gather"] = g

        # The same gather done by the GEMM itself: its epilogue stores this rank's output rows into every rank's buffer
        # (the peers' buffers are mapped into this process with CUDA IPC).  No collective kernel, nothing takes SMs
        # from the GEMM.  The buffers of the NCCL variant above are reused as the destinations.
        try:
            for full in fulls:
                full.fill_(0)
            torch.cuda.synchronize()
            env.barrier()
            # (GatheredOutput allocates its own buffer; here the existing ones are shared instead)
            dsts = [adopt_gathered(sharding, full, env) for full in fulls]

            def step_fused(i, sp):
                for layer, dst in zip(layers, dsts):
                    name, k, n_out, m, n, left, right, wp, w8, sw = layer[:10]
                    x = xin[k]
                    arr = (C.c_void_p * env.world)(*dst.ptrs)
                    for r0 in range(0, tloc, chunk):
                        rows = min(chunk, tloc - r0)
                        nat.check(lib.qo_w4a4_linear_gather(C.c_void_p(x.data_ptr() + r0 * k * 2), k, vp(left), vp(right), vp(wp), vp(sw), None,
                                                            arr, env.world, start + r0, rows, m, n, n_out, CLIP, nat.QO_BF16, nat.QO_BF16,
                                                            vp(ws), ws_need, sp))

            fregions, flaunches, fclocks = time_regions(env, step_fused, steps, 2, max(3, min(args.sub_repeats, 5)))
            f = summarize(fregions, steps)
            fsec = f["ms_per_step"] / 1e3
            torch.cuda.synchronize()
            env.barrier()
            fused_ok = True
            for r in range(env.world):
                s0, cnt = sharding.shard_rows(STACK_TOKENS, env.world, r)
                mine = torch.stack([full[s0:s0 + cnt].view(torch.int16).to(torch.int64).sum() for full in fulls])
                fused_ok = fused_ok and bool(torch.equal(mine, all_loc[r]))
            fused_ok = fused_ok and bool(torch.equal(fulls[0][start:start + tloc], layers[0][10]))
            f.update({"value": STACK_TOKENS / fsec, "unit": "tokens/s", "gathered_equals_local_slices": fused_ok,
                      "bytes_sent_per_gpu": recv, "nvlink_GBps_per_gpu": recv / fsec / 1e9,
                      "how": "qo_w4a4_linear_gather: the GEMM's epilogue stores its rows into every rank's buffer over NVLink (peer memory "
                             "mapped with CUDA IPC); no collective kernel",
                      "gpu_launches": flaunches, "clocks": fclocks})
            rec["with_gather_fused"] = f
            env.barrier()

            # Third variant: the plain layer, then copy-engine transfers of its output rows into every rank's buffer on a
            # side stream (no SM is used), under the next projection's kernels.
            for full in fulls:
                full.fill_(0)
            torch.cuda.synchronize()
            env.barrier()

            def step_push(i, sp):
                for layer, dst in zip(layers, dsts):
                    run_layer(layer, sp, dst.local_rows())  # the layer writes this rank's rows of its own gathered buffer
                    done = torch.cuda.Event()
                    done.record(env.stream)
                    comm.wait_event(done)
                    dst.push_rows(dst.local_rows(), start, comm, include_self=False)
                env.stream.wait_stream(comm)

            pregions, plaunches, pclocks = time_regions(env, step_push, steps, 2, max(3, min(args.sub_repeats, 5)))
            pr = summarize(pregions, steps)
            psec = pr["ms_per_step"] / 1e3
            torch.cuda.synchronize()
            env.barrier()
            push_ok = True
            for r in range(env.world):
                s0, cnt = sharding.shard_rows(STACK_TOKENS, env.world, r)
                mine = torch.stack([full[s0:s0 + cnt].view(torch.int16).to(torch.int64).sum() for full in fulls])
                push_ok = push_ok and bool(torch.equal(mine, all_loc[r]))
            pr.update({"value": STACK_TOKENS / psec, "unit": "tokens/s", "gathered_equals_local_slices": push_ok,
                       "bytes_sent_per_gpu": recv, "nvlink_GBps_per_gpu": recv / psec / 1e9,
                       "how": "the layer writes its rows of its own gathered buffer; GatheredOutput.push_rows sends them into the peers' "
                              "buffers (CUDA IPC) with copy-engine transfers on a side stream, under the next projection's kernels",
                       "gpu_launches": plaunches, "clocks": pclocks})
            rec["with_gather_copy_engine"] = pr
            env.barrier()
            for d in dsts:
                d.close()
        except Exception as e:  # the plain and the NCCL figures stand without it
            rec["with_gather_fused"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        del fulls
    else:
        rec["with_gather"] = {"skipped": "one rank: nothing to gather"}

    if env.world == 1 and not args.no_cpu_baseline:
        rec["cpu_baseline"] = cpu_stack(2048)
    del layers, xin, ws
    torch.cuda.empty_cache()
    return rec


def adopt_gathered(sharding, full, env):
    """A sharding.GatheredOutput around an existing [total_rows, cols] buffer of this rank (every rank calls this in
    the same order): the buffers are exported, exchanged and mapped exactly as GatheredOutput does for its own."""
    import torch.distributed as dist

    from quant_ops_b200 import _native as nat

    d = sharding.GatheredOutput.__new__(sharding.GatheredOutput)
    d.group, d.world, d.rank, d.full = None, env.world, env.rank, full
    d.start, d.count = sharding.shard_rows(full.shape[0], env.world, env.rank)
    handle = C.create_string_buffer(64)
    offset = C.c_int64()
    nat.check(nat.lib.qo_peer_export(C.c_void_p(full.data_ptr()), handle, C.byref(offset)))
    everyone = [None] * env.world
    dist.all_gather_object(everyone, (handle.raw, int(offset.value)))
    d._handles, d.ptrs = [], []
    for r, (h, off) in enumerate(everyone):
        if r == env.rank:
            d.ptrs.append(full.data_ptr())
        else:
            d.ptrs.append(sharding._open_peer(h) + off)
            d._handles.append(h)
    return d


def cpu_stack(sample):
    """The stack on the host cores over `sample` tokens (time is linear in the token count)."""
    import torch

    from oracle import torch_port
    from oracle import w4a4_oracle as O

    total = 0.0
    g = torch.Generator().manual_seed(SEED + 70)
    for idx, (name, k, n_out) in enumerate(STACK_SHAPES):
        m, n = (64, 64) if k == 4096 else (112, 128)
        left, right = make_transforms(m, n, SEED + 60 + idx)
        x = make_activations(sample, k, SEED + 50)
        wp = torch.randint(-2**31, 2**31 - 1, (n_out, k // 8), generator=g, dtype=torch.int32)
        sw = torch.rand(n_out, generator=g) * 0.01 + 0.001
        total += cpu_time(lambda: torch_port.linear(x, left, right, CLIP, wp, sw), 0, 1)
    return {"value": sample / total, "unit": "tokens/s", "cores": host_cores(), "kind": "port", "ms_per_step": total * 1e3,
            "sample": f"{sample} of the 65,536 tokens through all seven projections, one run (time is linear in tokens); torch CPU ops, {host_cores()} threads"}


# ---------------------------------------------------------------------------------------------------------------
# arms
# ---------------------------------------------------------------------------------------------------------------
def top_level(rec, env_world, args, metric, dtype, scaling, extra_config=None):
    cfg = {"workload": rec.pop("workload")}
    for key in ("l2", "kernel", "gemm_kernel", "parity_vs_oracle_sample", "tokens_per_gpu", "parallelism", "regions", "steps_per_region",
                "ms_per_step_min", "ms_per_step_max", "graph_ms_per_step", "l2_warm_ms_per_step"):
        if key in rec:
            cfg[key] = rec.pop(key)
    if extra_config:
        cfg.update(extra_config)
    if getattr(args, "policy", 0):
        cfg["kernel_policy"] = args.policy
    out = {"metric": metric, "value": rec.pop("value"), "unit": rec.pop("unit"), "n_gpus": env_world, "steps": args.steps,
           "warmup": max(3, args.warmup), "ms_per_step": rec.pop("ms_per_step"), "higher_is_better": True, "scaling": scaling,
           "vs_baseline": None, "dtype": dtype, "data": "synthetic", "config": cfg}
    out.update(rec)
    return out


def run_ours(args):
    env = Env()
    if args.policy:
        env.nat.check(env.lib.qo_set_kernel_policy(args.policy))
    wl = args.workload
    line = None
    if wl in ("all", "quantize"):
        rec = quantizer_record(env, args, TOKENS, M, N_, "quantize", headline=True)
        rec["tokens_per_gpu"] = TOKENS
        line = top_level(rec, env.world, args, "flatquant_quantize_GBps", "bf16", "weak",
                         {"timing": "median of R regions of K steps, each bracketed by barrier + synchronise; max over ranks per region"})
        if wl == "all":
            if env.world == 1:
                line["quantize_wide"] = quantizer_record(env, _sub(args), 4096, 112, 128, "quantize_wide")
                line["dequantize"] = dequantize_record(env, args)
                line["gemm"] = gemm_records(env, args, [4096, 11008, 14336])
                line["linear"] = linear_records(env, args, [1, 16, 256, 4096], [False, True])
            line["stack"] = stack_record(env, args)
            if env.world == 1:
                line["reference_cuda"] = reference_cuda_record()
    elif wl in ("quantize_wide", "quantize_tokens"):
        tokens, m, n = (4096, 112, 128) if wl == "quantize_wide" else (int(args.tokens or 65536), 64, 64)
        rec = quantizer_record(env, args, tokens, m, n, wl, headline=False)
        line = top_level(rec, env.world, args, "flatquant_quantize_GBps", "bf16", "weak")
    elif wl == "gemm":
        a2 = _sub(args, keep=True)
        rec = gemm_records(env, a2, [int(args.n_out or 4096)])[0]
        line = top_level(rec, env.world, args, "int4_matmul_TOPs", "s4 x s4 -> s32 -> f16", "weak")
    elif wl == "linear":
        a2 = _sub(args, keep=True)
        rec = linear_records(env, a2, [int(args.tokens or 16)], [bool(args.prepared)])[0]
        line = top_level(rec, env.world, args, "int4_matmul_TOPs", "bf16 -> s4 x s4 -> s32 -> bf16", "weak")
    elif wl == "stack":
        a2 = _sub(args, keep=True)
        rec = stack_record(env, a2)
        rec.pop("scaling", None)
        line = top_level(rec, env.world, args, "w4a4_stack_tokens_per_s", "bf16 -> s4 x s4 -> s32 -> bf16", "strong")
    if env.rank == 0:
        print(json.dumps(line))
    env.close()


def reference_cuda_record():
    """The reference's own CUDA extensions timed on this GPU by baseline/time_ref_cuda.py, in a process of its own
    (they register the dispatcher namespace the product's binding registers); this process is idle meanwhile."""
    import subprocess

    script = os.path.join(ROOT, "baseline", "time_ref_cuda.py")
    try:
        res = subprocess.run([sys.executable, script], capture_output=True, text=True, timeout=600)
        lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
        if res.returncode != 0 or not lines:
            return {"unavailable": f"time_ref_cuda.py exited {res.returncode}: {res.stderr[-300:]}"}
        return json.loads(lines[-1])
    except Exception as exc:
        return {"unavailable": str(exc)[:300]}


def _sub(args, keep=False):
    """Arguments for a sub-record: its own (smaller) step and repeat counts unless the workload was asked for by name."""
    a = argparse.Namespace(**vars(args))
    if keep:
        a.sub_steps, a.sub_repeats = args.steps, args.repeats
    else:
        a.steps, a.repeats = args.sub_steps, args.sub_repeats
    return a


def run_reference(args):
    """The reference's CPU implementation (torch CPU op chain) on the host cores; rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch

    from oracle import torch_port

    cores = host_cores()
    torch.set_num_threads(cores)
    wl = args.workload
    line = {"impl": "reference", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
            "vs_baseline": None, "data": "synthetic"}

    def finish(value, unit, ms, metric, dtype, scaling, workload, sample):
        line.update({"metric": metric, "value": value, "unit": unit, "ms_per_step": ms, "scaling": scaling, "dtype": dtype,
                     "config": {"workload": workload, "sample": sample},
                     "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
                     "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})

    if wl in ("all", "quantize", "quantize_wide", "quantize_tokens"):
        tokens, m, n = (4096, 112, 128) if wl == "quantize_wide" else ((int(args.tokens or 65536) if wl == "quantize_tokens" else TOKENS), 64, 64)
        x = make_activations(tokens, m * n, SEED)
        left, right = make_transforms(m, n, SEED + 1000)
        for _ in range(max(1, args.warmup)):
            torch_port.quantize(x, left, right, CLIP, True)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            torch_port.quantize(x, left, right, CLIP, True)
        sec = (time.perf_counter() - t0) / args.steps
        finish(quant_bytes(tokens, m, n) / sec / 1e9, "GB/s", sec * 1e3, "flatquant_quantize_GBps", "bf16", "weak",
               f"flatquant_quantize x[{tokens},{m * n}] bf16, 1% outlier channels x50, L {m}x{m} / R {n}x{n} orthogonal, clip {CLIP}, pack_int32",
               f"all {tokens} tokens per step (the same workload as the GPU arm); torch CPU ops, {cores} threads")
        if wl == "all":
            g = torch.Generator().manual_seed(SEED)
            ap = torch.randint(-2**31, 2**31 - 1, (4096, 512), generator=g, dtype=torch.int32)
            wp = torch.randint(-2**31, 2**31 - 1, (4096, 512), generator=g, dtype=torch.int32)
            sa, sw = torch.rand(4096, generator=g), torch.rand(4096, generator=g)
            sec = cpu_time(lambda: torch_port.matmul(ap, wp.t(), sa, sw), 0, 2)
            line["gemm"] = [{"workload": "int4_matmul 4096 x 4096 x 4096", "value": 2.0 * 4096**3 / sec / 1e12, "unit": "TOP/s",
                             "ms_per_step": sec * 1e3, "cores": cores, "sample": "the whole product, min of 2"}]
            line["stack"] = cpu_stack(2048)
    elif wl == "gemm":
        n_out = int(args.n_out or 4096)
        g = torch.Generator().manual_seed(SEED)
        ap = torch.randint(-2**31, 2**31 - 1, (4096, 512), generator=g, dtype=torch.int32)
        wp = torch.randint(-2**31, 2**31 - 1, (n_out, 512), generator=g, dtype=torch.int32)
        sa, sw = torch.rand(4096, generator=g), torch.rand(n_out, generator=g)
        steps = max(1, min(args.steps, 5))
        sec = cpu_time(lambda: torch_port.matmul(ap, wp.t(), sa, sw), min(1, args.warmup), steps)
        finish(2.0 * 4096 * 4096 * n_out / sec / 1e12, "TOP/s", sec * 1e3, "int4_matmul_TOPs", "s4 x s4 -> s32 -> f16", "weak",
               f"int4_matmul T=4096 K=4096 n_out={n_out}", f"the whole product per step, min of {steps} steps; torch CPU ops, {cores} threads")
    elif wl == "linear":
        t = int(args.tokens or 16)
        x = make_activations(t, 14336, SEED + 4 + t)
        left, right = make_transforms(112, 128, SEED + 4)
        g = torch.Generator().manual_seed(SEED)
        wp = torch.randint(-2**31, 2**31 - 1, (4096, 14336 // 8), generator=g, dtype=torch.int32)
        sw = torch.rand(4096, generator=g) * 0.01
        steps = max(1, min(args.steps, 3))
        sec = cpu_time(lambda: torch_port.linear(x, left, right, CLIP, wp, sw), 0, steps)
        finish(2.0 * t * 14336 * 4096 / sec / 1e12, "TOP/s", sec * 1e3, "int4_matmul_TOPs", "bf16 -> s4 x s4 -> s32 -> f16", "weak",
               f"w4a4_linear {t} tokens, 14336 -> 4096", f"the whole layer per step, min of {steps} steps; torch CPU ops, {cores} threads")
    elif wl == "stack":
        rec = cpu_stack(2048)
        finish(rec["value"], "tokens/s", rec["ms_per_step"], "w4a4_stack_tokens_per_s", "bf16 -> s4 x s4 -> s32 -> f16", "strong",
               "Llama-3-8B-shaped W4A4 projection stack, 65,536 tokens", rec["sample"])
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=31, help="timed regions of `steps` steps each; the median is reported")
    ap.add_argument("--sub-steps", type=int, default=10, help="steps per region of the sub-records of `--workload all`")
    ap.add_argument("--sub-repeats", type=int, default=9, help="regions per sub-record of `--workload all`")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="all", choices=["all", "quantize", "quantize_wide", "quantize_tokens", "gemm", "linear", "stack"])
    ap.add_argument("--tokens", type=int, default=None, help="rows of the `linear` (default 16) and `quantize_tokens` (default 65536) workloads")
    ap.add_argument("--n-out", type=int, default=None, help="output channels of the `gemm` workload (default 4096)")
    ap.add_argument("--prepared", action="store_true", help="`linear`: weights also kept widened to int8 (qo_prepare_weights)")
    ap.add_argument("--policy", type=int, default=0, choices=[0, 2, 3],
                    help="kernel selection (qo_set_kernel_policy): 0 automatic, 2 tcgen05 kernels only, 3 tcgen05 kernels "
                         "without the CTA-pair GEMMs (the single-CTA kernels the pair kernels replaced)")
    args = ap.parse_args()
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        # started by hand rather than by torchrun: start one rank per GPU ourselves
        import subprocess

        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.abspath(__file__), *sys.argv[1:]]
        raise SystemExit(subprocess.call(cmd))
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
