"""The Python / torch-dispatcher layer on the GPU: same calls a user of the reference makes."""
import ctypes as C

import numpy as np
import pytest
import torch

import quant_ops_b200 as q
from helpers import N, compare_codes, compare_scales, make_inputs, t2f
from oracle import w4a4_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_quantize_dequantize_matmul_chain():
    x, left, right = make_inputs(200, 4096, "bf16", 31, True)
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    codes, scales = q.flatquant_dynamic_quantize(xd, ld, rd, 0.9, True)
    assert codes.shape == (200, 512) and codes.dtype == torch.int32 and scales.shape == (200,) and scales.dtype == torch.float32
    rc, rs = O.flatquant_quantize(t2f(x), t2f(left), t2f(right), 0.9, True, "bf16")
    compare_scales(t2f(scales), rs)
    compare_codes(O.unpack_int32_to_int4(codes.cpu().numpy()), O.unpack_int32_to_int4(rc))
    c8, s8 = q.flatquant_dynamic_quantize(xd.view(200, 64, 64), ld, rd, 0.9, False)   # [T, M, N] input is accepted
    assert c8.shape == (200, 4096) and c8.dtype == torch.int8
    d_packed = q.dequantize_int4(codes, scales, True)
    d_int8 = q.dequantize_int4(c8, s8, False)
    assert d_packed.dtype == torch.float32 and torch.equal(d_packed, d_int8)          # packing loses nothing
    w = torch.randn(96, 4096, generator=torch.Generator().manual_seed(2)) * 0.02
    wp, sw = q.quantize_weights_int4(w.to(DEV))
    out = q.int4_matmul(codes, wp.t(), scales, sw)
    assert out.shape == (200, 96) and out.dtype == torch.float16
    ref = O.int4_matmul(codes.cpu().numpy(), wp.cpu().numpy().T, t2f(scales), t2f(sw), "fp16")
    np.testing.assert_array_equal(t2f(out), ref)
    fused = q.w4a4_linear(xd, ld, rd, wp, sw, None, 0.9, torch.float16)
    assert torch.equal(fused, out)
    out_bf, acc = q.int4_matmul_ex(codes, wp.t().contiguous(), scales, sw, torch.bfloat16, True)
    np.testing.assert_array_equal(acc.cpu().numpy(), O.int4_accumulators(codes.cpu().numpy(), wp.cpu().numpy().T))
    assert torch.equal(q.unpack_int32_to_int4(q.pack_int4_to_int32(c8)), c8)


def test_errors_are_raised_not_swallowed():
    x, left, right = make_inputs(8, 256, "fp16", 3, False)
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    with pytest.raises(RuntimeError, match="must equal M\\*N"):
        q.flatquant_dynamic_quantize(xd[:, :128], ld, rd)
    with pytest.raises(RuntimeError, match="dtype"):
        q.flatquant_dynamic_quantize(xd, ld.float(), rd)
    with pytest.raises(RuntimeError, match="float32"):
        q.int4_matmul(torch.zeros(2, 4, dtype=torch.int32, device=DEV), torch.zeros(4, 2, dtype=torch.int32, device=DEV),
                      torch.ones(2, device=DEV, dtype=torch.float16), torch.ones(2, device=DEV))
    with pytest.raises(RuntimeError, match="mismatch"):
        q.int4_matmul(torch.zeros(2, 4, dtype=torch.int32, device=DEV), torch.zeros(5, 2, dtype=torch.int32, device=DEV),
                      torch.ones(2, device=DEV), torch.ones(2, device=DEV))


def test_runs_on_a_side_stream_and_in_a_cuda_graph():
    x, left, right = make_inputs(64, 4096, "bf16", 5, True)
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    ref_c, ref_s = q.flatquant_dynamic_quantize(xd, ld, rd, 0.9, True)
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        c, s = q.flatquant_dynamic_quantize(xd, ld, rd, 0.9, True)
    st.synchronize()
    assert torch.equal(c, ref_c) and torch.equal(s, ref_s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        gc, gs = q.flatquant_dynamic_quantize(xd, ld, rd, 0.9, True)
    xd.copy_(torch.roll(xd, 1, 0))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(gc, torch.roll(ref_c, 1, 0)) and torch.equal(gs, torch.roll(ref_s, 1, 0))


def test_w4a4_linear_module_matches_the_two_step_path():
    """The layer object (load-time weight packing, any leading dimensions, bias, output in the input dtype)."""
    x, left, right = make_inputs(48, 4096, "bf16", 77, True)
    g = torch.Generator().manual_seed(8)
    w = torch.randn(256, 4096, generator=g) * 0.02
    bias = (torch.randn(256, generator=g) * 0.1).bfloat16()
    layer = q.W4A4Linear(4096, 256, bias=True, clip_ratio=0.9, dtype=torch.bfloat16, device=DEV)
    layer.load_float(w, left.to(DEV), right.to(DEV), bias.to(DEV))
    y = layer(x.to(DEV).view(4, 12, 4096))
    assert y.shape == (4, 12, 256) and y.dtype == torch.bfloat16
    codes, scales = q.flatquant_dynamic_quantize(x.to(DEV), left.to(DEV), right.to(DEV), 0.9, True)
    ref = q.int4_matmul_ex(codes, layer.weight_packed.t(), scales, layer.weight_scale, torch.bfloat16)
    ref = (ref.float() + bias.to(DEV).float()).bfloat16()
    assert torch.equal(y.view(48, 256), ref)
    # the same weights loaded as int8 codes + scales (the reference's checkpoint layout) give the same layer
    wq, sw = O.quantize_weights(w.numpy())
    layer2 = q.W4A4Linear(4096, 256, bias=True, clip_ratio=0.9, dtype=torch.bfloat16, device=DEV)
    layer2.load_quantized(torch.from_numpy(wq), torch.from_numpy(sw), left.to(DEV), right.to(DEV), bias.to(DEV))
    assert torch.equal(layer2.weight_packed, layer.weight_packed) and torch.equal(layer2(x.to(DEV)), y.view(48, 256))


@pytest.mark.parametrize("tokens,k,n_out", [(1, 4096, 256), (32, 4096, 512), (33, 4096, 256), (200, 14336, 512), (256, 4096, 4096),
                                             (1100, 4096, 512)])
def test_prepared_weights_give_identical_results(tokens, k, n_out):
    """The layer with an int8 copy of its weights (no per-call widening of either operand) against the plain fused op:
    few tokens (packed-weight route), K-split shapes and plain tiles."""
    x, left, right = make_inputs(tokens, k, "bf16", 5 * tokens + n_out, True)
    g = torch.Generator().manual_seed(tokens)
    w = torch.randn(n_out, k, generator=g) * 0.02
    bias = (torch.randn(n_out, generator=g) * 0.1).bfloat16().to(DEV)
    plain = q.W4A4Linear(k, n_out, bias=True, clip_ratio=0.9, dtype=torch.bfloat16, device=DEV)
    plain.load_float(w, left.to(DEV), right.to(DEV), bias)
    kept = q.W4A4Linear(k, n_out, bias=True, clip_ratio=0.9, dtype=torch.bfloat16, device=DEV, keep_int8_weights=True)
    kept.load_float(w, left.to(DEV), right.to(DEV), bias)
    # the kept copy is the GEMM's int8 operand: blocks of 256 output channels x 128 values, ordered [n_out/256][k/128]
    nb, ks = (n_out + 255) // 256, (k + 127) // 128
    assert kept.weight_int8 is not None and kept.weight_int8.shape == (nb * ks * 256 * 128,)
    rows = kept.weight_int8.view(torch.int8).view(nb, ks, 256, 128).permute(0, 2, 1, 3).reshape(nb * 256, ks * 128)
    assert torch.equal(rows[:n_out, :k], q.unpack_int32_to_int4(kept.weight_packed))
    y0, y1 = plain(x.to(DEV)), kept(x.to(DEV))
    assert torch.equal(y0, y1)
    assert N.lib.qo_device_status(C.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0


def test_layer_against_the_float_simulation():
    """End-to-end accuracy cross-check: W4A4Linear on the GPU vs the restated fake-quant layer of the reference."""
    tokens, k, n_out = 64, 4096, 320
    x, left, right = make_inputs(tokens, k, "bf16", 4242, True)
    g = torch.Generator().manual_seed(11)
    w = torch.randn(n_out, k, generator=g) * 0.02
    wq, sw = O.quantize_weights(w.numpy())
    layer = q.W4A4Linear(k, n_out, clip_ratio=0.9, dtype=torch.bfloat16, device=DEV)
    layer.load_quantized(torch.from_numpy(wq), torch.from_numpy(sw), left.to(DEV), right.to(DEV))
    y = layer(x.to(DEV)).float().cpu().numpy()
    sim = O.fake_quant_linear(t2f(x), t2f(left), t2f(right), 0.9, wq, sw, "bf16")
    bound = 2e-2 * np.abs(sim).max(axis=1, keepdims=True)
    assert np.all(np.abs(y - sim) <= bound), float((np.abs(y - sim) / bound).max())


def _layer_inputs(tokens, k, n_out, seed):
    x, left, right = make_inputs(tokens, k, "bf16", seed, True)
    w = torch.randn(n_out, k, generator=torch.Generator().manual_seed(seed + 1)) * 0.02
    wp, sw = q.quantize_weights_int4(w.to(DEV))
    return x.to(DEV), left.to(DEV), right.to(DEV), wp, sw


@pytest.mark.parametrize("tokens", [8, 200])
def test_gemm_and_fused_layer_in_a_cuda_graph(tokens):
    """int4_matmul and w4a4_linear (both GEMM kernels: weight-streaming and tensor-core) captured and replayed on new
    data: launches go to the capturing stream, nothing synchronises, the workspace comes from the graph's pool."""
    xd, ld, rd, wp, sw = _layer_inputs(tokens, 4096, 512, 100 + tokens)
    codes, scales = q.flatquant_dynamic_quantize(xd, ld, rd, 0.9, True)
    ref_mm = q.int4_matmul(codes, wp.t(), scales, sw)
    ref_lin = q.w4a4_linear(xd, ld, rd, wp, sw, None, 0.9, torch.bfloat16)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        g_codes, g_scales = q.flatquant_dynamic_quantize(xd, ld, rd, 0.9, True)
        g_mm = q.int4_matmul(g_codes, wp.t(), g_scales, sw)
        g_lin = q.w4a4_linear(xd, ld, rd, wp, sw, None, 0.9, torch.bfloat16)
    xd.copy_(torch.roll(xd, 3, 0))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(g_mm, torch.roll(ref_mm, 3, 0)) and torch.equal(g_lin, torch.roll(ref_lin, 3, 0))
    q.device_status()


@pytest.mark.parametrize("backend", ["aot_eager", "inductor"])
def test_ops_trace_under_torch_compile(backend):
    """quantize -> int4_matmul and the W4A4Linear module compiled as one graph (fullgraph=True: a graph break would
    raise): the dispatcher ops and their fake kernels carry the trace, as the reference's registration intends
    (src/quant_ops/ops/quantization/flatquant/kernels/cuda_quant_kernel.cu:393-417, src/quant_ops/meta_ops.py:22-37)."""
    xd, ld, rd, wp, sw = _layer_inputs(96, 4096, 256, 7)

    def chain(x, left, right, w, s):
        codes, scales = q.flatquant_dynamic_quantize(x, left, right, 0.9, True)
        return q.int4_matmul(codes, w.t(), scales, s), q.dequantize_int4(codes, scales, True)

    want_out, want_deq = chain(xd, ld, rd, wp, sw)
    got_out, got_deq = torch.compile(chain, fullgraph=True, backend=backend)(xd, ld, rd, wp, sw)
    assert torch.equal(got_out, want_out) and torch.equal(got_deq, want_deq)

    layer = q.W4A4Linear(4096, 256, clip_ratio=0.9, dtype=torch.bfloat16, device=DEV)
    layer.weight_packed.copy_(wp)
    layer.weight_scale.copy_(sw)
    layer.left_trans.copy_(ld)
    layer.right_trans.copy_(rd)
    want = layer(xd.view(8, 12, 4096))
    got = torch.compile(layer, fullgraph=True, backend=backend)(xd.view(8, 12, 4096))
    assert got.shape == (8, 12, 256) and torch.equal(got, want)
    q.device_status()


def test_scale_dtype_keyword_and_device_status():
    """The 2-byte scale store is reachable from Python; the values are the float32 scales (bf16 inputs give bf16 values)."""
    x, left, right = make_inputs(40, 4096, "bf16", 12, True)
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    c32, s32 = q.flatquant_dynamic_quantize(xd, ld, rd, 0.9, True)
    cb, sb = q.flatquant_dynamic_quantize(xd, ld, rd, 0.9, True, scale_dtype=torch.bfloat16)
    assert sb.dtype == torch.bfloat16 and torch.equal(cb, c32) and torch.equal(sb.float(), s32)
    ch, sh = q.flatquant_dynamic_quantize(xd, ld, rd, 0.9, True, scale_dtype=torch.float16)
    assert sh.dtype == torch.float16 and torch.equal(ch, c32) and torch.equal(sh, s32.half())
    assert torch.equal(q.dequantize_int4(cb, sb, True), q.dequantize_int4(c32, s32, True))
    q.device_status()
