"""GPU parity of the packed-int4 GEMM, dequantize, pack/unpack, weight quantizer and the fused layer (C ABI)."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import (N, QD, abi_int4_matmul, abi_quantize, bits_to_f32, bits_to_torch, golden, lib, make_inputs, ptr,
                     stream_ptr, t2f)
from oracle import w4a4_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rand_problem(t, k, n, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-8, 8, (t, k), generator=g, dtype=torch.int8)
    w = torch.randint(-8, 8, (n, k), generator=g, dtype=torch.int8)  # weight layout [n_out, K]
    sa = torch.rand(t, generator=g) * 0.1 + 0.01
    sb = torch.rand(n, generator=g) * 0.1 + 0.01
    ap = torch.from_numpy(O.pack_int4_to_int32(a.numpy()))
    wp = torch.from_numpy(O.pack_int4_to_int32(w.numpy()))  # [n, K/8]
    return a, w, ap, wp, sa, sb


def both_policies(fn):
    """Runs fn(policy) for the generic kernel and, where the shape has one, the tcgen05 kernel."""
    yield "generic", fn(1)
    try:
        res = fn(2)
    except N.QuantOpsError as e:
        assert e.status == N.QO_ERR_UNSUPPORTED
        return
    assert lib.qo_device_status(stream_ptr()) == N.QO_OK, lib.qo_last_error()
    yield "tcgen05", res
    res = fn(3)  # the same without the CTA-pair kernels: the single-CTA tcgen05 kernels keep their coverage
    assert lib.qo_device_status(stream_ptr()) == N.QO_OK, lib.qo_last_error()
    yield "tcgen05, single CTA", res


@pytest.mark.parametrize("name", ["gemm_64x512x96", "gemm_33x256x40"])
def test_against_reference_fixtures(name):
    g = golden(name)
    a, b = torch.from_numpy(g["a_packed"]).to(DEV), torch.from_numpy(g["b_packed"]).to(DEV)
    sa, sb = torch.from_numpy(g["scale_a"]).to(DEV), torch.from_numpy(g["scale_b"]).to(DEV)
    for label, (out, acc) in both_policies(lambda p: abi_int4_matmul(a, b, sa, sb, "fp16", True, policy=p)):
        np.testing.assert_array_equal(acc.cpu().numpy(), g["acc"], err_msg=label)
        np.testing.assert_array_equal(t2f(out), bits_to_f32(g["out_bits"], "fp16"), err_msg=label)


SHAPES = [(1, 64, 8), (1, 4096, 4096), (16, 14336, 512), (128, 256, 256), (129, 1000 * 8, 130), (300, 4096, 520),
          (1024, 1024, 1024), (256, 14336, 4096), (77, 8, 5),
          # the two-accumulator kernel: long K with ragged tiles, many tiles
          (2200, 8192, 4104), (4096, 512, 9472),
          # 512 tiles of 128 x 256 on 148 SMs, exact and with a ragged last column tile
          (4096, 256, 4096), (4096, 256, 3848),
          # K split over several CTAs per tile: 8 slices of 3 tiles, 2 slices of 8 ragged tiles
          (64, 8192, 768), (200, 2048, 1000), (100, 4096, 1000),
          # CTA-pair kernel that unpacks in the kernel: short K with many tiles per pair (the epilogue is the slower side),
          # a K that is no multiple of 128 (falls back to the widening path), ragged rows and columns
          (4096, 1024, 9472), (4096, 384, 9472), (3900, 4096, 4104), (4096, 1000 * 8, 4096)]


@pytest.mark.parametrize("t,k,n", SHAPES)
@pytest.mark.parametrize("layout", ["weights_t_view", "reference_contiguous"])
def test_accumulators_bit_exact_and_outputs(t, k, n, layout):
    a, w, ap, wp, sa, sb = rand_problem(t, k, n, t * 7 + k + n)
    acc_ref = O.int4_accumulators(ap.numpy(), wp.numpy().T)
    apd, sad, sbd = ap.to(DEV), sa.to(DEV), sb.to(DEV)
    bd = wp.to(DEV).t() if layout == "weights_t_view" else wp.to(DEV).t().contiguous()
    for out_dtype in ("fp16", "bf16"):
        ref = O.round_to((acc_ref.astype(np.float32) * sa.numpy()[:, None]) * sb.numpy()[None, :], out_dtype)
        for label, (out, acc) in both_policies(lambda p: abi_int4_matmul(apd, bd, sad, sbd, out_dtype, True, policy=p)):
            np.testing.assert_array_equal(acc.cpu().numpy(), acc_ref, err_msg=f"{label} accumulators")
            np.testing.assert_array_equal(t2f(out), ref, err_msg=f"{label} outputs")


SKINNY = [(1, 128, 16), (1, 4096, 4096), (5, 14336, 100), (8, 4096, 48), (9, 11008, 256), (16, 14336, 4096), (17, 256, 33),
          (32, 4096, 512),
          # staged activations above 92 KB: 32 channels per CTA share one copy (static + dynamic shared memory near the limit)
          (32, 8192, 256), (24, 14336, 256), (32, 11008, 256),
          # activations that do not fit at all are read through the caches
          (32, 14336, 64)]


@pytest.mark.parametrize("t,k,n", SKINNY)
def test_weight_streaming_kernel_for_few_rows(t, k, n):
    """Automatic policy sends 1..32 rows against K-contiguous weights to the weight-streaming kernel."""
    a, w, ap, wp, sa, sb = rand_problem(t, k, n, 3 * t + k + 5 * n)
    acc_ref = O.int4_accumulators(ap.numpy(), wp.numpy().T)
    apd, bd, sad, sbd = ap.to(DEV), wp.to(DEV).t(), sa.to(DEV), sb.to(DEV)
    for out_dtype in ("fp16", "bf16"):
        ref = O.round_to((acc_ref.astype(np.float32) * sa.numpy()[:, None]) * sb.numpy()[None, :], out_dtype)
        out, acc = abi_int4_matmul(apd, bd, sad, sbd, out_dtype, True, policy=0)
        assert lib.qo_last_gemm_path() == 3
        np.testing.assert_array_equal(acc.cpu().numpy(), acc_ref)
        np.testing.assert_array_equal(t2f(out), ref)
    # extreme codes: every product is (-8) * (-8)
    zeros_a = torch.zeros((t, k // 8), dtype=torch.int32, device=DEV)
    zeros_w = torch.zeros((n, k // 8), dtype=torch.int32, device=DEV)
    out, acc = abi_int4_matmul(zeros_a, zeros_w.t(), sad, sbd, "fp16", True, policy=0)
    assert int(acc.min()) == int(acc.max()) == 64 * k
    # rows that are views with a larger stride
    wide = torch.zeros((t, k // 8 + 4), dtype=torch.int32, device=DEV)
    wide[:, : k // 8] = apd
    out2, acc2 = abi_int4_matmul(wide[:, : k // 8], bd, sad, sbd, "fp16", True, policy=0)
    np.testing.assert_array_equal(acc2.cpu().numpy(), acc_ref)


def test_extreme_codes_do_not_overflow():
    t, k, n = 64, 14336, 64
    ap = torch.full((t, k // 8), 0, dtype=torch.int32)          # all nibbles 0 -> code -8
    wp = torch.full((n, k // 8), 0, dtype=torch.int32)
    one = torch.ones(max(t, n))
    for label, (out, acc) in both_policies(lambda p: abi_int4_matmul(ap.to(DEV), wp.to(DEV).t(), one[:t].to(DEV) * 1e-3,
                                                                     one[:n].to(DEV) * 1e-3, "fp16", True, policy=p)):
        assert int(acc.min()) == int(acc.max()) == 64 * k


def test_library_owned_workspace_and_too_small_workspace():
    a, w, ap, wp, sa, sb = rand_problem(256, 4096, 256, 5)
    apd, bd, sad, sbd = ap.to(DEV), wp.to(DEV).t(), sa.to(DEV), sb.to(DEV)
    ref = abi_int4_matmul(apd, bd, sad, sbd, "fp16")
    got = abi_int4_matmul(apd, bd, sad, sbd, "fp16", use_workspace=False)
    assert torch.equal(ref, got)
    need = lib.qo_int4_matmul_workspace_bytes(256, 4096, 256)
    if need:
        small = torch.empty(16, dtype=torch.uint8, device=DEV)
        out = torch.empty(256, 256, dtype=torch.float16, device=DEV)
        rc = lib.qo_int4_matmul(ptr(apd), 512, ptr(bd), bd.stride(0), bd.stride(1), ptr(sad), ptr(sbd), ptr(out), N.QO_F16,
                                256, 4096, 256, None, ptr(small), 16, stream_ptr())
        assert rc == N.QO_ERR_WORKSPACE


@pytest.mark.parametrize("n_out", [4096, 11008, 14336])
def test_gemm_on_quantizer_output_full_size(n_out):
    """T = K = 4096 with A produced by the quantizer and n_out swept over the three projection widths: exact
    accumulators and outputs on sampled rows, linearity in the scales."""
    x, left, right = make_inputs(4096, 4096, "bf16", 20242, True)
    aq, sa = abi_quantize(x.to(DEV), left.to(DEV), right.to(DEV), 0.9, True, "bf16")
    g = torch.Generator().manual_seed(20243)
    w = torch.randn(n_out, 4096, generator=g) * 0.02
    wq, sw = O.quantize_weights(w.numpy())
    wp = torch.from_numpy(O.pack_int4_to_int32(wq)).to(DEV)
    swd = torch.from_numpy(sw).to(DEV)
    out, acc = abi_int4_matmul(aq, wp.t(), sa, swd, "fp16", True)
    assert lib.qo_last_gemm_path() == 2 and lib.qo_device_status(stream_ptr()) == N.QO_OK
    rows = np.random.default_rng(1).choice(4096, 96, replace=False)
    acc_ref = O.int4_accumulators(aq.cpu().numpy()[rows], wp.cpu().numpy().T)
    np.testing.assert_array_equal(acc.cpu().numpy()[rows], acc_ref)
    ref = O.round_to((acc_ref.astype(np.float32) * t2f(sa)[rows, None]) * sw[None, :], "fp16")
    np.testing.assert_array_equal(t2f(out)[rows], ref)
    out2 = abi_int4_matmul(aq, wp.t(), sa * 2, swd, "fp16")
    np.testing.assert_allclose(t2f(out2), 2 * t2f(out), rtol=2e-3, atol=1e-6)
    # EVERY accumulator and output of the full product: float32 sums of integer products below 2^24 are exact in any
    # order, so a float32 matmul of the unpacked codes (no TF32) is an exact integer reference at full size
    assert not torch.backends.cuda.matmul.allow_tf32
    sh = torch.arange(8, device=DEV, dtype=torch.int32) * 4
    a_codes = (((aq[:, :, None] >> sh) & 15) - 8).reshape(4096, 4096).float()
    w_codes = (((wp[:, :, None] >> sh) & 15) - 8).reshape(n_out, 4096).float()
    acc_all = a_codes @ w_codes.t()
    assert torch.equal(acc.float(), acc_all)
    assert torch.equal(out, ((acc_all * sa[:, None]) * swd[None, :]).half())


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("scale_dtype", ["fp32", "bf16", "fp16"])
def test_dequantize(packed, scale_dtype):
    g = torch.Generator().manual_seed(4)
    codes = torch.randint(-8, 8, (37, 1024), generator=g, dtype=torch.int8)
    scales = (torch.rand(37, generator=g) + 0.01).to({"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[scale_dtype])
    q = torch.from_numpy(O.pack_int4_to_int32(codes.numpy())) if packed else codes
    out = torch.empty(37, 1024, device=DEV)
    qd, sd = q.to(DEV), scales.to(DEV)  # keep the device buffers alive across the call
    N.check(lib.qo_dequantize_int4(ptr(qd), ptr(sd), ptr(out), 37, 1024, int(packed), QD[scale_dtype], stream_ptr()))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(out.cpu().numpy(), O.dequantize_int4(q.numpy(), t2f(scales), packed))


def test_dequantize_reference_fixture_and_odd_width():
    g = golden("quant_bf16_4096_packed")
    out = torch.empty(2, 4096, device=DEV)
    cd, sd = torch.from_numpy(g["codes"][:2].copy()).to(DEV), torch.from_numpy(g["scales"][:2].copy()).to(DEV)
    N.check(lib.qo_dequantize_int4(ptr(cd), ptr(sd), ptr(out), 2, 4096, 1, N.QO_F32, stream_ptr()))
    np.testing.assert_array_equal(out.cpu().numpy(), g["dequant_head"])
    codes = torch.randint(-8, 8, (5, 15), dtype=torch.int8)
    s = torch.rand(5) + 0.5
    out = torch.empty(5, 15, device=DEV)
    cd, sd = codes.to(DEV), s.to(DEV)
    N.check(lib.qo_dequantize_int4(ptr(cd), ptr(sd), ptr(out), 5, 15, 0, N.QO_F32, stream_ptr()))
    np.testing.assert_array_equal(out.cpu().numpy(), O.dequantize_int4(codes.numpy(), s.numpy(), False))


def test_pack_unpack_and_weight_quantizer():
    g = torch.Generator().manual_seed(6)
    codes = torch.randint(-8, 8, (100, 4096), generator=g, dtype=torch.int8)
    packed = torch.empty(100, 512, dtype=torch.int32, device=DEV)
    codes_d = codes.to(DEV)
    N.check(lib.qo_pack_int4(ptr(codes_d), ptr(packed), 100, 4096, stream_ptr()))
    np.testing.assert_array_equal(packed.cpu().numpy(), O.pack_int4_to_int32(codes.numpy()))
    back = torch.empty(100, 4096, dtype=torch.int8, device=DEV)
    N.check(lib.qo_unpack_int4(ptr(packed), ptr(back), 100, 4096, stream_ptr()))
    assert torch.equal(back.cpu(), codes)
    w = torch.randn(300, 1024, generator=g) * 0.02
    w[7] = 0
    wp = torch.empty(300, 128, dtype=torch.int32, device=DEV)
    sw = torch.empty(300, device=DEV)
    w_d = w.to(DEV)
    N.check(lib.qo_quantize_weights_int4(ptr(w_d), ptr(wp), ptr(sw), 300, 1024, stream_ptr()))
    wq_ref, sw_ref = O.quantize_weights(w.numpy())
    np.testing.assert_array_equal(sw.cpu().numpy(), sw_ref)
    np.testing.assert_array_equal(O.unpack_int32_to_int4(wp.cpu().numpy()), wq_ref)


def abi_linear(x, left, right, wp, sw, bias, clip, dtype, out_dtype):
    tokens, k = x.shape
    n_out = wp.shape[0]
    out = torch.empty(tokens, n_out, dtype={"fp16": torch.float16, "bf16": torch.bfloat16}[out_dtype], device=DEV)
    need = lib.qo_w4a4_linear_workspace_bytes(tokens, k, n_out)
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    N.check(lib.qo_w4a4_linear(ptr(x), x.stride(0), ptr(left), ptr(right), ptr(wp), ptr(sw), ptr(bias), ptr(out), tokens,
                               left.shape[0], right.shape[0], n_out, clip, QD[dtype], QD[out_dtype], ptr(ws), need, stream_ptr()))
    torch.cuda.synchronize()
    return out


def test_fused_layer_reference_fixture():
    g = golden("linear_bf16_1024x48")
    x, left, right = (bits_to_torch(g[k], "bf16").to(DEV) for k in ("x", "left", "right"))
    out = abi_linear(x, left, right, torch.from_numpy(g["w_packed"]).to(DEV), torch.from_numpy(g["w_scale"]).to(DEV), None,
                     float(g["clip"]), "bf16", "fp16")
    aq, sa = abi_quantize(x, left, right, float(g["clip"]), True, "bf16")
    assert_layer_close(t2f(out), bits_to_f32(g["out_bits"], "fp16"), O.unpack_int32_to_int4(aq.cpu().numpy()),
                       O.unpack_int32_to_int4(g["a_packed"]), t2f(sa), g["a_scale"])


def assert_layer_close(got, ref, codes_got=None, codes_ref=None, scales_got=None, scales_ref=None):
    """|got - ref| <= 1e-2 * max(|ref|, row range), for every output.

    Why the row range: a +-1 code flip (allowed on at most 0.1 % of the codes, where the tensor cores' summation order
    moves a value across a rounding boundary) shifts every output of its row by up to |w_j| * scale_a * scale_w, a few
    thousandths of the row's range, so an output near zero is measured against the range rather than against itself.
    With codes and scales of both sides at hand, rows that agree in both must also agree in every output bit for bit
    (the GEMM is exact), and the only rows that may miss the bound are those whose SCALE differs by one unit in the last
    place of the 16-bit format (the token's absmax sat on a rounding boundary; about 1 % of such a row's codes move
    with it) -- at most 0.1 % of the rows."""
    scale = np.abs(ref).max(axis=1, keepdims=True)
    ok = np.abs(got - ref) <= 1e-2 * np.maximum(np.abs(ref), scale)
    if codes_got is None:
        assert ok.all(), f"{(~ok).sum()} outputs outside 1e-2 of the row range"
        return
    same_scale = scales_got == scales_ref
    same = (codes_got == codes_ref).all(axis=1) & same_scale
    np.testing.assert_array_equal(got[same], ref[same])
    assert ok[same_scale].all(), "an output of a row with the oracle's scale is outside the bound"
    assert (~same_scale).sum() <= max(1, len(same) // 1000), f"{(~same_scale).sum()} rows with a different scale"
    assert ok[~same_scale].mean() > 0.99 if (~same_scale).any() else True


@pytest.mark.parametrize("tokens", [1, 16, 256, 4096])
def test_fused_layer_down_proj_shape(tokens):
    """The fused layer at the down-projection shape (14336 -> 4096), decode to prefill: against the oracle (all rows up to
    256 tokens, 64 sampled rows at 4096) and bit-equal to quantize -> GEMM through the two separate entry points."""
    x, left, right = make_inputs(tokens, 14336, "bf16", 20244 + tokens, True)
    g = torch.Generator().manual_seed(20245)
    w = torch.randn(4096, 14336, generator=g) * 0.02
    wq, sw = O.quantize_weights(w.numpy())
    wp = O.pack_int4_to_int32(wq)
    bias = (torch.randn(4096, generator=g) * 0.1).bfloat16()
    wpd, swd = torch.from_numpy(wp).to(DEV), torch.from_numpy(sw).to(DEV)
    out = abi_linear(x.to(DEV), left.to(DEV), right.to(DEV), wpd, swd, bias.to(DEV), 0.9, "bf16", "bf16")
    assert lib.qo_device_status(stream_ptr()) == N.QO_OK, lib.qo_last_error()
    rows = np.arange(tokens) if tokens <= 256 else np.sort(np.random.default_rng(3).choice(tokens, 64, replace=False))
    # oracle with its own codes checks the whole layer
    rc, rs = O.flatquant_quantize(t2f(x)[rows], t2f(left), t2f(right), 0.9, True, "bf16")
    ref = O.round_to(O.int4_matmul(rc, wp.T, rs, sw, "bf16") + t2f(bias)[None, :], "bf16")
    got = t2f(out)
    aq, sa = abi_quantize(x.to(DEV), left.to(DEV), right.to(DEV), 0.9, True, "bf16")
    assert_layer_close(got[rows], ref, O.unpack_int32_to_int4(aq.cpu().numpy()[rows]), O.unpack_int32_to_int4(rc),
                       t2f(sa)[rows], rs)
    # the GEMM in isolation: the two-call path on the GPU's own codes must give the same bits, and so must the oracle
    two_call = abi_int4_matmul(aq, wpd.t(), sa, swd, "bf16")
    two_call = (two_call.float() + bias.to(DEV).float()).bfloat16()
    assert torch.equal(out, two_call)
    exact = O.round_to(O.int4_matmul(aq.cpu().numpy()[rows], wp.T, t2f(sa)[rows], sw, "bf16") + t2f(bias)[None, :], "bf16")
    np.testing.assert_array_equal(got[rows], exact)


@pytest.mark.parametrize("n_out", [4096, 1024 + 4096])
def test_gather_variant_writes_this_ranks_rows_into_every_destination(n_out):
    """qo_w4a4_linear_gather with two destination buffers on this GPU standing in for two ranks' buffers: rows
    row_offset .. row_offset + tokens of BOTH hold the bits of the plain fused layer, every other row is untouched.
    (Mapping another process's buffer is exercised by the multi-GPU benchmark; the kernel sees plain pointers.)"""
    tokens, k, total, row_offset = 2048, 4096, 5000, 1111
    x, left, right = make_inputs(tokens, k, "bf16", 20270, True)
    g = torch.Generator().manual_seed(20271)
    wq, sw = O.quantize_weights((torch.randn(n_out, k, generator=g) * 0.02).numpy())
    wpd, swd = torch.from_numpy(O.pack_int4_to_int32(wq)).to(DEV), torch.from_numpy(sw).to(DEV)
    bias = (torch.randn(n_out, generator=g) * 0.1).bfloat16().to(DEV)
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    want = abi_linear(xd, ld, rd, wpd, swd, bias, 0.9, "bf16", "bf16")
    dsts = [torch.full((total, n_out), -7.0, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    arr = (C.c_void_p * 2)(*[d.data_ptr() for d in dsts])
    N.check(lib.qo_w4a4_linear_gather(ptr(xd), xd.stride(0), ptr(ld), ptr(rd), ptr(wpd), ptr(swd), ptr(bias), arr, 2, row_offset, tokens,
                                      left.shape[0], right.shape[0], n_out, 0.9, QD["bf16"], QD["bf16"], None, 0, stream_ptr()))
    assert lib.qo_device_status(stream_ptr()) == N.QO_OK, lib.qo_last_error()
    for d in dsts:
        assert torch.equal(d[row_offset:row_offset + tokens], want)
        assert bool((d[:row_offset] == -7.0).all()) and bool((d[row_offset + tokens:] == -7.0).all())
    # a decode-sized call has no fused gather: the caller is told, nothing is written
    rc = lib.qo_w4a4_linear_gather(ptr(xd), xd.stride(0), ptr(ld), ptr(rd), ptr(wpd), ptr(swd), ptr(bias), arr, 2, 0, 16,
                                   left.shape[0], right.shape[0], n_out, 0.9, QD["bf16"], QD["bf16"], None, 0, stream_ptr())
    assert rc == N.QO_ERR_UNSUPPORTED and b"prefill" in lib.qo_last_error()


def abi_linear_prepared(x, left, right, wp, w8, sw, bias, clip, dtype, out_dtype):
    tokens, k = x.shape
    n_out = wp.shape[0]
    out = torch.empty(tokens, n_out, dtype={"fp16": torch.float16, "bf16": torch.bfloat16}[out_dtype], device=DEV)
    need = lib.qo_w4a4_linear_prepared_workspace_bytes(tokens, k, n_out)
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    N.check(lib.qo_w4a4_linear_prepared(ptr(x), x.stride(0), ptr(left), ptr(right), ptr(wp), ptr(w8), ptr(sw), ptr(bias), ptr(out),
                                        tokens, left.shape[0], right.shape[0], n_out, clip, QD[dtype], QD[out_dtype], ptr(ws), need,
                                        stream_ptr()))
    torch.cuda.synchronize()
    return out


def test_prepared_layer_at_prefill_size_matches_the_plain_layer():
    """4096 tokens, 14336 -> 4096: the layer with weights kept as int8 (the route into the two-accumulator GEMM) gives
    the bits of the plain fused layer."""
    x, left, right = make_inputs(4096, 14336, "bf16", 20260, True)
    g = torch.Generator().manual_seed(20261)
    wq = torch.randint(-8, 8, (4096, 14336), generator=g, dtype=torch.int8)
    wpd = torch.from_numpy(O.pack_int4_to_int32(wq.numpy())).to(DEV)
    swd = (torch.rand(4096, generator=g) * 0.01 + 0.001).to(DEV)
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    w8 = torch.empty(lib.qo_prepared_weights_bytes(4096, 14336), dtype=torch.uint8, device=DEV)
    N.check(lib.qo_prepare_weights(ptr(wpd), ptr(w8), 4096, 14336, stream_ptr()))
    plain = abi_linear(xd, ld, rd, wpd, swd, None, 0.9, "bf16", "bf16")
    kept = abi_linear_prepared(xd, ld, rd, wpd, w8, swd, None, 0.9, "bf16", "bf16")
    assert lib.qo_device_status(stream_ptr()) == N.QO_OK, lib.qo_last_error()
    assert torch.equal(plain, kept)


STACK = [("q", 4096, 4096), ("k", 4096, 1024), ("v", 4096, 1024), ("o", 4096, 4096), ("gate", 4096, 14336), ("up", 4096, 14336),
         ("down", 14336, 4096)]


@pytest.mark.parametrize("name,k,n_out", STACK)
def test_projection_stack_slice_against_the_oracle(name, k, n_out):
    """The seven projections of the Llama-3-8B-shaped stack on one rank's slice of the tokens (rows 3 * 8192 .. of
    65,536 split over 8 ranks; 2048 of its rows are computed here), with per-layer random-orthogonal L / R and weights
    quantized per output channel from N(0, 0.02): the fused layer, plain and with prepared weights, against the
    oracle on sampled rows; the two forms bit-equal on all rows."""
    from quant_ops_b200 import sharding

    start, count = sharding.shard_rows(65536, 8, 3)
    assert (start, count) == (24576, 8192)
    tokens = 2048
    seed = 20250 + sum(map(ord, name))
    x, left, right = make_inputs(tokens, k, "bf16", seed, True)
    g = torch.Generator().manual_seed(seed + 1)
    w = torch.randn(n_out, k, generator=g) * 0.02
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    wpd = torch.empty(n_out, k // 8, dtype=torch.int32, device=DEV)
    swd = torch.empty(n_out, device=DEV)
    wd = w.to(DEV)
    N.check(lib.qo_quantize_weights_int4(ptr(wd), ptr(wpd), ptr(swd), n_out, k, stream_ptr()))
    wq_ref, sw_ref = O.quantize_weights(w.numpy())
    np.testing.assert_array_equal(swd.cpu().numpy(), sw_ref)
    wp = O.pack_int4_to_int32(wq_ref)
    np.testing.assert_array_equal(wpd.cpu().numpy(), wp)
    w8 = torch.empty(lib.qo_prepared_weights_bytes(n_out, k), dtype=torch.uint8, device=DEV)
    N.check(lib.qo_prepare_weights(ptr(wpd), ptr(w8), n_out, k, stream_ptr()))
    plain = abi_linear(xd, ld, rd, wpd, swd, None, 0.9, "bf16", "bf16")
    kept = abi_linear_prepared(xd, ld, rd, wpd, w8, swd, None, 0.9, "bf16", "bf16")
    assert lib.qo_device_status(stream_ptr()) == N.QO_OK, lib.qo_last_error()
    assert torch.equal(plain, kept)
    rows = np.sort(np.random.default_rng(seed).choice(tokens, 48, replace=False))
    rc, rs = O.flatquant_quantize(t2f(x)[rows], t2f(left), t2f(right), 0.9, True, "bf16")
    ref = O.int4_matmul(rc, wp.T, rs, sw_ref, "bf16")
    aq, sa = abi_quantize(xd, ld, rd, 0.9, True, "bf16")
    assert_layer_close(t2f(kept)[rows], ref, O.unpack_int32_to_int4(aq.cpu().numpy()[rows]), O.unpack_int32_to_int4(rc),
                       t2f(sa)[rows], rs)


@pytest.mark.parametrize("tokens,k,n_out", [(1, 4096, 4096), (7, 4096, 14336), (16, 4096, 1024), (20, 14336, 4096), (32, 4096, 11008), (3, 4096, 200)])
def test_fused_layer_decode_shapes(tokens, k, n_out):
    """Decode-sized fused layer over the projection shapes: inside the layer the GEMM keeps its weight rows resident in
    shared memory (fetched beside the quantizer); bit-equal to quantize -> GEMM through the two separate entry points,
    whose GEMM is the weight-streaming kernel."""
    x, left, right = make_inputs(tokens, k, "bf16", 777 + tokens + n_out, True)
    g = torch.Generator().manual_seed(n_out)
    wq = torch.randint(-8, 8, (n_out, k), generator=g, dtype=torch.int8)
    wpd = torch.from_numpy(O.pack_int4_to_int32(wq.numpy())).to(DEV)
    swd = (torch.rand(n_out, generator=g) * 0.01 + 0.001).to(DEV)
    bias = (torch.randn(n_out, generator=g) * 0.1).bfloat16().to(DEV)
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    out = abi_linear(xd, ld, rd, wpd, swd, bias, 0.9, "bf16", "bf16")
    assert lib.qo_device_status(stream_ptr()) == N.QO_OK, lib.qo_last_error()
    aq, sa = abi_quantize(xd, ld, rd, 0.9, True, "bf16")
    two_call, acc = abi_int4_matmul(aq, wpd.t(), sa, swd, "bf16", True)
    np.testing.assert_array_equal(acc.cpu().numpy(), O.int4_accumulators(aq.cpu().numpy(), wpd.cpu().numpy().T))
    assert torch.equal(out, (two_call.float() + bias.float()).bfloat16())
