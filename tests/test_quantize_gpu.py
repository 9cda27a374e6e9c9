"""GPU parity of the FlatQuant quantizer: the C-ABI entry point against the numpy oracle and against the golden
fixtures made from the reference.  Tolerances are the stated ones: scales within 1e-3 relative, codes identical
except +-1 on at most 0.1 % of the elements."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import (N, QD, abi_quantize, bits_to_f32, bits_to_torch, compare_codes, compare_scales, golden, lib,
                     make_inputs, ptr, stream_ptr, t2f)
from oracle import w4a4_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLD = ["quant_fp16_4096_int8", "quant_bf16_4096_packed", "quant_bf16_14336_packed", "quant_bf16_11008_packed",
        "quant_fp32_2048_int8", "quant_fp16_4096_randnLR", "quant_fp16_256_packed", "quant_bf16_1024_int8"]




def run_both(x, left, right, clip, pack, dtype):
    """Yields (label, codes, scales) for the generic kernel and, if the shape has one, the tcgen05 kernel."""
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    codes, scales = abi_quantize(xd, ld, rd, clip, pack, dtype, policy=1)
    assert lib.qo_last_quantizer_path() == 1
    yield "generic", codes.cpu().numpy(), t2f(scales)
    try:
        codes, scales = abi_quantize(xd, ld, rd, clip, pack, dtype, policy=2)
    except N.QuantOpsError as e:
        assert e.status == N.QO_ERR_UNSUPPORTED
        return
    assert lib.qo_last_quantizer_path() == 2
    assert lib.qo_device_status(stream_ptr()) == N.QO_OK, lib.qo_last_error()
    yield "tcgen05", codes.cpu().numpy(), t2f(scales)


def check(codes, scales, ref_codes, ref_scales, pack):
    if pack:
        codes, ref_codes = O.unpack_int32_to_int4(codes), O.unpack_int32_to_int4(ref_codes)
    compare_scales(scales, ref_scales, 1e-3)
    return compare_codes(codes, ref_codes, 1e-3)


@pytest.mark.parametrize("name", GOLD)
def test_against_reference_fixtures(name):
    g = golden(name)
    dtype, clip, pack = str(g["dtype"]), float(g["clip"]), bool(g["pack"])
    x, left, right = (bits_to_torch(g[k], dtype) for k in ("x", "left", "right"))
    for label, codes, scales in run_both(x, left, right, clip, pack, dtype):
        assert codes.dtype == g["codes"].dtype and codes.shape == g["codes"].shape, label
        check(codes, scales, g["codes"], g["scales"], pack)


@pytest.mark.parametrize("dtype", ["bf16", "fp16", "fp32"])
def test_known_answer_rows(dtype):
    g = golden(f"kat_identity_{dtype}")
    x = torch.from_numpy(g["x"]).to(getattr(torch, {"bf16": "bfloat16", "fp16": "float16", "fp32": "float32"}[dtype]))
    eye = torch.eye(4, dtype=x.dtype)
    for clip, key in ((1.0, "c10"), (0.5, "c5")):
        for pack, suffix in ((False, "i"), (True, "p")):
            for label, codes, scales in run_both(x, eye, eye, clip, pack, dtype):
                rows = slice(0, 4) if dtype == "fp16" else slice(0, 5)
                np.testing.assert_array_equal(codes[rows], g[f"codes_{key}_{suffix}"][rows], err_msg=label)
                np.testing.assert_array_equal(scales[rows], g[f"scales_{key}_{suffix}"][rows], err_msg=label)
                if not pack:
                    assert codes[4].tolist() == [0] * 16  # zero row: code 0 in every dtype, never NaN garbage


CASES = [
    # tokens, features, dtype, clip, pack, outliers
    (128, 4096, "fp16", 1.0, False, False),   # the reference's CPU-runnable configuration
    (257, 4096, "bf16", 0.9, True, True),     # activation-scale configuration, ragged token count
    (1, 4096, "bf16", 0.9, True, True),
    (3, 14336, "bf16", 0.9, True, True),      # down_proj shape (112, 128)
    (130, 14336, "fp16", 1.0, False, True),
    (5, 11008, "bf16", 0.9, True, True),      # (86, 128)
    (33, 2048, "fp16", 0.6, True, False),     # (32, 64)
    (64, 1024, "bf16", 1.0, False, True),     # (32, 32)
    (127, 256, "fp32", 1.0, True, False),     # (16, 16)
    (7, 15, "fp32", 1.0, False, False),       # (3, 5): odd sizes, no packing possible
    (19, 8192, "bf16", 0.9, True, True),      # (64, 128)
]


@pytest.mark.parametrize("tokens,feat,dtype,clip,pack,outliers", CASES)
def test_against_oracle(tokens, feat, dtype, clip, pack, outliers):
    x, left, right = make_inputs(tokens, feat, dtype, 20240 + tokens + feat, outliers)
    ref_codes, ref_scales = O.flatquant_quantize(t2f(x), t2f(left), t2f(right), clip, pack, dtype)
    for label, codes, scales in run_both(x, left, right, clip, pack, dtype):
        check(codes, scales, ref_codes, ref_scales, pack)


WIDE = [(16, "bf16", 37, True), (32, "fp16", 9, False), (48, "bf16", 5, True), (64, "bf16", 131, True), (40, "bf16", 6, True),
        (100, "fp16", 3, True), (112, "bf16", 300, True), (128, "bf16", 4, False), (86, "fp16", 150, False)]
NARROWER = [(32, 32, "bf16", 149, True), (32, 48, "fp16", 77, True), (16, 16, "bf16", 33, False), (24, 32, "bf16", 5, True),
            (64, 48, "bf16", 6, False), (48, 16, "fp16", 300, True),
            (64, 80, "bf16", 150, True), (64, 96, "bf16", 33, True), (64, 112, "fp16", 150, False), (100, 96, "bf16", 7, True),
            (32, 80, "fp16", 9, True), (48, 112, "bf16", 10, False), (128, 80, "bf16", 5, True), (72, 112, "bf16", 149, True)]


@pytest.mark.parametrize("m,dtype,tokens,pack", WIDE)
def test_right_transform_of_size_128(m, dtype, tokens, pack):
    """Explicit (M, 128) factorisations: tiles of two tokens (M <= 64, multiple of 16) and of one token, M not a
    multiple of 16, odd and even token counts."""
    x, left, right = make_inputs(tokens, m * 128, dtype, 31 * m + tokens, True, mn=(m, 128))
    ref_codes, ref_scales = O.flatquant_quantize(t2f(x), t2f(left), t2f(right), 0.9, pack, dtype)
    for label, codes, scales in run_both(x, left, right, 0.9, pack, dtype):
        check(codes, scales, ref_codes, ref_scales, pack)


@pytest.mark.parametrize("m,n,dtype,tokens,pack", NARROWER)
def test_right_transforms_other_than_64_and_128(m, n, dtype, tokens, pack):
    """1024 = 32 x 32, 1536 = 32 x 48, 5120 = 64 x 80, 6144 = 64 x 96, 7168 = 64 x 112 and relatives run in the kernels for
    N = 64 / N = 128 with zero-padded columns."""
    x, left, right = make_inputs(tokens, m * n, dtype, 13 * m + n + tokens, True, mn=(m, n))
    ref_codes, ref_scales = O.flatquant_quantize(t2f(x), t2f(left), t2f(right), 0.9, pack, dtype)
    for label, codes, scales in run_both(x, left, right, 0.9, pack, dtype):
        check(codes, scales, ref_codes, ref_scales, pack)
    N.check(lib.qo_set_kernel_policy(2))  # the shape must have a tcgen05 kernel
    try:
        abi_quantize(x.to(DEV), left.to(DEV), right.to(DEV), 0.9, pack, dtype, policy=2)
    finally:
        lib.qo_set_kernel_policy(0)


@pytest.mark.parametrize("m,dtype,tokens,pack", [(16, "bf16", 41, True), (48, "bf16", 77, True), (48, "fp16", 6, False), (32, "bf16", 3, True),
                                                 (56, "bf16", 100, True), (40, "bf16", 9, True), (24, "fp16", 33, False),
                                                 (20, "bf16", 7, True), (36, "fp16", 50, False)])
def test_right_transform_of_size_64_small_left(m, dtype, tokens, pack):
    """(M, 64) with M < 64, e.g. 3072 = 48 x 64: groups of two tokens whose rows do not fill whole warps; 3584 = 56 x 64
    and other multiples of 8 pad each token's reduction length; M = 20 or 36 take the shape-general tcgen05 kernel."""
    x, left, right = make_inputs(tokens, m * 64, dtype, 17 * m + tokens, True, mn=(m, 64))
    ref_codes, ref_scales = O.flatquant_quantize(t2f(x), t2f(left), t2f(right), 0.9, pack, dtype)
    for label, codes, scales in run_both(x, left, right, 0.9, pack, dtype):
        check(codes, scales, ref_codes, ref_scales, pack)


@pytest.mark.parametrize("feat,dtype", [(28672, "bf16"), (32768, "fp16"), (24576, "fp32")])
def test_very_wide_rows_take_the_generic_kernel(feat, dtype):
    """28672 = 128 x 224 (the down-projection input of the 70B-class models) and 32768 = 128 x 256 have no tensor-core
    kernel (right transform above 128); the SIMT kernel must take them."""
    x, left, right = make_inputs(3, feat, dtype, feat + 3, True)
    ref_codes, ref_scales = O.flatquant_quantize(t2f(x), t2f(left), t2f(right), 0.9, True, dtype)
    codes, scales = abi_quantize(x.to(DEV), left.to(DEV), right.to(DEV), 0.9, True, dtype, policy=0)
    assert lib.qo_last_quantizer_path() == 1
    check(codes.cpu().numpy(), t2f(scales), ref_codes, ref_scales, True)


def test_activation_scale_config_sampled_rows():
    """8192 x 4096 bf16, 1 % outlier channels, clip 0.9, packed: every row quantized on the GPU, a seeded sample of
    rows compared with the oracle (rows are independent), and a dequantize round trip over everything."""
    x, left, right = make_inputs(8192, 4096, "bf16", 20242, True)
    rows = np.random.default_rng(5).choice(8192, 192, replace=False)
    rows.sort()
    ref_codes, ref_scales = O.flatquant_quantize(t2f(x[rows]), t2f(left), t2f(right), 0.9, True, "bf16")
    for label, codes, scales in run_both(x, left, right, 0.9, True, "bf16"):
        check(codes[rows], scales[rows], ref_codes, ref_scales, True)
        unpacked = O.unpack_int32_to_int4(codes)
        assert unpacked.min() >= -8 and unpacked.max() <= 7
        assert np.all(np.isfinite(scales)) and np.all(scales > 0)
        # each row reaches full scale on at least one side when clip <= 1 (the extreme value maps to +-7 or beyond)
        assert np.all(np.abs(unpacked.astype(np.int32)).max(axis=1) >= 7)


@pytest.mark.parametrize("tokens,feat", [(8192, 4096), (4096, 14336)])
def test_full_size_every_row_follows_from_the_transform(tokens, feat):
    """Full benchmark sizes, EVERY row: the scales and codes the tensor-core kernel stores are exactly what the reference's
    elementwise steps (flatquant/ops.py:108-117: row extremes, clip, division by 7, quotient, round half to even, clamp)
    give when applied, in bf16 like the reference, to the transformed activations the same kernel produces through its
    transform-only entry point.  (The transform itself is compared with the oracle on sampled rows in the tests above;
    rows are independent, so together the two cover every row at full size.)"""
    m, n = O.get_decompose_dim(feat)
    x, left, right = make_inputs(tokens, feat, "bf16", 20251, True)
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    codes, scales = abi_quantize(xd, ld, rd, 0.9, True, "bf16", policy=2)
    assert lib.qo_last_quantizer_path() == 2
    z = torch.empty(tokens, feat, device=DEV)
    N.check(lib.qo_set_kernel_policy(2))
    N.check(lib.qo_flatquant_transform(ptr(xd), feat, ptr(ld), ptr(rd), ptr(z), tokens, m, n, QD["bf16"], stream_ptr()))
    lib.qo_set_kernel_policy(0)
    assert lib.qo_device_status(stream_ptr()) == N.QO_OK
    zb = z.bfloat16()
    assert torch.equal(zb.float(), z)                                   # the entry point returns values of the activation dtype
    xmax = torch.maximum((zb.amin(dim=1) * 0.9).abs(), zb.amax(dim=1) * 0.9)    # bf16 tensor times a Python float, as in the reference
    want_s = (xmax / 7).clamp(min=1e-8)
    assert torch.equal(scales, want_s.float())
    want_q = torch.round(zb / want_s[:, None]).clamp(-8, 7).to(torch.int32)
    sh = torch.arange(8, device=DEV, dtype=torch.int32) * 4
    got_q = ((codes[:, :, None] >> sh) & 15).reshape(tokens, feat) - 8   # nibble i of word p = code[8p + i] + 8
    assert torch.equal(got_q, want_q)


def test_row_stride_and_scale_dtype():
    x, left, right = make_inputs(40, 4096, "bf16", 77, True)
    wide = torch.zeros(40, 4096 + 64, dtype=x.dtype)
    wide[:, :4096] = x
    xd = wide.to(DEV)[:, :4096]
    assert xd.stride(0) == 4160
    ref_codes, ref_scales = O.flatquant_quantize(t2f(x), t2f(left), t2f(right), 0.9, True, "bf16")
    for policy in (1, 0):
        codes, scales = abi_quantize(xd, left.to(DEV), right.to(DEV), 0.9, True, "bf16", scale_dtype="fp16", policy=policy)
        assert scales.dtype == torch.float16
        check(codes.cpu().numpy(), t2f(scales), ref_codes, O.round_to(ref_scales, "fp16"), True)


def test_zero_tokens_and_bad_arguments():
    x, left, right = make_inputs(4, 256, "bf16", 1, False)
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    codes, scales = abi_quantize(xd[:0], ld, rd, 1.0, True, "bf16")
    assert codes.shape == (0, 32) and scales.shape == (0,)
    out = torch.empty(4, 256, dtype=torch.int8, device=DEV)
    sc = torch.empty(4, device=DEV)
    rc = lib.qo_flatquant_quantize(ptr(xd), 100, ptr(ld), ptr(rd), ptr(out), ptr(sc), 4, 16, 16, 1.0, N.QO_BF16, 0, N.QO_F32, stream_ptr())
    assert rc == N.QO_ERR_INVALID_ARGUMENT
    rc = lib.qo_flatquant_quantize(None, 256, ptr(ld), ptr(rd), ptr(out), ptr(sc), 4, 16, 16, 1.0, N.QO_BF16, 0, N.QO_F32, stream_ptr())
    assert rc == N.QO_ERR_INVALID_ARGUMENT


def test_idempotent_and_deterministic():
    x, left, right = make_inputs(300, 4096, "bf16", 9, True)
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    c1, s1 = abi_quantize(xd, ld, rd, 0.9, True, "bf16")
    c2, s2 = abi_quantize(xd, ld, rd, 0.9, True, "bf16")
    assert torch.equal(c1, c2) and torch.equal(s1, s2)
    # permuting the tokens permutes the outputs (rows are independent)
    perm = torch.randperm(300, generator=torch.Generator().manual_seed(3)).to(DEV)
    c3, s3 = abi_quantize(xd[perm].contiguous(), ld, rd, 0.9, True, "bf16")
    assert torch.equal(c3, c1[perm]) and torch.equal(s3, s1[perm])


def test_host_buffer_entry_point():
    x, left, right = make_inputs(3000, 4096, "bf16", 11, True)
    xp = x.pin_memory()
    codes = torch.empty(3000, 512, dtype=torch.int32).pin_memory()
    scales = torch.empty(3000, dtype=torch.float32).pin_memory()
    N.check(lib.qo_flatquant_quantize_host(ptr(xp), ptr(left), ptr(right), ptr(codes), ptr(scales), 3000, 64, 64, 0.9,
                                           N.QO_BF16, 1, N.QO_F32))
    c_dev, s_dev = abi_quantize(x.to(DEV), left.to(DEV), right.to(DEV), 0.9, True, "bf16")
    assert torch.equal(codes, c_dev.cpu()) and torch.equal(scales, s_dev.cpu())


@pytest.mark.parametrize("tokens,feat,dtype", [(5, 4096, "bf16"), (3, 14336, "fp16"), (4, 11008, "bf16"), (6, 256, "fp32")])
def test_transform_entry_point(tokens, feat, dtype):
    """The Kronecker transform alone, both kernels, against the oracle (a handful of 1-ulp roundings may differ:
    the products are accumulated in a different order)."""
    x, left, right = make_inputs(tokens, feat, dtype, 55, True)
    ref = O.kronecker_transform(t2f(x), t2f(left), t2f(right), dtype)
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    for policy in (1, 2):
        z = torch.empty(tokens, feat, device=DEV)
        N.check(lib.qo_set_kernel_policy(policy))
        rc = lib.qo_flatquant_transform(ptr(xd), feat, ptr(ld), ptr(rd), ptr(z), tokens, left.shape[0], right.shape[0],
                                        QD[dtype], stream_ptr())
        lib.qo_set_kernel_policy(0)
        if rc == N.QO_ERR_UNSUPPORTED and policy == 2:
            continue
        N.check(rc)
        assert lib.qo_device_status(stream_ptr()) == N.QO_OK
        got = t2f(z)
        ulp = {"bf16": 2.0 ** -7, "fp16": 2.0 ** -10, "fp32": 2.0 ** -20}[dtype]
        # a flipped rounding of Y moves Z by a fraction of Y's spacing, so the bound is relative to the row's range
        assert np.all(np.abs(got - ref) <= ulp * np.abs(ref).max(axis=1, keepdims=True) * 1.01 + 1e-6)
        assert (got != ref).mean() < 2e-2
