"""Pins the numpy oracle to the reference: every fixture under tests/golden/ was produced by the reference's own
PyTorch functions on CPU (tests/golden/make_golden.py); the oracle must reproduce them."""
import numpy as np
import pytest

from helpers import bits_to_f32, compare_codes, compare_scales, golden
from oracle import w4a4_oracle as O

QUANT = ["quant_fp16_4096_int8", "quant_bf16_4096_packed", "quant_bf16_14336_packed", "quant_bf16_11008_packed",
         "quant_fp32_2048_int8", "quant_fp16_4096_randnLR", "quant_fp16_256_packed", "quant_bf16_1024_int8"]


def test_decompose_matches_reference():
    g = golden("decompose")
    for n, (m_ref, n_ref) in zip(g["n"], g["mn"]):
        assert O.get_decompose_dim(int(n)) == (int(m_ref), int(n_ref))


def test_decompose_rejects_2_mod_4():
    for n in (2, 6, 10, 4098):
        with pytest.raises(ValueError):
            O.get_decompose_dim(n)


@pytest.mark.parametrize("name", QUANT)
def test_quantizer_matches_reference(name):
    g = golden(name)
    dtype, clip, pack = str(g["dtype"]), float(g["clip"]), bool(g["pack"])
    x, left, right = (bits_to_f32(g[k], dtype) for k in ("x", "left", "right"))
    codes, scales = O.flatquant_quantize(x, left, right, clip, pack, dtype)
    assert codes.dtype == g["codes"].dtype and codes.shape == g["codes"].shape
    ref, got = g["codes"], codes
    if pack:
        ref, got = O.unpack_int32_to_int4(ref), O.unpack_int32_to_int4(got)
    # accumulation order inside the reference's matmul is not pinned: allow its one-in-a-million rounding flips
    compare_codes(got, ref, max_frac=2e-5)
    compare_scales(scales, g["scales"], rel=1e-6)
    deq = O.dequantize_int4(g["codes"][:2], g["scales"][:2], pack)
    np.testing.assert_array_equal(deq, g["dequant_head"])


@pytest.mark.parametrize("dtype", ["bf16", "fp16", "fp32"])
def test_known_answer_rows(dtype):
    g = golden(f"kat_identity_{dtype}")
    x = g["x"]
    eye = np.eye(4, dtype=np.float32)
    for clip, key in ((1.0, "c10"), (0.5, "c5")):
        for pack, suffix in ((False, "i"), (True, "p")):
            codes, scales = O.flatquant_quantize(x, eye, eye, clip, pack, dtype)
            rows = slice(0, 4) if dtype == "fp16" else slice(0, 5)  # fp16 zero row: 0/0 in the reference, cast undefined
            np.testing.assert_array_equal(codes[rows], g[f"codes_{key}_{suffix}"][rows])
            np.testing.assert_array_equal(scales[rows], g[f"scales_{key}_{suffix}"][rows])
    # the documented known answers
    codes, scales = O.flatquant_quantize(x, eye, eye, 1.0, False, dtype)
    assert codes[0, :8].tolist() == [7, 4, 2, 2, 0, 0, -2, -4] and scales[0] == 1.0
    assert codes[2, :2].tolist() == [-7, 1]
    assert codes[4].tolist() == [0] * 16
    packed, _ = O.flatquant_quantize(x, eye, eye, 1.0, True, dtype)
    assert packed.view(np.uint32)[3, 0] == 0xF8888888 and packed.view(np.uint32)[3, 1] == 0x88888888
    codes, scales = O.flatquant_quantize(x, eye, eye, 0.5, False, dtype)
    assert codes[1, :4].tolist() == [-8, 7, 7, -8]


@pytest.mark.parametrize("name", ["gemm_64x512x96", "gemm_33x256x40"])
def test_gemm_matches_reference(name):
    g = golden(name)
    np.testing.assert_array_equal(O.pack_int4_to_int32(g["a_codes"]), g["a_packed"])
    np.testing.assert_array_equal(O.unpack_int32_to_int4(g["a_packed"]), g["a_codes"])
    np.testing.assert_array_equal(O.pack_int4_to_int32(np.ascontiguousarray(g["b_codes"].T)).T, g["b_packed"])
    np.testing.assert_array_equal(O.int4_accumulators(g["a_packed"], g["b_packed"]), g["acc"])
    out = O.int4_matmul(g["a_packed"], g["b_packed"], g["scale_a"], g["scale_b"], "fp16")
    np.testing.assert_array_equal(out, bits_to_f32(g["out_bits"], "fp16"))


def test_fused_layer_matches_reference():
    g = golden("linear_bf16_1024x48")
    x, left, right = (bits_to_f32(g[k], "bf16") for k in ("x", "left", "right"))
    a, s = O.flatquant_quantize(x, left, right, float(g["clip"]), True, "bf16")
    np.testing.assert_array_equal(a, g["a_packed"])
    np.testing.assert_array_equal(s, g["a_scale"])
    out = O.w4a4_linear(x, left, right, float(g["clip"]), g["w_packed"], g["w_scale"], "bf16", "fp16")
    np.testing.assert_array_equal(out, bits_to_f32(g["out_bits"], "fp16"))


def test_empty_and_errors():
    eye = np.eye(4, dtype=np.float32)
    c, s = O.flatquant_quantize(np.zeros((0, 16), np.float32), eye, eye, 1.0, True, "bf16")
    assert c.shape == (0, 2) and s.shape == (0,)
    with pytest.raises(ValueError):
        O.flatquant_quantize(np.zeros((2, 15), np.float32), eye, eye)
    with pytest.raises(ValueError):
        O.pack_int4_to_int32(np.zeros((2, 12), np.int8))


def test_round_to_matches_torch():
    import torch

    rng = np.random.default_rng(0)
    v = (rng.standard_normal(20000) * np.exp(rng.uniform(-20, 20, 20000))).astype(np.float32)
    v[:4] = [0.0, -0.0, 1.00390625, 3.0e38]
    np.testing.assert_array_equal(O.round_to(v, "bf16"), torch.from_numpy(v).bfloat16().float().numpy())
    np.testing.assert_array_equal(O.round_to(v, "fp16"), torch.from_numpy(v).half().float().numpy())


@pytest.mark.parametrize("name", ["quant_bf16_4096_packed", "quant_fp16_4096_int8", "quant_bf16_14336_packed"])
def test_torch_port_matches_reference(name):
    """The torch restatement timed as the CPU baseline computes what the reference computes."""
    import torch

    from helpers import bits_to_torch
    from oracle import torch_port

    g = golden(name)
    dtype = str(g["dtype"])
    x, left, right = (bits_to_torch(g[k], dtype) for k in ("x", "left", "right"))
    torch.set_num_threads(1)
    codes, scales = torch_port.quantize(x, left, right, float(g["clip"]), bool(g["pack"]))
    np.testing.assert_array_equal(codes.numpy(), g["codes"])
    np.testing.assert_array_equal(scales.float().numpy(), g["scales"])


def test_torch_port_matmul_matches_reference():
    import torch

    from oracle import torch_port

    g = golden("gemm_64x512x96")
    out = torch_port.matmul(*(torch.from_numpy(g[k]) for k in ("a_packed", "b_packed", "scale_a", "scale_b")))
    np.testing.assert_array_equal(out.float().numpy(), bits_to_f32(g["out_bits"], "fp16"))


def test_float_simulation_of_the_layer_agrees_with_the_integer_path():
    """The reference's fake-quant layer (restated in the oracle) and the integer path describe the same layer:
    identical scales and codes for rows that straddle zero, outputs equal up to the dtype rounding of the
    de-quantized operands."""
    rng = np.random.default_rng(7)
    m, n, n_out, tokens = 16, 16, 40, 24
    x = O.round_to(rng.standard_normal((tokens, m * n)).astype(np.float32), "bf16")
    left = O.round_to(np.linalg.qr(rng.standard_normal((m, m)))[0].astype(np.float32), "bf16")
    right = O.round_to(np.linalg.qr(rng.standard_normal((n, n)))[0].astype(np.float32), "bf16")
    wq, sw = O.quantize_weights((rng.standard_normal((n_out, m * n)) * 0.02).astype(np.float32))
    exact = O.w4a4_linear(x, left, right, 0.9, O.pack_int4_to_int32(wq), sw, "bf16", "bf16")
    sim = O.fake_quant_linear(x, left, right, 0.9, wq, sw, "bf16")
    assert exact.shape == sim.shape == (tokens, n_out)
    bound = 2e-2 * np.abs(exact).max(axis=1, keepdims=True)
    assert np.all(np.abs(exact - sim) <= bound)
