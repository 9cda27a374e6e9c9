"""Exhaustive CPU checks of the exactness arguments the quantizer kernels rely on.

The tcgen05 quantizers (quant_ops_b200/csrc/flatquant_sm100_n64.cu, flatquant_sm100_common.cuh) replace two
divisions of the reference (src/quant_ops/ops/quantization/flatquant/ops.py:113, :116) by cheaper sequences and
claim the results are identical:

  1. scale:     round16(top * 0.142857149f)  ==  round16(top / 7)      for every value `top` of the 16-bit dtype
  2. quotient:  bf16: fma_bf16(z, hi, mul_bf16(z, lo)) == round_bf16(z / s), hi + lo ~ 1/s as two bf16 terms
                fp16: two float32 FMAs refine z * (1/s) to the correctly rounded float32 quotient, which rounds to
                      fp16 like the exact quotient

Everything is integer or exactly representable floating-point arithmetic, so the checks are exact; they cover every
significand (the computations are invariant under scaling by powers of two) and both signs where the sign matters.
"""
import numpy as np
import torch


def _all_16bit_values(dtype):
    bits = torch.arange(0, 1 << 16, dtype=torch.int32).to(torch.int16)
    v = bits.view(dtype).float()
    v = v[torch.isfinite(v) & (v >= 0)]
    return v


def test_scale_product_with_one_seventh_rounds_like_the_division():
    """round(top * 0.142857149f) == round(top / 7) in bf16 and fp16, for every non-negative finite `top`."""
    seventh = torch.tensor(0.142857149, dtype=torch.float32)
    for dtype in (torch.bfloat16, torch.float16):
        top = _all_16bit_values(dtype)
        prod = (top * seventh).to(dtype)                          # one float32 product, one rounding to 16 bits
        quot = (top / 7.0).to(dtype)                              # the reference: float32 division, then 16 bits
        exact = (top.double() / 7.0)
        # the float32 quotient rounds to 16 bits like the exact one (no double-rounding case exists) ...
        assert torch.equal(quot, _round_exact(exact, dtype))
        # ... and so does the product with the float32 constant
        assert torch.equal(prod, quot), f"{dtype}: {(prod != quot).sum().item()} values differ"


def _round_exact(x64: torch.Tensor, dtype) -> torch.Tensor:
    """float64 -> 16-bit type with a single rounding (float64 -> 16 bit conversions in torch round once)."""
    return x64.to(dtype)


def _round_sig(v: int, bits: int):
    """(mantissa, exponent) of the non-negative integer v rounded to `bits` significant bits, half to even."""
    if v == 0:
        return 0, 0
    sh = v.bit_length() - bits
    if sh <= 0:
        return v, 0
    q, r = v >> sh, v & ((1 << sh) - 1)
    half = 1 << (sh - 1)
    if r > half or (r == half and (q & 1)):
        q += 1
    return q, sh


def _round_frac(num: int, den: int, bits: int):
    """num / den (positive) rounded to `bits` significant bits, half to even, as a (mantissa, exponent) pair."""
    # scale so that the integer quotient has at least bits + 2 bits, keep the remainder as a sticky bit
    e = 0
    while (num << e) // den < (1 << (bits + 1)):
        e += 1
    q, rem = divmod(num << e, den)
    q = (q << 1) | (1 if rem else 0)  # sticky
    m, sh = _round_sig(q, bits)
    return m, sh - e - 1


def test_two_term_bf16_quotient_is_exact_for_every_significand_pair():
    """fma(z, hi, round(z * lo)) == round(z / s) in bf16, hi = round(1/s), lo = round(1/s - hi), 1/s in float32."""
    bad = 0
    for ks in range(128, 256):                       # s = ks / 128 in [1, 2)
        # float32 reciprocal, correctly rounded: 1/s = 128 / ks
        im, ie = _round_frac(128, ks, 24)            # inv = im * 2**ie
        hm, hs = _round_sig(im, 8)                   # hi = hm * 2**(ie + hs)
        hi_num, hi_exp = hm, ie + hs
        # rest = inv - hi, exact in float32; both at exponent ie
        rest = im - (hm << hs)
        neg = rest < 0
        lm, ls = _round_sig(abs(rest), 8)
        lo_num, lo_exp = (-lm if neg else lm), ie + ls
        for kz in range(128, 256):                   # z = kz / 128; the sign of z flips every term, RNE is symmetric
            # t = round_bf16(z * lo): product kz * lo_num at exponent lo_exp - 7
            p = kz * lo_num
            tm, ts = _round_sig(abs(p), 8)
            t_num, t_exp = (-tm if p < 0 else tm), lo_exp - 7 + ts
            # got = round_bf16(z * hi + t), a single rounding of the exact sum
            a_num, a_exp = kz * hi_num, hi_exp - 7
            e = min(a_exp, t_exp)
            total = (a_num << (a_exp - e)) + (t_num << (t_exp - e))
            gm, gs = _round_sig(total, 8)
            got = (gm, gs + e)
            wm, we = _round_frac(kz, ks, 8)
            want = (wm, we)
            # normalise both (mantissa may be 2**8 after a carry)
            def norm(m, x):
                while m and m % 2 == 0:
                    m //= 2
                    x += 1
                return m, x
            if norm(*got) != norm(*want):
                bad += 1
    assert bad == 0, f"{bad} of {128 * 128} significand pairs differ"


def test_fp16_quotient_through_two_float32_fmas_is_correctly_rounded():
    """q = z * r; q' = fma(fma(-q, s, z), r, q) with r = float32(1/s) equals float32(z / s) for all fp16 significands,
    and float16(float32(z / s)) == float16(z / s): no double rounding."""
    rng = np.random.default_rng(7)
    ks_all = np.arange(1024, 2048)
    # every s significand against a different random third of the z significands each (exact integer arithmetic is
    # slow in Python; 350,000 pairs), plus all pairs with the extreme significands
    bad = 0
    cases = 0
    for ks in ks_all:
        im, ie = _round_frac(1024, int(ks), 24)      # r = float32(1 / s), s = ks / 1024
        kzs = set(rng.choice(np.arange(1024, 2048), 340, replace=False).tolist()) | {1024, 1025, 2046, 2047}
        for kz in kzs:
            # q0 = float32(z * r): kz * im at exponent ie - 10
            qm, qs = _round_sig(kz * im, 24)
            q_exp = ie - 10 + qs
            # e1 = fma(-q0, s, z) exactly representable (checked): z - q0 * s
            # common exponent: q0 * s = qm * ks * 2**(q_exp - 10); z = kz * 2**-10
            ex = min(q_exp - 10, -10)
            res = (kz << (-10 - ex)) - ((qm * int(ks)) << (q_exp - 10 - ex))
            rm, rs = _round_sig(abs(res), 24)
            assert rs == 0                             # the residual is exact in float32
            r_num = -rm if res < 0 else rm
            # q1 = float32(e1 * r + q0)
            a_num, a_exp = r_num * im, ex + ie
            e = min(a_exp, q_exp)
            total = (a_num << (a_exp - e)) + (qm << (q_exp - e))
            gm, gs = _round_sig(total, 24)
            wm, we = _round_frac(kz, int(ks), 24)
            g, w = gm * 2.0 ** (gs + e), wm * 2.0 ** we
            cases += 1
            if g != w:
                bad += 1
            # float16 of the float32 quotient == float16 of the exact quotient
            hm, he = _round_frac(kz, int(ks), 11)
            if np.float16(np.float32(w)) != np.float16(hm * 2.0 ** he):
                bad += 1
    assert bad == 0, f"{bad} mismatches in {cases} cases"
