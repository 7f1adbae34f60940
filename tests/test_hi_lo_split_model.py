"""Host model of the operand split of the tcgen05 dequant-GEMM (tang_b200/csrc/qgemm_umma.cu): a Q4 weight is
q * scale with q in -8..7 and an f16 scale, up to 15 significant bits, and goes to the tensor core as two bf16 numbers
    s_hi = bf16(scale), s_lo = bf16(scale - s_hi), t = bf16(q * s_lo),
    hi = bf16(fma(q, s_hi, t)),  lo = bf16(bf16(fma(q, s_hi, -hi)) + t).
The claim checked here, for EVERY finite f16 scale and every q: s_hi + s_lo = scale, t is exact, and hi + lo = q * scale
exactly, so that two MMAs reproduce exact products.  bf16 arithmetic is emulated in f64 with one round-to-nearest-even
to eight significant bits per operation (all magnitudes here are far inside bf16's normal range).  No GPU."""
import numpy as np


def rn_bf16(x):
    """Round f64 to eight significant bits, ties to even."""
    x = np.asarray(x, np.float64)
    m, e = np.frexp(x)                      # x = m * 2^e, 0.5 <= |m| < 1
    return np.ldexp(np.rint(np.ldexp(m, 8)), e - 8)


def test_hi_plus_lo_is_the_exact_product_for_every_f16_scale():
    bits = np.arange(1 << 16, dtype=np.uint16)
    scale = bits.view(np.float16).astype(np.float64)
    scale = scale[np.isfinite(scale)]
    s_hi = rn_bf16(scale)
    s_lo = rn_bf16(scale - s_hi)
    assert np.array_equal(s_hi + s_lo, scale)                 # 11 significant bits = 8 + 3
    for q in range(-8, 8):
        qf = float(q)
        t = rn_bf16(qf * s_lo)
        assert np.array_equal(t, qf * s_lo)                   # at most 7 bits: exact
        hi = rn_bf16(qf * s_hi + t)                           # fma: one rounding of the exact sum
        r = rn_bf16(qf * s_hi - hi)                           # fma(q, s_hi, -hi)
        assert np.array_equal(r, qf * s_hi - hi)              # the rounding error of hi without t: exact
        lo = rn_bf16(r + t)
        assert np.array_equal(lo, r + t)
        assert np.array_equal(hi + lo, qf * scale), q         # two terms carry the whole product


def test_single_term_is_within_half_a_bf16_ulp():
    """bf16 results use hi alone: the product rounded once, i.e. within 2^-8 relative (half a last place of an
    eight-bit significand)."""
    bits = np.arange(1 << 16, dtype=np.uint16)
    scale = bits.view(np.float16).astype(np.float64)
    scale = scale[np.isfinite(scale) & (scale != 0)]
    s_hi = rn_bf16(scale)
    s_lo = rn_bf16(scale - s_hi)
    for q in (-8, -7, -3, 1, 5, 7):
        hi = rn_bf16(q * s_hi + rn_bf16(q * s_lo))
        assert np.all(np.abs(hi - q * scale) <= np.abs(q * scale) * 2.0 ** -8)
        assert np.array_equal(hi, rn_bf16(q * scale))                 # and it IS the correctly rounded product


def test_f32_scales_keep_fifteen_bits():
    """Block formats with f32 scales (tang-infer's native Q4 and Q8 blocks): s_hi + s_lo holds 16 of the scale's 24 bits
    and q * s_lo is itself rounded for int8 codes, so hi + lo is the product to within 2^-15 relative, not exactly."""
    rng = np.random.default_rng(0)
    s = np.concatenate([(rng.random(200000) * 0.009 + 0.001), np.exp2(rng.uniform(-20, 4, 200000))])
    s = s.astype(np.float32).astype(np.float64)
    worst = 0.0
    for q in list(range(-8, 0)) + list(range(1, 8)) + [-127, -101, -77, 64, 85, 100, 127]:
        s_hi = rn_bf16(s)
        s_lo = rn_bf16(s - s_hi)
        t = rn_bf16(q * s_lo)
        hi = rn_bf16(q * s_hi + t)
        lo = rn_bf16(rn_bf16(q * s_hi - hi) + t)
        worst = max(worst, float(np.max(np.abs(hi + lo - q * s) / np.abs(q * s))))
    assert worst < 2.0 ** -15
