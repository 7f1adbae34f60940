"""Pins the CPU oracle before anything is compared against it.

Three kinds of pin, all CPU-only:
  * the reference's own unit-test cases for this path, replayed with the reference's tolerances
    (crates/tang-infer/src/quantize.rs:297-374, crates/tang-compute/src/cpu.rs:938-983,1095-1134,
    crates/tang-compute/src/modules.rs:629-641,717-728, crates/tang-compute/src/ops.rs:216-229,
    crates/tang-infer/src/sampling.rs:290-320);
  * bit-level rules the reference source defines but its tests do not check (nibble order, +8
    bias, round half away from zero, zero-block scale, ragged tail);
  * tests/golden/quantize_kat.json, produced by an independent restatement (see the script
    beside it), compared bit for bit.
"""
import json
import os
import struct

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quantize_kat.json")


def _f32(hexes):
    return np.array([struct.unpack("<f", bytes.fromhex(h))[0] for h in hexes], np.float32)


def _f64(hexes):
    return np.array([struct.unpack("<d", bytes.fromhex(h))[0] for h in hexes], np.float64)


# ---------------------------------------------------------------- reference unit tests, replayed

def test_ref_q8_roundtrip(orc):
    data = np.array([0.5, -1.0, 2.0, -3.0, 0.0, 1.5, -0.7, 0.3], np.float32)
    s, v = orc.quantize_q8(data)
    back = orc.dequantize_q8(s, v)
    assert np.all(np.abs(back[:8] - data) < 0.05)          # quantize.rs:304-309


def test_ref_q4_roundtrip(orc):
    data = np.array([0.5, -1.0, 2.0, -3.0, 0.0, 1.5, -0.7, 0.3], np.float32)
    s, p = orc.quantize_q4(data)
    back = orc.dequantize_q4(s, p)
    assert np.all(np.abs(back[:8] - data) < 1.0)           # quantize.rs:319-324


def test_ref_q8_matvec_basic(orc):
    s, v = orc.quantize_matrix_q8([1, 2, 3, 4, 5, 6], 2, 3)
    y = orc.q8_matvec(s, v, 2, 3, [1.0, 0.5, -1.0])
    assert abs(y[0] + 1.0) < 0.15 and abs(y[1] - 0.5) < 0.15   # quantize.rs:336-339


def test_ref_q4_matvec_basic(orc):
    s, p = orc.quantize_matrix_q4([1, 2, 3, 4, 5, 6], 2, 3)
    y = orc.q4_matvec(s, p, 2, 3, [1.0, 0.5, -1.0])
    assert abs(y[0] + 1.0) < 1.5 and abs(y[1] - 0.5) < 1.5     # quantize.rs:351-353


def test_ref_tensor_roundtrip(orc):
    data = np.array([1, -2, 3, -4, 5, -6], np.float32)       # quantize.rs:358-373 (flattened, one block)
    s, v = orc.quantize_q8(data)
    assert np.all(np.abs(orc.dequantize_q8(s, v)[:6] - data) < 0.1)


def test_ref_kv_attention_cases(orc):
    # cpu.rs:938-954: a query at position 0 sees only V[0].
    out = orc.kv_attention_f32([1, 0], [1, 0], [1, 2], 0, 1, 1, 1, 2)
    assert abs(out[0] - 1) < 1e-4 and abs(out[1] - 2) < 1e-4
    # cpu.rs:957-983: batched causal, first row = V[0], second leans to V[1].
    q = k = [1, 0, 0, 1, 1, 1]
    out = orc.kv_attention_f32(q, k, [1, 2, 3, 4, 5, 6], 0, 3, 1, 1, 2)
    assert abs(out[0] - 1) < 1e-5 and abs(out[1] - 2) < 1e-5
    assert out[2] > 1.5 and out[3] > 2.5
    w = np.exp(np.array([0.0, 1 / np.sqrt(2)]))
    w /= w.sum()
    assert abs(out[2] - (w[0] * 1 + w[1] * 3)) < 1e-5


def test_ref_kv_attention_batched_matches_sequential(orc):
    nh, nkv, hd, ql = 2, 1, 4, 4                             # cpu.rs:1095-1134
    td, kvd = nh * hd, nkv * hd
    q = np.array([((i * 7 + 3) % 13) / 13.0 for i in range(ql * td)], np.float32)
    k = np.array([((i * 11 + 5) % 17) / 17.0 for i in range(ql * kvd)], np.float32)
    v = np.array([((i * 13 + 7) % 19) / 19.0 for i in range(ql * kvd)], np.float32)
    batched = orc.kv_attention_f32(q, k, v, 0, ql, nh, nkv, hd)
    seq = np.concatenate([
        orc.kv_attention_f32(q[i * td:(i + 1) * td], k[:(i + 1) * kvd], v[:(i + 1) * kvd], i, 1, nh, nkv, hd)
        for i in range(ql)])
    assert np.max(np.abs(batched - seq)) < 1e-5


def test_ref_linear_forward(orc):
    # modules.rs:629-641: W=[[1,0],[0,1],[1,1]], b=[.1,.2,.3], x=[2,3] -> [2.1,3.2,5.3]
    y = orc.matmul_b_transposed_f32([2, 3], [1, 0, 0, 1, 1, 1], 1, 2, 3) + np.array([0.1, 0.2, 0.3], np.float32)
    assert np.allclose(y, [2.1, 3.2, 5.3], atol=1e-4)


def test_ref_rope_identity_at_pos_zero(orc):
    cos, sin = orc.rope_tables_f32(4, 32, 10000.0)           # modules.rs:717-728
    out = orc.rope_forward_f32([1, 2, 3, 4], cos, sin, 1, 1, 4, 0)
    assert np.allclose(out, [1, 2, 3, 4], atol=1e-5)
    # the f64 per-head rotation used by the decode loop agrees with the f32 table form
    x = np.arange(1, 9, dtype=np.float64)
    cos, sin = orc.rope_tables_f32(4, 32, 10000.0)
    a = orc.rope_forward_f32(x, cos, sin, 1, 2, 4, 5)
    b = orc.rope_heads_f64(x, 2, 4, 5, 10000.0)
    assert np.allclose(a, b, atol=1e-5)


def test_ref_swiglu(orc):
    v = orc.swiglu_f32([0, 1, -1], [1, 1, 1])                # ops.rs:216-229
    assert abs(v[0]) < 1e-5 and abs(v[1] - 0.7311) < 1e-3 and abs(v[2] + 0.2689) < 1e-3
    assert np.allclose(orc.swiglu_f64([0, 1, -1], [1, 1, 1]), v, atol=1e-6)


def test_ref_sampling_rules(orc):
    assert orc.argmax_f64([1.0, 2.0, 5.0, 3.0]) == 2         # sampling.rs:290-296
    assert orc.argmax_f64([5.0, 5.0]) == 0                   # strict '>' keeps the first maximum
    p = orc.topk_filter_f64([1.0, 100.0, 0.1, 99.0], 2)      # sampling.rs:298-320
    assert p[0] == 0 and p[2] == 0 and p[1] > 0 and p[3] > 0
    assert list(orc.topk_indices_f64([1.0, 3.0, 3.0, 2.0, 3.0], 3)) == [1, 2, 4]


def test_rms_norm_and_softmax(orc):
    x = np.array([1, 2, 3, 4], np.float32)
    w = np.array([1, 1, 2, 2], np.float32)
    exp = x / np.sqrt(np.mean(x * x) + 1e-5) * w
    assert np.allclose(orc.rms_norm_f32(x, w, 1, 4, 1e-5), exp, rtol=1e-6)
    assert np.allclose(orc.rms_norm_f64(x, w, 1e-5), exp, rtol=1e-6)
    out, s = orc.rms_norm_residual_f32(x, x, w, 1, 4, 1e-5)
    assert np.allclose(s, 2 * x) and np.allclose(out, orc.rms_norm_f32(2 * x, w, 1, 4, 1e-5))
    sm = orc.softmax_f32([1, 2, 3, 1, 1, 1], 2, 3)
    assert np.allclose(sm[:3], np.exp([1, 2, 3]) / np.exp([1, 2, 3]).sum(), rtol=1e-6)
    assert np.allclose(sm[3:], 1 / 3, rtol=1e-6)


# ---------------------------------------------------------------- bit-level rules from the source

def test_q4_nibble_order_and_bias(orc):
    # quantize.rs:110-111,125-126: byte = (q_even+8) | (q_odd+8)<<4 ; unpack = nibble-8.
    data = np.zeros(32, np.float32)
    data[0], data[1], data[2] = 7.0, -7.0, 1.0   # scale = 1 exactly (amax 7)
    s, p = orc.quantize_q4(data)
    assert s[0] == np.float32(1.0)
    assert p[0] == ((7 + 8) | ((-7 + 8) << 4)) and p[1] == ((1 + 8) | (8 << 4)) and np.all(p[2:] == 0x88)
    assert list(orc.unpack_q4(p)[:4]) == [7, -7, 1, 0]
    assert list(orc.unpack_q4(np.array([0x00, 0xFF, 0x8F], np.uint8))) == [-8, -8, 7, 7, 7, 0]


def test_round_half_away_and_clamp(orc):
    data = np.zeros(32, np.float32)
    data[:6] = [127.0, 0.5, -0.5, 1.5, -2.5, 126.5]          # scale 1: ties go away from zero
    s, v = orc.quantize_q8(data)
    assert s[0] == np.float32(1.0) and list(v[:6]) == [127, 1, -1, 2, -3, 127]
    data = np.zeros(32, np.float32)
    data[:3] = [-7.0, 6.5, -6.5]                              # q4: -7 stays, +-6.5 -> +-7; -8 only via clamp
    s, p = orc.quantize_q4(data)
    assert list(orc.unpack_q4(p)[:3]) == [-7, 7, -7]


def test_zero_block_scale_and_ragged_tail(orc):
    s, v = orc.quantize_q8(np.zeros(40, np.float32))
    assert list(s) == [1.0, 1.0] and not v.any()              # quantize.rs:58
    s, p = orc.quantize_q4(np.arange(1, 36, dtype=np.float32))
    assert s.size == 2 and p.size == 32
    assert np.all(p[18:] == 0x88) and (p[17] >> 4) == 8       # 3 live values in block 2, rest q=0
    # matvec must ignore the padded tail: cols=35
    w = np.arange(70, dtype=np.float32).reshape(2, 35)
    sc, pk = orc.quantize_matrix_q4(w, 2, 35)
    x = np.ones(35)
    y = orc.q4_matvec(sc, pk, 2, 35, x)
    deq = orc.dequantize_q4(sc.reshape(-1), pk.reshape(-1)).reshape(2, 64)[:, :35].astype(np.float64)
    assert np.allclose(y, deq.sum(axis=1), rtol=1e-6)   # dequantize rounds v*scale to f32, matvec does not


def test_matvec_is_sequential_f64(orc):
    # The reference adds (v*scale)*x term by term in f64 (quantize.rs:246,279-283).  Reproduce that
    # order in Python and demand bit equality on a case where order matters.
    rng = np.random.default_rng(7)
    rows, cols = 3, 96
    w = rng.standard_normal((rows, cols)).astype(np.float32)
    x = rng.standard_normal(cols) * np.logspace(-6, 6, cols)
    for bits in (8, 4):
        if bits == 8:
            sc, pv = orc.quantize_matrix_q8(w, rows, cols)
            ints = pv.astype(np.int64)
            y = orc.q8_matvec(sc, pv, rows, cols, x)
        else:
            sc, pv = orc.quantize_matrix_q4(w, rows, cols)
            ints = orc.unpack_q4(pv).reshape(rows, cols).astype(np.int64)
            y = orc.q4_matvec(sc, pv, rows, cols, x)
        for r in range(rows):
            s = 0.0
            for k in range(cols):
                s += float(ints[r, k]) * float(sc[r, k // 32]) * float(x[k])
            assert y[r] == s
    # thread count must not change a bit
    sc, pv = orc.quantize_matrix_q4(w, rows, cols)
    assert np.array_equal(orc.qmatmul(orc.KIND_Q4_F32, sc, pv, rows, cols, x, threads=1),
                          orc.qmatmul(orc.KIND_Q4_F32, sc, pv, rows, cols, x, threads=4))


def test_scale_variants_follow_block_matvec(orc):
    rng = np.random.default_rng(11)
    rows, cols = 5, 64
    packed = rng.integers(0, 256, (rows, cols // 2), dtype=np.uint8)
    scales32 = rng.uniform(0.002, 0.02, (rows, cols // 32)).astype(np.float32)
    f16 = scales32.astype(np.float16)
    x = rng.standard_normal(cols)
    a = orc.qmatmul(orc.KIND_Q4_F16, f16.view(np.uint16), packed, rows, cols, x)
    b = orc.qmatmul(orc.KIND_Q4_F32, f16.astype(np.float32), packed, rows, cols, x)
    assert np.array_equal(a, b)
    w8 = rng.integers(-127, 128, (rows, cols), dtype=np.int8)
    rs = rng.uniform(0.001, 0.01, rows).astype(np.float32)
    a = orc.qmatmul(orc.KIND_I8_ROW, rs, w8, rows, cols, x)
    b = orc.qmatmul(orc.KIND_Q8_F32, np.repeat(rs[:, None], cols // 32, 1), w8, rows, cols, x)
    assert np.array_equal(a, b)


def test_float_format_conversions(orc):
    L = orc.lib()
    # f16 -> f32 on every bit pattern, against numpy's IEEE half (NaNs compared as NaNs)
    allbits = np.arange(65536, dtype=np.uint16)
    ref = allbits.view(np.float16).astype(np.float32)
    got = orc.f16_bits_to_f32(allbits)
    nan = np.isnan(ref)
    assert np.array_equal(got[~nan], ref[~nan]) and np.all(np.isnan(got[nan]))
    # f32 -> f16 -> f32 is the identity on every finite half
    fin = allbits[np.isfinite(ref)]
    back = np.array([L.orc_f32_to_f16(float(v)) for v in ref[np.isfinite(ref)][::7]], np.uint16)
    assert np.array_equal(back, fin[::7])
    # bf16 round-to-nearest-even (cuda.rs:22-27): tie to even, ordinary rounding, exact values
    cases = {0x3F808000: 0x3F80, 0x3F818000: 0x3F82, 0x3F808001: 0x3F81, 0x3F800000: 0x3F80, 0xBF80C000: 0xBF81}
    for bits, want in cases.items():
        f = struct.unpack("<f", struct.pack("<I", bits))[0]
        assert L.orc_f32_to_bf16(f) == want
    x = np.random.default_rng(3).standard_normal(1000).astype(np.float32)
    assert np.array_equal(orc.f32_to_bf16_bits(x), np.array([L.orc_f32_to_bf16(float(v)) for v in x], np.uint16))


# ---------------------------------------------------------------- golden file

def test_golden_quantize(orc):
    g = json.load(open(GOLDEN))
    for name, case in g["quantize"].items():
        data = _f32(case["data_f32_hex"])
        if name.endswith("_q8"):
            s, v = orc.quantize_q8(data)
            payload = v.view(np.uint8)
        else:
            s, payload = orc.quantize_q4(data)
        assert [struct.pack("<f", x).hex() for x in s] == case["scales_f32_hex"], name
        assert list(payload) == case["payload_u8"], name


def test_golden_matvec(orc):
    g = json.load(open(GOLDEN))
    for name, case in g["matvec"].items():
        w, rows, cols = _f32(case["w_f32_hex"]), case["rows"], case["cols"]
        x, want = _f64(case["x_f64_hex"]), _f64(case["y_f64_hex"])
        if name.endswith("_q8"):
            s, v = orc.quantize_matrix_q8(w, rows, cols)
            y = orc.q8_matvec(s, v, rows, cols, x)
        else:
            s, p = orc.quantize_matrix_q4(w, rows, cols)
            y = orc.q4_matvec(s, p, rows, cols, x)
        assert np.array_equal(y, want), name


# ---------------------------------------------------------------------------------------------
# Sampler (crates/tang-infer/src/sampling.rs)
# ---------------------------------------------------------------------------------------------
def test_lcg_known_answers(orc):
    """sampling.rs:72-79: state' = state * 6364136223846793005 + 1442695040888963407 (mod 2^64), r = (state' >> 11) / 2^53,
    recomputed here with Python integers."""
    state = 42   # Sampler::new's seed (sampling.rs:63-68)
    for _ in range(5):
        want_state = (state * 6364136223846793005 + 1442695040888963407) % (1 << 64)
        r, got_state = orc.lcg_next_f64(state)
        assert got_state == want_state
        assert r == (want_state >> 11) / float(1 << 53) and 0.0 <= r < 1.0
        state = got_state


def test_sampler_reference_cases(orc):
    """The reference's own sampler tests (sampling.rs:265-340)."""
    greedy = orc.SamplerConfig(0.0, 0, 1.0, 1.0)
    assert orc.sampler_sample([1.0, 3.0, 10.0, 2.0], greedy, 42)[0] == 2            # greedy_sampling
    st = 42
    for _ in range(10):                                                              # greedy_sampling_repeated
        tok, st = orc.sampler_sample([1.0, 5.0, 3.0], greedy, st)
        assert tok == 1
    assert orc.sampler_sample([1.0, 2.0, 5.0, 3.0], greedy, 42)[0] == 2              # temperature_zero_is_greedy
    cfg = orc.SamplerConfig(1.0, 2, 1.0, 1.0)                                        # top_k_filters, seed 12345
    st, seen = 12345, set()
    for _ in range(100):
        tok, st = orc.sampler_sample([1.0, 100.0, 0.1, 99.0], cfg, st)
        seen.add(tok)
    assert seen == {1, 3}
    cfg = orc.SamplerConfig(1.0, 0, 0.5, 1.0)                                        # top_p_filters, seed 99
    st = 99
    for _ in range(20):
        tok, st = orc.sampler_sample([10.0, 0.0, 0.0, 0.0], cfg, st)
        assert tok == 0


def test_sampler_rules_read_from_the_source(orc):
    # repetition penalty: once per occurrence; positive logits are divided, the others multiplied (sampling.rs:94-104)
    cfg = orc.SamplerConfig(0.0, 0, 1.0, 2.0)
    assert orc.sampler_sample([4.0, 3.0, 1.0], cfg, 1, past=[0])[0] == 1             # 4/2 = 2 < 3
    assert orc.sampler_sample([4.0, 1.5, 1.0], cfg, 1, past=[0])[0] == 0             # 4/2 = 2 > 1.5
    assert orc.sampler_sample([4.0, 1.5, 1.0], cfg, 1, past=[0, 0])[0] == 1          # 4/2/2 = 1 < 1.5
    assert orc.sampler_sample([-1.0, -1.5, -3.0], cfg, 1, past=[0])[0] == 1          # -1*2 = -2 < -1.5
    # top-k keeps every entry that ties with the k-th largest (sampling.rs:127-133): k = 1 with two equal maxima
    cfg = orc.SamplerConfig(1.0, 1, 1.0, 1.0)
    st, seen = 7, set()
    for _ in range(200):
        tok, st = orc.sampler_sample([2.0, 5.0, 5.0, 1.0], cfg, st)
        seen.add(tok)
    assert seen == {1, 2}
    # top-p cuts after the first rank whose running sum reaches p; equal probabilities keep index order
    cfg = orc.SamplerConfig(1.0, 0, 0.5, 1.0)
    st, seen = 3, set()
    for _ in range(200):
        tok, st = orc.sampler_sample([1.0, 1.0, 1.0, 1.0], cfg, st)   # 0.25 each: ranks 0, 1 reach 0.5
        seen.add(tok)
    assert seen == {0, 1}
    # the draw itself: r < running sum, probabilities in index order
    cfg = orc.SamplerConfig(1.0, 0, 1.0, 1.0)
    logits = np.log(np.array([0.1, 0.2, 0.3, 0.4]))
    st = 2024
    for _ in range(50):
        r, _ = orc.lcg_next_f64(st)
        tok, st = orc.sampler_sample(logits, cfg, st)
        p = np.exp(logits - logits.max())
        p /= p.sum()
        assert tok == int(np.searchsorted(np.cumsum(p), r, side="right"))


def test_kv_cache_trim_reference_case(orc):
    """kv_cache.rs:228-252 (kv_cache_trim): five tokens whose rows hold 0..4, trim_to(3) keeps tokens 2, 3, 4 at rows
    0..2; trimming to at least the current length changes nothing (kv_cache.rs:139-141)."""
    kv_dim = 4
    rows = np.zeros((16, kv_dim), np.uint16)
    for i in range(5):
        rows[i] = i
    assert orc.kv_trim_to(rows, 5, 3) == 3
    assert [int(rows[r, 0]) for r in range(3)] == [2, 3, 4]
    before = rows.copy()
    assert orc.kv_trim_to(rows, 3, 3) == 3 and orc.kv_trim_to(rows, 3, 7) == 3
    assert np.array_equal(rows, before)
