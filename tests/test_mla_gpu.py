"""GPU parity of the MLA decode attention against the oracle (parity unpinned: the reference has no
MLA).  The oracle's absorbed form mirrors the device's two bf16 rounding points; its naive form
(keys and values materialised per head) checks the absorption algebra itself."""
import numpy as np
import pytest

from util import bf16_round, rel_err

C_, R_, NOPE, VD = 512, 64, 128, 128


@pytest.fixture(scope="module")
def dev():
    import tang_b200

    d = tang_b200.QuantComputeDevice(0)
    yield d
    d.close()


def make(rng, H, B, max_seq):
    w_qk = rng.integers(-127, 128, (H * C_, NOPE), dtype=np.int8)
    s_qk = rng.uniform(0.001, 0.01, H * C_).astype(np.float32)
    w_uv = rng.integers(-127, 128, (H * VD, C_), dtype=np.int8)
    s_uv = rng.uniform(0.001, 0.01, H * VD).astype(np.float32)
    qn = bf16_round(rng.standard_normal((B, H, NOPE)).astype(np.float32))
    qr = bf16_round(rng.standard_normal((B, H, R_)).astype(np.float32))
    cache = bf16_round(rng.standard_normal((B, max_seq, C_ + R_)).astype(np.float32))
    return w_qk, s_qk, w_uv, s_uv, qn, qr, cache


@pytest.mark.gpu
@pytest.mark.parametrize("H,B,lens", [(16, 1, [200]), (32, 3, [1, 64, 333]), (128, 2, [4096, 1000]), (16, 4, [65, 128, 129, 700])])
def test_mla_decode_matches_oracle(dev, orc, H, B, lens):
    import tang_b200 as tb

    rng = np.random.default_rng(H + B)
    max_seq = max(lens) + 2
    w_qk, s_qk, w_uv, s_uv, qn, qr, cache = make(rng, H, B, max_seq)
    wq = dev.upload_qarrays(tb.I8_ROW, w_qk, s_qk, H * C_, NOPE)
    wu = dev.upload_qarrays(tb.I8_ROW, w_uv, s_uv, H * VD, C_)
    out = tb.mla_decode(dev, wq, wu, dev.upload(qn[0], tb.BF16), dev.upload(qr[0], tb.BF16), dev.upload(cache[0], tb.BF16),
                        np.array(lens, np.int32), B, H, NOPE, VD, max_seq * (C_ + R_), max(lens))
    dev.sync()
    got = out.to_vec().reshape(B, H * VD)
    dims = orc.MlaDims(H, C_, NOPE, R_, VD)
    for b in range(B):
        want = orc.mla_decode_f64(dims, qn[1][b].astype(np.float64), qr[1][b].astype(np.float64), cache[0][b], lens[b],
                                  w_qk, s_qk, w_uv, s_uv, absorbed=True)
        # q_lat and o_lat pass through bf16 on both sides: a one-ulp flip there moves the result by a
        # fraction of a percent of its rms, so the bar is relative to max(|ref|, rms)
        assert rel_err(got[b], want, floor_frac=1.0) < 2e-3, (b, lens[b])


def test_absorbed_equals_naive_in_the_oracle(orc):
    rng = np.random.default_rng(3)
    H, ctx = 4, 37
    w_qk, s_qk, w_uv, s_uv, qn, qr, cache = make(rng, H, 1, ctx)
    dims = orc.MlaDims(H, C_, NOPE, R_, VD)
    # small queries keep the softmax smooth, so the check is about the algebra and not about how a peaky
    # softmax amplifies the absorbed form's bf16 rounding of q_lat
    args = (dims, 0.05 * qn[1][0].astype(np.float64), 0.05 * qr[1][0].astype(np.float64), cache[0][0], ctx, w_qk, s_qk, w_uv, s_uv)
    a = orc.mla_decode_f64(*args, absorbed=True)
    n = orc.mla_decode_f64(*args, absorbed=False)
    assert rel_err(a, n, floor_frac=1.0) < 1e-2      # only the two bf16 roundings of the absorbed form apart


@pytest.mark.gpu
def test_head_shards_concatenate_to_the_full_result(dev, orc):
    """Tensor parallelism of MLA decode is by head with the latent cache replicated: running the two halves of
    the heads (their rows of W_UK / W_UV, their queries) separately gives the full output's halves bit for bit;
    only the row-parallel W_O that follows needs an all-reduce (tests/test_tp.py covers that pattern)."""
    import tang_b200 as tb

    rng = np.random.default_rng(77)
    H, B, lens = 32, 2, [300, 77]
    max_seq = max(lens) + 1
    w_qk, s_qk, w_uv, s_uv, qn, qr, cache = make(rng, H, B, max_seq)
    cbuf = dev.upload(cache[0], tb.BF16)

    def run(h0, h1):
        n = h1 - h0
        wq = dev.upload_qarrays(tb.I8_ROW, w_qk[h0 * C_:h1 * C_], s_qk[h0 * C_:h1 * C_], n * C_, NOPE)
        wu = dev.upload_qarrays(tb.I8_ROW, w_uv[h0 * VD:h1 * VD], s_uv[h0 * VD:h1 * VD], n * VD, C_)
        o = tb.mla_decode(dev, wq, wu, dev.upload(np.ascontiguousarray(qn[0][:, h0:h1]), tb.BF16),
                          dev.upload(np.ascontiguousarray(qr[0][:, h0:h1]), tb.BF16), cbuf, np.array(lens, np.int32), B, n, NOPE, VD,
                          max_seq * (C_ + R_), max(lens))
        dev.sync()
        return o.to_vec().reshape(B, n * VD)

    full = run(0, H)
    halves = np.concatenate([run(0, H // 2), run(H // 2, H)], axis=1)
    assert np.array_equal(full, halves)


@pytest.mark.gpu
@pytest.mark.parametrize("ctx,B", [(16384, 1), (32768, 1), (16384, 16)])
def test_mla_decode_long_contexts(dev, orc, ctx, B):
    """The benchmark's long contexts with all 128 heads; the oracle checks a seeded sample of the sequences."""
    import tang_b200 as tb

    H = 128
    rng = np.random.default_rng(ctx + B)
    max_seq = ctx
    w_qk = rng.integers(-127, 128, (H * C_, NOPE), dtype=np.int8)
    s_qk = rng.uniform(0.001, 0.01, H * C_).astype(np.float32)
    w_uv = rng.integers(-127, 128, (H * VD, C_), dtype=np.int8)
    s_uv = rng.uniform(0.001, 0.01, H * VD).astype(np.float32)
    qn = bf16_round(rng.standard_normal((B, H, NOPE)).astype(np.float32))
    qr = bf16_round(rng.standard_normal((B, H, R_)).astype(np.float32))
    lens = [ctx] + [int(v) for v in rng.integers(ctx // 2, ctx + 1, B - 1)]
    sample = [0] if B == 1 else [0, int(rng.integers(1, B))]
    cbuf = dev.alloc(B * max_seq * (C_ + R_), tb.BF16)
    kept = {}
    for b in range(B):                                         # sequence by sequence keeps the host arrays small
        cb = bf16_round(rng.standard_normal((max_seq, C_ + R_)).astype(np.float32))[0]
        dev._check(dev._L.tq_upload(dev._ctx, cbuf.ptr + b * max_seq * (C_ + R_) * 2, cb.ctypes.data, cb.nbytes))
        if b in sample:
            kept[b] = cb
    wq = dev.upload_qarrays(tb.I8_ROW, w_qk, s_qk, H * C_, NOPE)
    wu = dev.upload_qarrays(tb.I8_ROW, w_uv, s_uv, H * VD, C_)
    out = tb.mla_decode(dev, wq, wu, dev.upload(qn[0], tb.BF16), dev.upload(qr[0], tb.BF16), cbuf,
                        np.array(lens, np.int32), B, H, NOPE, VD, max_seq * (C_ + R_), max(lens))
    dev.sync()
    got = out.to_vec().reshape(B, H * VD)
    assert np.all(np.isfinite(got))
    dims = orc.MlaDims(H, C_, NOPE, R_, VD)
    for b in sample:
        want = orc.mla_decode_f64(dims, qn[1][b].astype(np.float64), qr[1][b].astype(np.float64), kept[b], lens[b],
                                  w_qk, s_qk, w_uv, s_uv, absorbed=True)
        assert rel_err(got[b], want, floor_frac=1.0) < 2e-3, (b, lens[b])
