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


# ---- the MLA layer: q_a -> RMSNorm -> q_b -> RoPE -> absorbed attention -> W_UV -> row-parallel W_O ----------------
def _i8_matvec(w, s, x):
    """(w * s[:, None]) @ x in f64, a block of rows at a time (int8 weights, one f32 scale per row)."""
    out = np.empty(w.shape[0], np.float64)
    for r in range(0, w.shape[0], 2048):
        out[r:r + 2048] = (w[r:r + 2048].astype(np.float64) @ x) * s[r:r + 2048].astype(np.float64)
    return out


def _layer_weights(rng, d, H, q_lora):
    def mat(rows, cols):
        return rng.integers(-127, 128, (rows, cols), dtype=np.int8), rng.uniform(0.001, 0.01, rows).astype(np.float32)
    w = {"q_a": mat(q_lora, d), "q_b": mat(H * (NOPE + R_), q_lora), "w_qk": mat(H * C_, NOPE), "w_uv": mat(H * VD, C_),
         "w_o": mat(d, H * VD)}
    # a small gain keeps the queries (and with them the softmax) in a realistic range
    gain = bf16_round((0.03 * (1.0 + 0.1 * rng.standard_normal(q_lora))).astype(np.float32))
    return w, gain


def _layer_oracle(orc, w, gain, h, cache_b, length, H, heads, base, eps, max_pos):
    """Output of the heads in `heads` (a slice) for one sequence; the device's bf16 rounding points mirrored."""
    cq = _i8_matvec(*w["q_a"], h).astype(np.float32).astype(np.float64)
    xn = bf16_round(orc.rms_norm_f64(cq, gain[1].astype(np.float64), eps).astype(np.float32))[1].astype(np.float64)
    qh = NOPE + R_
    rows = slice(heads.start * qh, heads.stop * qh)
    q = bf16_round(_i8_matvec(w["q_b"][0][rows], w["q_b"][1][rows], xn).astype(np.float32))[1].reshape(-1, qh)
    nh = q.shape[0]
    cos, sin = orc.rope_tables_f32(R_, max_pos, base)
    pos = length - 1
    c, s = cos.reshape(max_pos, R_ // 2)[pos], sin.reshape(max_pos, R_ // 2)[pos]
    x0, x1 = q[:, NOPE::2], q[:, NOPE + 1::2]
    qr = np.empty((nh, R_), np.float32)
    qr[:, 0::2] = x0 * c - x1 * s
    qr[:, 1::2] = x0 * s + x1 * c
    qr = bf16_round(qr)[1]
    dims = orc.MlaDims(nh, C_, NOPE, R_, VD)
    hs = slice(heads.start * C_, heads.stop * C_)
    vs = slice(heads.start * VD, heads.stop * VD)
    o = orc.mla_decode_f64(dims, q[:, :NOPE].astype(np.float64), qr.astype(np.float64), cache_b, length, w["w_qk"][0][hs],
                           w["w_qk"][1][hs], w["w_uv"][0][vs], w["w_uv"][1][vs], absorbed=True)
    o = bf16_round(np.asarray(o, np.float32))[1].astype(np.float64)
    return _i8_matvec(np.ascontiguousarray(w["w_o"][0][:, vs]), w["w_o"][1], o)


def _make_layer(dev, tb, w, gain, d, H, heads, q_lora, max_batch, max_pos, base, eps):
    qh = NOPE + R_
    nh = heads.stop - heads.start
    up = lambda a, s, r, c: dev.upload_qarrays(tb.I8_ROW, np.ascontiguousarray(a), np.ascontiguousarray(s), r, c)
    cfg = tb.MlaConfig(d, nh, q_lora, C_, NOPE, R_, VD, max_batch, max_pos, eps)
    return tb.MlaLayer(
        dev, cfg, up(*w["q_a"], q_lora, d), dev.upload(gain[0], tb.BF16),
        up(w["q_b"][0][heads.start * qh:heads.stop * qh], w["q_b"][1][heads.start * qh:heads.stop * qh], nh * qh, q_lora),
        up(w["w_qk"][0][heads.start * C_:heads.stop * C_], w["w_qk"][1][heads.start * C_:heads.stop * C_], nh * C_, NOPE),
        up(w["w_uv"][0][heads.start * VD:heads.stop * VD], w["w_uv"][1][heads.start * VD:heads.stop * VD], nh * VD, C_),
        up(w["w_o"][0][:, heads.start * VD:heads.stop * VD], w["w_o"][1], d, nh * VD), rope_base=base)


@pytest.mark.gpu
@pytest.mark.parametrize("d,H,q_lora,B,lens", [(1024, 32, 512, 3, [5, 300, 64]), (7168, 128, 1536, 2, [700, 129]),
                                                (1024, 32, 512, 12, [40 + 17 * i for i in range(12)])])
def test_mla_layer_matches_oracle(dev, orc, d, H, q_lora, B, lens):
    """The whole layer at the DeepSeek-V3 widths (d_model 7168 is an assumption: the benchmark configuration names
    no hidden size), batches on both sides of the 8-row GEMV limit, and the heads split over two ranks' worth of
    weights whose outputs must add up to the unsharded result (the row-parallel W_O)."""
    import tang_b200 as tb

    rng = np.random.default_rng(d + H + B)
    base, eps, max_pos = 10000.0, 1e-6, max(lens) + 3
    max_seq = max(lens) + 2
    w, gain = _layer_weights(rng, d, H, q_lora)
    h = bf16_round(rng.standard_normal((B, d)).astype(np.float32))
    cache = bf16_round(rng.standard_normal((B, max_seq, C_ + R_)).astype(np.float32))
    hb, cb = dev.upload(h[0], tb.BF16), dev.upload(cache[0], tb.BF16)
    lb = dev.upload(np.array(lens, np.int32), tb.I32)
    full = _make_layer(dev, tb, w, gain, d, H, slice(0, H), q_lora, B, max_pos, base, eps)
    got = full.decode(hb, cb, lb, B, max_seq * (C_ + R_), max(lens))
    dev.sync()
    got = got.to_vec().reshape(B, d)
    for b in range(B if d < 7168 else 1):
        want = _layer_oracle(orc, w, gain, h[1][b].astype(np.float64), cache[0][b], lens[b], H, slice(0, H), base, eps, max_pos)
        # four bf16 hand-overs (c_q, q, q_lat, o_lat | o) on both sides: where the device's f32 sum and the oracle's
        # f64 sum land on different sides of a bf16 rounding boundary the result moves by a few 1e-3 of its rms
        # (observed: up to 3.6e-3); the bar is half of the 2e-2 allowed for bf16 outputs
        assert rel_err(got[b], want, floor_frac=1.0) < 1e-2, (b, lens[b])
    # two head shards, each with its rows of q_b / W_UK / W_UV and its columns of W_O: partial outputs add up
    parts = []
    for heads in (slice(0, H // 2), slice(H // 2, H)):
        layer = _make_layer(dev, tb, w, gain, d, H, heads, q_lora, B, max_pos, base, eps)
        o = layer.decode(hb, cb, lb, B, max_seq * (C_ + R_), max(lens))
        dev.sync()
        parts.append(o.to_vec().reshape(B, d).astype(np.float64))
        layer.destroy()
    # (a shard's projections have other shapes than the full layer's, so their f32 sums run in another order and a
    # bf16 hand-over can round the other way: a few 1e-3 of the rms on the rows where that happens)
    assert rel_err(parts[0] + parts[1], got, floor_frac=1.0) < 5e-3
    # graph capture: the layer allocates nothing while it runs
    out2 = dev.alloc(B * d, tb.F32)
    dev.begin_capture()
    full.decode(hb, cb, lb, B, max_seq * (C_ + R_), max(lens), out=out2)
    g = dev.end_capture()
    g.launch()
    dev.sync()
    assert np.array_equal(out2.to_vec().reshape(B, d), got.astype(np.float32))
    g.free()
    full.destroy()
