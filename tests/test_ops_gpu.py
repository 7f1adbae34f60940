"""GPU parity of the small decode-step operators and of decode attention against the CPU oracle
(the restated CpuDevice functions, crates/tang-compute/src/cpu.rs / device.rs)."""
import numpy as np
import pytest

from util import bf16_round, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import tang_b200

    d = tang_b200.QuantComputeDevice(0)
    yield d
    d.close()


def bf16_to_f32(bits):
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def test_rms_norm(dev, orc):
    import tang_b200 as tb

    rng = np.random.default_rng(0)
    for n, dim in [(1, 4096), (5, 576), (3, 100), (2, 8192)]:
        x = rng.standard_normal((n, dim)).astype(np.float32)
        w = rng.normal(1, 0.1, dim).astype(np.float32)
        got = dev.rms_norm(dev.upload(x), dev.upload(w), n, dim, 1e-5).to_vec()
        assert rel_err(got, orc.rms_norm_f32(x, w, n, dim, 1e-5)) < 1e-5
        res = rng.standard_normal((n, dim)).astype(np.float32)
        out, s = dev.rms_norm_residual(dev.upload(x), dev.upload(res), dev.upload(w), n, dim, 1e-6)
        want, want_s = orc.rms_norm_residual_f32(x, res, w, n, dim, 1e-6)
        assert np.array_equal(s.to_vec(), want_s) and rel_err(out.to_vec(), want) < 1e-5
        # bf16 gains and bf16 output, as the decode step uses it
        wb, wf = bf16_round(w)
        got16 = dev.rms_norm(dev.upload(x), dev.upload(wb, tb.BF16), n, dim, 1e-5, out_dtype=tb.BF16).to_vec()
        assert rel_err(bf16_to_f32(got16), orc.rms_norm_f32(x, wf, n, dim, 1e-5)) < 2e-2


def test_rope(dev, orc):
    import tang_b200 as tb

    rng = np.random.default_rng(1)
    cos, sin = dev.rope_tables(128, 4096, 500000.0)
    oc, osn = orc.rope_tables_f32(128, 4096, 500000.0)
    assert np.array_equal(cos.to_vec(), oc) and np.array_equal(sin.to_vec(), osn)   # f64 host math, same libm
    x = rng.standard_normal((5, 8, 128)).astype(np.float32)
    got = dev.rope_forward(dev.upload(x), cos, sin, 5, 8, 128, start_pos=2040).to_vec()
    assert rel_err(got, orc.rope_forward_f32(x, oc, osn, 5, 8, 128, 2040)) < 1e-5   # the GPU fuses x0*c - x1*s
    # identity at position 0 (modules.rs:717-728)
    c4, s4 = dev.rope_tables(4, 32, 10000.0)
    assert np.allclose(dev.rope_forward(dev.upload([1, 2, 3, 4]), c4, s4, 1, 1, 4, 0).to_vec(), [1, 2, 3, 4], atol=1e-5)
    # per-row positions (decode: one token per sequence)
    pos = np.array([7, 0, 2047, 33], np.int32)
    x = rng.standard_normal((4, 2, 128)).astype(np.float32)
    got = dev.rope_forward(dev.upload(x), cos, sin, 4, 2, 128, positions=dev.upload(pos, tb.I32)).to_vec().reshape(4, -1)
    for r in range(4):
        assert rel_err(got[r], orc.rope_forward_f32(x[r], oc, osn, 1, 2, 128, int(pos[r]))) < 1e-5


def test_swiglu_and_embedding(dev, orc):
    import tang_b200 as tb

    rng = np.random.default_rng(2)
    g, u = rng.standard_normal(1000).astype(np.float32) * 3, rng.standard_normal(1000).astype(np.float32)
    assert rel_err(dev.swiglu_fused(dev.upload(g), dev.upload(u)).to_vec(), orc.swiglu_f32(g, u)) < 1e-5
    v = dev.swiglu_fused(dev.upload([0, 1, -1]), dev.upload([1, 1, 1])).to_vec()      # ops.rs:216-229
    assert abs(v[0]) < 1e-5 and abs(v[1] - 0.7311) < 1e-3 and abs(v[2] + 0.2689) < 1e-3
    w = rng.standard_normal((50, 64)).astype(np.float32)
    ids = np.array([3, 49, 0, 3], np.int32)
    got = dev.embedding(dev.upload(w), ids, 4, 64).to_vec()
    assert np.array_equal(got, orc.embedding_f32(w, ids.astype(np.uint32), 64))


def test_kv_attention_reference_signature(dev, orc):
    rng = np.random.default_rng(3)
    # the reference's own cases (cpu.rs:938-983)
    out = dev.kv_attention(dev.upload([1, 0]), dev.upload([1, 0]), dev.upload([1, 2]), 0, 1, 1, 1, 2).to_vec()
    assert abs(out[0] - 1) < 1e-4 and abs(out[1] - 2) < 1e-4
    q = k = [1, 0, 0, 1, 1, 1]
    out = dev.kv_attention(dev.upload(q), dev.upload(k), dev.upload([1, 2, 3, 4, 5, 6]), 0, 3, 1, 1, 2).to_vec()
    assert np.allclose(out, orc.kv_attention_f32(q, k, [1, 2, 3, 4, 5, 6], 0, 3, 1, 1, 2), atol=1e-5)
    # GQA shapes, decode and prefill
    for (cs, ql, nh, nkv, hd) in [(100, 1, 8, 2, 64), (0, 7, 4, 4, 32), (33, 5, 9, 3, 64), (2048, 1, 32, 8, 128)]:
        total = cs + ql
        qv = rng.standard_normal((ql, nh * hd)).astype(np.float32)
        kv = rng.standard_normal((total, nkv * hd)).astype(np.float32)
        vv = rng.standard_normal((total, nkv * hd)).astype(np.float32)
        got = dev.kv_attention(dev.upload(qv), dev.upload(kv), dev.upload(vv), cs, ql, nh, nkv, hd).to_vec()
        assert rel_err(got, orc.kv_attention_f32(qv, kv, vv, cs, ql, nh, nkv, hd)) < 1e-3


@pytest.mark.parametrize("B,nh,nkv,lens", [(1, 32, 8, [2049]), (3, 8, 2, [1, 70, 200]), (2, 4, 4, [64, 65]),
                                           (5, 16, 2, [17, 128, 129, 1000, 513]), (16, 32, 8, [2049] * 16)])
def test_gqa_decode_bf16_cache(dev, orc, B, nh, nkv, lens):
    """Batched decode attention over a bf16 cache vs the f64 attention of the decode loop
    (crates/tang-train/examples/smollm.rs:101-154) on the same bf16 values."""
    import tang_b200 as tb

    rng = np.random.default_rng(B * 100 + nh)
    hd, max_seq = 128, max(lens) + 3
    kv_dim = nkv * hd
    qb, qf = bf16_round(rng.standard_normal((B, nh * hd)).astype(np.float32))
    kb, kf = bf16_round(rng.standard_normal((B, max_seq, kv_dim)).astype(np.float32))
    vb, vf = bf16_round(rng.standard_normal((B, max_seq, kv_dim)).astype(np.float32))
    out = dev.gqa_decode(dev.upload(qb, tb.BF16), dev.upload(kb, tb.BF16), dev.upload(vb, tb.BF16), np.array(lens, np.int32),
                         B, nh, nkv, hd, max_seq * kv_dim, max(lens), out_dtype=tb.F32).to_vec().reshape(B, nh * hd)
    for b in range(B):
        want = orc.attention_decode_f64(qf[b], kf[b, :lens[b]], vf[b, :lens[b]], lens[b], nh, nkv, hd)
        assert rel_err(out[b], want) < 1e-3, (b, lens[b])      # f32-accumulated; P carries 16 bits
    out16 = dev.gqa_decode(dev.upload(qb, tb.BF16), dev.upload(kb, tb.BF16), dev.upload(vb, tb.BF16), np.array(lens, np.int32),
                           B, nh, nkv, hd, max_seq * kv_dim, max(lens)).to_vec().reshape(B, nh * hd)
    assert np.array_equal(out16, bf16_round(out)[0])


@pytest.mark.parametrize("B,nh,nkv,q_len,starts", [(2, 8, 2, 50, [0, 37]),        # group 4, ragged chunk, a cached prefix
                                                  (1, 4, 4, 64, [0]),            # no grouping, exactly one CTA tile of positions
                                                  (1, 8, 1, 33, [100]),          # group 8 (8 positions per CTA)
                                                  (3, 4, 2, 130, [0, 5, 63]),    # several query tiles, tile-boundary prefixes
                                                  (1, 32, 8, 512, [0])])         # Llama-3-8B heads, a 512-token chunk
def test_gqa_prefill_causal_chunk(dev, orc, B, nh, nkv, q_len, starts):
    """kv_attention with q_len > 1 (device.rs:161-180; cpu.rs:257-315) on bf16 caches: query i attends positions
    0 .. cache_start + i.  Probabilities pass through bf16 on their way into the tensor core, so the bar is the
    bf16 one, measured against max(|ref|, rms)."""
    import tang_b200 as tb

    rng = np.random.default_rng(B * 1000 + nh + q_len)
    hd = 128
    max_seq = max(starts) + q_len + 3
    kv_dim = nkv * hd
    qb, qf = bf16_round(rng.standard_normal((B, q_len, nh * hd)).astype(np.float32))
    kb, kf = bf16_round(rng.standard_normal((B, max_seq, kv_dim)).astype(np.float32))
    vb, vf = bf16_round(rng.standard_normal((B, max_seq, kv_dim)).astype(np.float32))
    out = dev.gqa_prefill(dev.upload(qb, tb.BF16), dev.upload(kb, tb.BF16), dev.upload(vb, tb.BF16), np.array(starts, np.int32),
                          B, q_len, nh, nkv, hd, max_seq * kv_dim, out_dtype=tb.F32)
    dev.sync()
    got = out.to_vec().reshape(B, q_len, nh * hd)
    pick = range(q_len) if q_len <= 64 else sorted(set([0, 1, 15, 16, 63, 64, q_len // 2, q_len - 2, q_len - 1]))
    for b in range(B):
        for i in pick:
            n = starts[b] + i + 1
            want = orc.attention_decode_f64(qf[b, i], kf[b, :n], vf[b, :n], n, nh, nkv, hd)
            assert rel_err(got[b, i], want, floor_frac=1.0) < 1e-2, (b, i)
    out16 = dev.gqa_prefill(dev.upload(qb, tb.BF16), dev.upload(kb, tb.BF16), dev.upload(vb, tb.BF16), np.array(starts, np.int32),
                            B, q_len, nh, nkv, hd, max_seq * kv_dim).to_vec().reshape(B, q_len, nh * hd)
    assert np.array_equal(out16, bf16_round(got)[0])
    # a chunk of one position is the decode case
    dec = dev.gqa_decode(dev.upload(np.ascontiguousarray(qb[:, 0]), tb.BF16), dev.upload(kb, tb.BF16), dev.upload(vb, tb.BF16),
                         np.array([s + 1 for s in starts], np.int32), B, nh, nkv, hd, max_seq * kv_dim, max(starts) + 1,
                         out_dtype=tb.F32).to_vec().reshape(B, nh * hd)
    assert rel_err(got[:, 0], dec, floor_frac=1.0) < 1e-2
