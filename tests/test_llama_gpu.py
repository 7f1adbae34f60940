"""GPU parity of the Llama-shaped decode step against the oracle's restatement of the reference
decode loop (crates/tang-train/examples/smollm.rs:215-296) with the quantised matvec."""
import ctypes as C

import numpy as np
import pytest

from llama_util import HostLlama
from util import bf16_round, rel_err

pytestmark = pytest.mark.gpu

# Activations and the KV cache are bf16 on both sides.  Every operator on its own matches the oracle
# to 1e-4 or better (test_layer_stage_by_stage), but a difference of a few f32 ulps ahead of a bf16
# rounding point flips the rounding of a few percent of the elements by one bf16 ulp (0.4 %), and the
# following projections spread those flips over every output.  End-to-end logits are therefore held
# to the bf16 bar, 2e-2, measured against max(|logit|, rms of the logits).
TOL_LOGITS = 2e-2


def logits_err(got, want):
    return rel_err(got, want, floor_frac=1.0)


@pytest.fixture(scope="module")
def dev():
    import tang_b200

    d = tang_b200.QuantComputeDevice(0)
    yield d
    d.close()


def run_case(dev, orc, host, B, ctx_lens, max_seq, steps=1, interleave=True):
    import tang_b200 as tb

    rng = np.random.default_rng(99)
    kv_dim = host.n_kv * host.hd
    model = host.to_device(dev, max_seq, B, interleave=interleave)
    # prefill caches with bf16 N(0,1) on both sides
    ok, ov = [], []
    for li in range(host.n_layers):
        kb = bf16_round(rng.standard_normal((B, max_seq, kv_dim)).astype(np.float32))[0]
        vb = bf16_round(rng.standard_normal((B, max_seq, kv_dim)).astype(np.float32))[0]
        kbuf, vbuf, stride = model.kv_buffers(li)
        assert stride == max_seq * kv_dim
        dev._check(dev._L.tq_upload(dev._ctx, kbuf.ptr, kb.ctypes.data, kb.nbytes))
        dev._check(dev._L.tq_upload(dev._ctx, vbuf.ptr, vb.ctypes.data, vb.nbytes))
        ok.append(kb.copy())
        ov.append(vb.copy())
    logits = dev.alloc(B * host.vocab, tb.F32)
    pos = np.array(ctx_lens, np.int32)
    for step in range(steps):
        tokens = rng.integers(0, host.vocab, B).astype(np.int32)
        model.decode(dev.upload(tokens, tb.I32), dev.upload(pos, tb.I32), B, int(pos.max()) + 1, logits)
        dev.sync()
        got = logits.to_vec().reshape(B, host.vocab)
        for b in range(B):
            want = host.oracle_decode(orc, int(tokens[b]), [k[b] for k in ok], [v[b] for v in ov], int(pos[b]))
            assert logits_err(got[b], want) < TOL_LOGITS, (step, b)
            top = orc.argmax_f64(want)
            assert got[b][top] >= np.max(got[b]) - 2e-2 * float(np.sqrt(np.mean(want * want)))   # greedy pick within the bar
        # the appended cache rows must hold the same bf16 numbers (a 1-ulp flip at a rounding tie is allowed)
        for li in range(host.n_layers):
            kbuf, vbuf, _ = model.kv_buffers(li)
            kd = kbuf.to_vec().reshape(B, max_seq, kv_dim)
            vd = vbuf.to_vec().reshape(B, max_seq, kv_dim)
            for b in range(B):
                for d_, o_ in ((kd, ok[li]), (vd, ov[li])):
                    a = (d_[b, pos[b]].astype(np.uint32) << 16).view(np.float32)
                    w = (o_[b, pos[b]].astype(np.uint32) << 16).view(np.float32)
                    assert rel_err(a, w, floor_frac=1.0) < 1e-2
        pos = pos + 1
    model.destroy()


def test_small_model_ragged_batch(dev, orc):
    host = HostLlama(np.random.default_rng(1), n_layers=2, d=256, n_heads=4, n_kv=2, hd=128, ffn=512, vocab=1024)
    run_case(dev, orc, host, B=3, ctx_lens=[0, 70, 131], max_seq=160, steps=2)


def test_gate_up_in_the_reference_order_takes_the_separate_swiglu(dev, orc):
    """[gate; up] as the reference concatenates it (no interleaving): same result through the separate operator."""
    host = HostLlama(np.random.default_rng(1), n_layers=2, d=256, n_heads=4, n_kv=2, hd=128, ffn=512, vocab=1024)
    run_case(dev, orc, host, B=3, ctx_lens=[0, 70, 131], max_seq=160, steps=1, interleave=False)
    run_case(dev, orc, host, B=12, ctx_lens=list(range(5, 125, 10)), max_seq=160, steps=1, interleave=True)   # > 8 rows: separate operators


def test_four_to_eight_rows_hand_the_sums_of_squares_over(dev, orc):
    """From four rows on, the output and down projections add the residual themselves and leave each row's sum of
    squares per 16-row block; the pre-norm fused into the next projection adds those instead of reading the row twice."""
    host = HostLlama(np.random.default_rng(4), n_layers=2, d=256, n_heads=4, n_kv=2, hd=128, ffn=512, vocab=1024)
    run_case(dev, orc, host, B=5, ctx_lens=[0, 17, 70, 131, 140], max_seq=160, steps=2)
    run_case(dev, orc, host, B=8, ctx_lens=[3, 0, 64, 65, 127, 128, 129, 150], max_seq=160, steps=1)


def test_llama3_8b_width_four_rows(dev, orc):
    """Full Llama-3-8B layer widths at four rows (K in two slabs, 256 partial sums of squares per row)."""
    host = HostLlama(np.random.default_rng(5), n_layers=2, d=4096, n_heads=32, n_kv=8, hd=128, ffn=14336, vocab=128256)
    run_case(dev, orc, host, B=4, ctx_lens=[600, 0, 257, 31], max_seq=640)


def test_single_sequence_many_heads(dev, orc):
    host = HostLlama(np.random.default_rng(2), n_layers=1, d=512, n_heads=8, n_kv=1, hd=128, ffn=1024, vocab=2048)
    run_case(dev, orc, host, B=1, ctx_lens=[300], max_seq=320)


def test_llama3_8b_width_two_layers(dev, orc):
    """Full Llama-3-8B layer shapes (d 4096, 32/8 heads of 128, FFN 14336, vocab 128256, RoPE theta
    500000), context 2048, two layers."""
    host = HostLlama(np.random.default_rng(3), n_layers=2, d=4096, n_heads=32, n_kv=8, hd=128, ffn=14336, vocab=128256)
    run_case(dev, orc, host, B=2, ctx_lens=[2048, 1000], max_seq=2049)


def test_layer_stage_by_stage(dev, orc):
    """Each operator of one block against the oracle on the SAME inputs (no error carried over):
    norm and RoPE outputs must agree bit for bit after bf16 rounding, projections and attention to
    f32-accumulation accuracy."""
    import tang_b200 as tb
    from llama_util import KIND

    rng = np.random.default_rng(1)
    d, hd, nh, nkv, pos, max_seq = 256, 128, 4, 2, 70, 128
    host = HostLlama(rng, n_layers=1, d=d, n_heads=nh, n_kv=nkv, hd=hd, ffn=512, vocab=1024)
    L = host.layers[0]
    f = lambda bits: (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)
    h = f(host.embed[5]).astype(np.float64)
    xn_o = orc.round_bf16(orc.rms_norm_f64(h, f(L["attn_norm"]).astype(np.float64), 1e-5).astype(np.float32))
    xn_d = dev.rms_norm(dev.upload(h.astype(np.float32)), dev.upload(L["attn_norm"], tb.BF16), 1, d, 1e-5, out_dtype=tb.BF16)
    assert np.count_nonzero(f(xn_d.to_vec()) != xn_o) <= 1

    def lin(name, x):
        sc, pay, r, c = L[name]
        yd = dev.qlinear(x, dev.upload_qarrays(KIND, pay, sc, r, c), 1).to_vec()
        yo = orc.qmatmul(KIND, sc, pay, r, c, f(x.to_vec()).astype(np.float64))
        assert rel_err(yd, yo) < 1e-3, name
        return yd, yo

    (qd, qo), (kd, ko), (vd, _) = lin("wq", xn_d), lin("wk", xn_d), lin("wv", xn_d)
    cos, sin = dev.rope_tables(hd, max_seq, 500000.0)
    qr_d = dev.rope_forward(dev.upload(qd), cos, sin, 1, nh, hd, start_pos=pos, out_dtype=tb.BF16)
    qr_o = orc.round_bf16(orc.rope_heads_f64(qo, nh, hd, pos, 500000.0).astype(np.float32))
    assert np.count_nonzero(f(qr_d.to_vec()) != qr_o) <= 2
    kr_d = dev.rope_forward(dev.upload(kd), cos, sin, 1, nkv, hd, start_pos=pos, out_dtype=tb.BF16)
    kr_o = orc.round_bf16(orc.rope_heads_f64(ko, nkv, hd, pos, 500000.0).astype(np.float32))
    assert np.count_nonzero(f(kr_d.to_vec()) != kr_o) <= 2
    kb = bf16_round(rng.standard_normal((max_seq, nkv * hd)).astype(np.float32))[0]
    vb = bf16_round(rng.standard_normal((max_seq, nkv * hd)).astype(np.float32))[0]
    kb[pos], vb[pos] = kr_d.to_vec(), bf16_round(vd)[0]
    att_d = dev.gqa_decode(qr_d, dev.upload(kb, tb.BF16), dev.upload(vb, tb.BF16), np.array([pos + 1], np.int32), 1, nh, nkv,
                           hd, max_seq * nkv * hd, pos + 1, out_dtype=tb.F32).to_vec()
    att_o = orc.attention_decode_f64(f(qr_d.to_vec()).astype(np.float64), f(kb[:pos + 1]).astype(np.float64),
                                     f(vb[:pos + 1]).astype(np.float64), pos + 1, nh, nkv, hd)
    assert rel_err(att_d, att_o) < 1e-3


def test_prefill_chunk_equals_token_by_token(dev, orc):
    """tq_llama_prefill over a 40-token prompt (tcgen05 GEMMs over all rows, chunk attention) against the oracle's
    token-by-token loop: the last position's logits, the cache rows it appended, and a decode step that follows."""
    import tang_b200 as tb

    host = HostLlama(np.random.default_rng(21), n_layers=2, d=256, n_heads=4, n_kv=2, hd=128, ffn=512, vocab=1024)
    B, P, max_seq = 2, 40, 64
    rng = np.random.default_rng(22)
    prompts = rng.integers(0, host.vocab, (B, P)).astype(np.int32)
    kv_dim = host.n_kv * host.hd
    model = host.to_device(dev, max_seq, B)
    logits = dev.alloc(B * host.vocab, tb.F32)
    model.prefill(dev.upload(prompts, tb.I32), dev.upload(np.zeros(B, np.int32), tb.I32), B, P, logits)
    dev.sync()
    got = logits.to_vec().reshape(B, host.vocab)
    nxt = rng.integers(0, host.vocab, B).astype(np.int32)
    model.decode(dev.upload(nxt, tb.I32), dev.upload(np.full(B, P, np.int32), tb.I32), B, P + 1, logits)
    dev.sync()
    got2 = logits.to_vec().reshape(B, host.vocab)
    for b in range(B):
        kc = [np.zeros((max_seq, kv_dim), np.uint16) for _ in range(host.n_layers)]
        vc = [np.zeros((max_seq, kv_dim), np.uint16) for _ in range(host.n_layers)]
        for p in range(P):
            want = host.oracle_decode(orc, int(prompts[b, p]), kc, vc, p)
        assert logits_err(got[b], want) < TOL_LOGITS, b
        for li in range(host.n_layers):
            kbuf, vbuf, _ = model.kv_buffers(li)
            kd = kbuf.to_vec().reshape(B, max_seq, kv_dim)[b, :P]
            vd = vbuf.to_vec().reshape(B, max_seq, kv_dim)[b, :P]
            f = lambda bits: (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)
            assert rel_err(f(kd), f(kc[li][:P]), floor_frac=1.0) < 2e-2
            assert rel_err(f(vd), f(vc[li][:P]), floor_frac=1.0) < 2e-2
        want2 = host.oracle_decode(orc, int(nxt[b]), kc, vc, P)
        assert logits_err(got2[b], want2) < TOL_LOGITS, b
    # a second chunk continues from the cache: prefill of [0, 24) then [24, 40) gives the same last logits
    m2 = host.to_device(dev, max_seq, B)
    lg2 = dev.alloc(B * host.vocab, tb.F32)
    m2.prefill(dev.upload(np.ascontiguousarray(prompts[:, :24]), tb.I32), dev.upload(np.zeros(B, np.int32), tb.I32), B, 24, lg2)
    m2.prefill(dev.upload(np.ascontiguousarray(prompts[:, 24:]), tb.I32), dev.upload(np.full(B, 24, np.int32), tb.I32), B, P - 24, lg2)
    dev.sync()
    assert logits_err(lg2.to_vec().reshape(B, host.vocab), got) < TOL_LOGITS
    model.destroy()
    m2.destroy()


def test_positions_outside_the_cache_are_reported_not_followed(dev, orc):
    """A position of max_seq or -1 (device-resident, e.g. one replay too many of a generation graph) must not become
    an access outside the cache or the RoPE tables: the row is skipped, the cache keeps its contents, and the next
    tq_sync reports the bad position."""
    import tang_b200 as tb

    host = HostLlama(np.random.default_rng(11), n_layers=1, d=256, n_heads=4, n_kv=2, hd=128, ffn=512, vocab=1024)
    max_seq, B = 32, 2
    kv_dim = host.n_kv * host.hd
    model = host.to_device(dev, max_seq, B)
    kbuf, vbuf, _ = model.kv_buffers(0)
    fill = np.full((B, max_seq, kv_dim), 0x3F80, np.uint16)          # bf16 1.0 everywhere
    for buf in (kbuf, vbuf):
        dev._check(dev._L.tq_upload(dev._ctx, buf.ptr, fill.ctypes.data, fill.nbytes))
    logits = dev.alloc(B * host.vocab, tb.F32)
    tokens = dev.upload(np.array([1, 2], np.int32), tb.I32)
    for bad in (max_seq, -1, max_seq + 1000):
        pos = dev.upload(np.array([3, bad], np.int32), tb.I32)
        model.decode(tokens, pos, B, max_seq, logits)
        with pytest.raises(tb.TangqError) as e:
            dev.sync()
        assert e.value.status == tb._lib.TQ_EINVAL and "position" in str(e.value)
        kd = kbuf.to_vec().reshape(B, max_seq, kv_dim)
        assert np.all(kd[1] == 0x3F80)                               # sequence 1: nothing appended anywhere
        assert np.any(kd[0, 3] != 0x3F80)                            # sequence 0 went through
        fill_row = np.full(kv_dim, 0x3F80, np.uint16)                # put sequence 0's row back for the next round
        kd[0, 3] = fill_row
        dev._check(dev._L.tq_upload(dev._ctx, kbuf.ptr, kd.ctypes.data, kd.nbytes))
    # a good step afterwards works and the status is clean
    model.decode(tokens, dev.upload(np.array([3, 4], np.int32), tb.I32), B, max_seq, logits)
    dev.sync()
    # prefill: a chunk that would run past the cache is refused the same way
    ids = dev.upload(np.zeros((B, 8), np.int32), tb.I32)
    model.prefill(ids, dev.upload(np.array([0, max_seq - 4], np.int32), tb.I32), B, 8, logits)
    with pytest.raises(tb.TangqError) as e:
        dev.sync()
    assert e.value.status == tb._lib.TQ_EINVAL
    model.destroy()


def test_graph_recorded_before_a_workspace_grew_refuses_to_launch(dev, orc):
    """The kernels of a recorded graph hold the addresses of the context's workspaces; once a later call has made a
    workspace grow (free + allocate) the graph must not be replayed."""
    import tang_b200 as tb

    d2 = tb.QuantComputeDevice(0)            # a context of its own: its workspaces start small
    rng = np.random.default_rng(5)
    B, nh, nkv, hd, L = 2, 8, 2, 128, 600
    q = d2.upload(bf16_round(rng.standard_normal((B, nh * hd)).astype(np.float32))[0], tb.BF16)
    kv = d2.upload(bf16_round(rng.standard_normal((B, L, nkv * hd)).astype(np.float32))[0], tb.BF16)
    lens = d2.upload(np.array([L, L // 2], np.int32), tb.I32)
    out = d2.alloc(B * nh * hd, tb.BF16)

    def attend():          # the raw call: nothing in it allocates or synchronises, so it can be recorded
        d2._check(d2._L.tq_gqa_decode(d2._ctx, C.c_void_p(q.ptr), C.c_void_p(kv.ptr), C.c_void_p(kv.ptr), C.c_void_p(lens.ptr),
                                      B, nh, nkv, hd, L * nkv * hd, L, C.c_void_p(out.ptr), tb.BF16))

    attend()               # eager: sizes the partials' workspace
    d2.sync()
    d2.begin_capture()
    attend()
    g = d2.end_capture()
    g.launch()
    d2.sync()
    first = out.to_vec().copy()
    # a call that needs a larger workspace makes it grow (freed and allocated anew): 600 host vectors of 1024
    # doubles through the reference-shaped matvec call stage about 15 MB in the same workspace
    from util import make_weight

    sc, pay = make_weight(rng, 1, 1024, 1024)
    w = d2.upload_qarrays(1, pay, sc, 1024, 1024)
    d2.q_matmul_host(w, rng.standard_normal((600, 1024)), 600)
    d2.sync()
    with pytest.raises(tb.TangqError) as e:
        g.launch()
    assert e.value.status == tb._lib.TQ_EINVAL and "record" in str(e.value)
    # recording it again works and gives the same numbers
    d2.memset(out)
    d2.begin_capture()
    attend()
    g2 = d2.end_capture()
    g2.launch()
    d2.sync()
    assert np.array_equal(out.to_vec(), first)
    d2.close()


@pytest.mark.parametrize("B", [16, 64])
def test_llama3_8b_width_decode_batches(dev, orc, B):
    """The benchmark's decode batches at full Llama-3-8B layer widths (two layers, context 2048): from 17 rows on
    every linear layer of the step runs on the tcgen05 GEMM (split K for the narrow ones), which the small batches
    above never reach.  The oracle checks a seeded sample of the sequences."""
    import tang_b200 as tb

    host = HostLlama(np.random.default_rng(3), n_layers=2, d=4096, n_heads=32, n_kv=8, hd=128, ffn=14336, vocab=128256)
    rng = np.random.default_rng(700 + B)
    max_seq = 2049
    kv_dim = host.n_kv * host.hd
    model = host.to_device(dev, max_seq, B)
    sample = np.sort(rng.choice(B, 3, replace=False))
    pos = rng.integers(1500, 2049, B).astype(np.int32)
    pos[sample[0]] = 2048
    ok, ov = {}, {}
    for li in range(host.n_layers):
        kbuf, vbuf, stride = model.kv_buffers(li)
        for b in range(B):       # sequence by sequence keeps the host arrays small
            kb = bf16_round(rng.standard_normal((max_seq, kv_dim)).astype(np.float32))[0]
            vb = bf16_round(rng.standard_normal((max_seq, kv_dim)).astype(np.float32))[0]
            dev._check(dev._L.tq_upload(dev._ctx, kbuf.ptr + b * stride * 2, kb.ctypes.data, kb.nbytes))
            dev._check(dev._L.tq_upload(dev._ctx, vbuf.ptr + b * stride * 2, vb.ctypes.data, vb.nbytes))
            if b in sample:
                ok[(li, b)], ov[(li, b)] = kb, vb
    tokens = rng.integers(0, host.vocab, B).astype(np.int32)
    logits = dev.alloc(B * host.vocab, tb.F32)
    model.decode(dev.upload(tokens, tb.I32), dev.upload(pos, tb.I32), B, 2049, logits)
    dev.sync()
    got = logits.to_vec().reshape(B, host.vocab)
    assert np.all(np.isfinite(got))
    for b in sample:
        want = host.oracle_decode(orc, int(tokens[b]), [ok[(li, b)] for li in range(host.n_layers)],
                                  [ov[(li, b)] for li in range(host.n_layers)], int(pos[b]))
        assert logits_err(got[b], want) < TOL_LOGITS, b
    model.destroy()


def test_trimmed_cache_keeps_the_last_tokens(dev, orc):
    """KVCache::trim_to (crates/tang-infer/src/kv_cache.rs:138-149): every sequence keeps its LAST `keep` positions, moved
    to the front of its cache rows in every layer; shorter sequences are untouched.  The device cache after
    tq_llama_kv_trim equals the oracle's trimmed rows bit for bit, and a decode step on top of it (appended at row
    `keep`, rotated for the running position) matches the oracle run on the trimmed rows."""
    import tang_b200 as tb

    host = HostLlama(np.random.default_rng(21), n_layers=2, d=256, n_heads=4, n_kv=2, hd=128, ffn=512, vocab=1024)
    rng = np.random.default_rng(22)
    B, max_seq, keep = 3, 160, 64
    lens = np.array([131, 20, 65], np.int32)            # 131 and 65 are trimmed to 64, 20 stays
    kv_dim = host.n_kv * host.hd
    model = host.to_device(dev, max_seq, B)
    ok, ov = [], []
    for li in range(host.n_layers):
        kb = bf16_round(rng.standard_normal((B, max_seq, kv_dim)).astype(np.float32))[0]
        vb = bf16_round(rng.standard_normal((B, max_seq, kv_dim)).astype(np.float32))[0]
        kbuf, vbuf, _ = model.kv_buffers(li)
        dev._check(dev._L.tq_upload(dev._ctx, kbuf.ptr, kb.ctypes.data, kb.nbytes))
        dev._check(dev._L.tq_upload(dev._ctx, vbuf.ptr, vb.ctypes.data, vb.nbytes))
        ok.append(kb.copy())
        ov.append(vb.copy())
    lens_dev = dev.upload(lens, tb.I32)
    model.trim_to(lens_dev, B, keep)
    dev.sync()
    new_lens = lens_dev.to_vec()
    want_lens = []
    for b in range(B):
        want_lens.append(orc.kv_trim_to(ok[0][b], int(lens[b]), keep))
        orc.kv_trim_to(ov[0][b], int(lens[b]), keep)
        for li in range(1, host.n_layers):
            orc.kv_trim_to(ok[li][b], int(lens[b]), keep)
            orc.kv_trim_to(ov[li][b], int(lens[b]), keep)
    assert list(new_lens) == want_lens == [64, 20, 64]
    for li in range(host.n_layers):
        kbuf, vbuf, _ = model.kv_buffers(li)
        kd = kbuf.to_vec().reshape(B, max_seq, kv_dim)
        vd = vbuf.to_vec().reshape(B, max_seq, kv_dim)
        for b in range(B):
            n = want_lens[b]
            assert np.array_equal(kd[b, :n], ok[li][b, :n]) and np.array_equal(vd[b, :n], ov[li][b, :n]), (li, b)
    # one decode step on the trimmed caches: cache row = new length, rotation = the running position
    tokens = rng.integers(0, host.vocab, B).astype(np.int32)
    logits = dev.alloc(B * host.vocab, tb.F32)
    model.decode(dev.upload(tokens, tb.I32), lens_dev, B, keep + 1, logits, rope_positions=dev.upload(lens, tb.I32))
    dev.sync()
    got = logits.to_vec().reshape(B, host.vocab)
    for b in range(B):
        want = host.oracle_decode(orc, int(tokens[b]), [k[b] for k in ok], [v[b] for v in ov], want_lens[b], rope_pos=int(lens[b]))
        assert logits_err(got[b], want) < TOL_LOGITS, b
    # keep >= every length: nothing moves
    model.trim_to(lens_dev, B, max_seq)
    dev.sync()
    assert list(lens_dev.to_vec()) == want_lens
    model.destroy()
