"""Greedy sampling and the generation loop on the device (crates/tang-infer/src/sampling.rs:108-111,
183-194 argmax with the first maximum winning; :229-256 generate)."""
import numpy as np
import pytest

from llama_util import HostLlama

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import tang_b200

    d = tang_b200.QuantComputeDevice(0)
    yield d
    d.close()


def test_argmax_reference_cases(dev, orc):
    """sampling.rs:265-296: greedy picks token 2 of [1,3,10,2], token 1 of [1,5,3], token 2 of [1,2,5,3]."""
    for row, want in (([1.0, 3.0, 10.0, 2.0], 2), ([1.0, 5.0, 3.0], 1), ([1.0, 2.0, 5.0, 3.0], 2)):
        x = np.array(row, np.float32)
        assert orc.argmax_f64(x.astype(np.float64)) == want
        assert dev.argmax_rows(dev.upload(x), 1, x.size).to_vec()[0] == want


@pytest.mark.parametrize("rows,cols", [(1, 5), (3, 1000), (4, 128256), (64, 4099)])
def test_argmax_first_maximum_bit_exact(dev, orc, rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    x[0, :] = np.float32(0.5)                       # all equal: index 0
    if rows > 1:
        j = rng.integers(0, cols, 5)
        x[1, j] = np.float32(9.0)                   # several exact ties at the top: the lowest index
        x[1, j.min() - 1 if j.min() > 0 else 0] = np.float32(np.nan) if j.min() > 0 else x[1, 0]
    if rows > 2:
        x[2, :] = -np.inf                           # nothing exceeds -inf: 0
        x[2, cols // 2] = np.nan
    got = dev.argmax_rows(dev.upload(x), rows, cols).to_vec()
    want = [orc.argmax_f64(r.astype(np.float64)) for r in x]
    assert list(got) == want


def test_argmax_over_rank_major_slices(dev, orc):
    """A vocabulary gathered from 4 tensor-parallel ranks: [slice][row][cols]; index = slice*cols + col."""
    rng = np.random.default_rng(5)
    S, R, Cc = 4, 3, 501
    full = rng.standard_normal((R, S * Cc)).astype(np.float32)
    sliced = np.ascontiguousarray(full.reshape(R, S, Cc).transpose(1, 0, 2))
    got = dev.argmax_rows(dev.upload(sliced), R, Cc, slices=S).to_vec()
    assert list(got) == [orc.argmax_f64(r.astype(np.float64)) for r in full]


def test_generate_greedy_follows_the_oracle(dev, orc):
    """Prompt of 3 tokens, 4 generated, batch 2.  The device never downloads logits; every token it chose must
    be the oracle's greedy choice for the same prefix, or tie with it inside the logits' parity bar (2e-2 of
    the logits' rms: the bf16 pipeline's end-to-end tolerance)."""
    host = HostLlama(np.random.default_rng(11), n_layers=2, d=256, n_heads=4, n_kv=2, hd=128, ffn=512, vocab=1024)
    B, P, N, max_seq = 2, 3, 4, 16
    prompts = np.array([[5, 17, 900], [44, 3, 271]], np.int32)
    model = host.to_device(dev, max_seq, B)
    out = model.generate_greedy(prompts, N)
    assert out.shape == (B, N)
    kv_dim = host.n_kv * host.hd
    for b in range(B):
        kc = [np.zeros((max_seq, kv_dim), np.uint16) for _ in range(host.n_layers)]
        vc = [np.zeros((max_seq, kv_dim), np.uint16) for _ in range(host.n_layers)]
        seq = list(prompts[b])
        for p in range(P + N - 1):
            logits = host.oracle_decode(orc, int(seq[p]), kc, vc, p)
            if p >= P - 1:
                tok = int(out[b, p - (P - 1)])
                rms = float(np.sqrt(np.mean(logits * logits)))
                assert logits[tok] >= logits.max() - 2e-2 * rms, (b, p, tok, orc.argmax_f64(logits))
                seq.append(tok)                    # follow the device's choice so that prefixes stay equal
    # the same call again gives the same tokens (the graph replays deterministically)
    model2 = host.to_device(dev, max_seq, B)
    assert np.array_equal(model2.generate_greedy(prompts, N), out)
    model.destroy()
    model2.destroy()


def _draws(dev, orc, logits, cfg_vals, seeds, n_draws, past=None, slices=1):
    """`n_draws` successive tq_sample calls on the same logits [rows, V] against the oracle's Sampler, row by row."""
    import tang_b200 as tb

    rows, V = logits.shape
    x = logits
    if slices > 1:
        x = np.ascontiguousarray(logits.reshape(rows, slices, V // slices).transpose(1, 0, 2))
    xb = dev.upload(x.astype(np.float32))
    st = dev.upload(np.array(seeds, np.uint64).view(np.float64), tb.F64)
    cfg = tb.SamplerConfig(*cfg_vals)
    pb = lb = None
    ld = 0
    if past is not None:
        ld = max(len(p) for p in past)
        arr = np.zeros((rows, ld), np.int32)
        for r, p in enumerate(past):
            arr[r, :len(p)] = p
        pb, lb = dev.upload(arr, tb.I32), dev.upload(np.array([len(p) for p in past], np.int32), tb.I32)
    got = np.stack([dev.sample(xb, rows, V // slices, cfg, st, pb, lb, ld, slices=slices).to_vec() for _ in range(n_draws)], axis=1)
    dev.sync()
    ocfg = orc.SamplerConfig(*cfg_vals)
    want = np.zeros_like(got)
    final = []
    for r in range(rows):
        s = int(seeds[r])
        for j in range(n_draws):
            want[r, j], s = orc.sampler_sample(logits[r].astype(np.float32).astype(np.float64), ocfg, s, past[r] if past is not None else ())
        final.append(s)
    if cfg_vals[0] != 0.0:
        assert list(st.to_vec().view(np.uint64)) == final          # the LCG states advanced exactly as the reference's
    return got, want


def test_sampler_reference_cases_on_device(dev, orc):
    """sampling.rs:298-340: top_k = 2 over [1, 100, 0.1, 99] only ever yields tokens 1 and 3 (seed 12345);
    top_p = 0.5 over [10, 0, 0, 0] always yields 0 (seed 99)."""
    got, want = _draws(dev, orc, np.array([[1.0, 100.0, 0.1, 99.0]]), (1.0, 2, 1.0, 1.0), [12345], 100)
    assert np.array_equal(got, want) and set(got[0]) == {1, 3}
    got, want = _draws(dev, orc, np.array([[10.0, 0.0, 0.0, 0.0]]), (1.0, 0, 0.5, 1.0), [99], 20)
    assert np.array_equal(got, want) and set(got[0]) == {0}


@pytest.mark.parametrize("cfg", [(0.7, 40, 0.9, 1.0),      # SamplingConfig::standard()
                                 (1.0, 5, 1.0, 1.0),       # top-k only
                                 (1.3, 50, 0.6, 1.0),
                                 (1.0, 1, 1.0, 1.0)])
def test_sampler_matches_the_oracle_draw_for_draw(dev, orc, cfg):
    rng = np.random.default_rng(int(cfg[1]) + 17)
    logits = (rng.standard_normal((4, 32000)) * 3).astype(np.float32)
    logits[1, [7, 900, 31999]] = logits[1].max() + 1.0        # exact ties at the top
    got, want = _draws(dev, orc, logits, cfg, [1, 2, 3, 2 ** 63 + 5], 40)
    assert np.array_equal(got, want)


def test_sampler_repetition_penalty_and_greedy(dev, orc):
    rng = np.random.default_rng(4)
    logits = rng.standard_normal((3, 5000)).astype(np.float32)
    past = [[int(np.argmax(logits[0]))] * 3 + [5, 9], [], list(range(0, 5000, 7))]
    for cfg in ((0.0, 0, 1.0, 1.7), (0.8, 20, 0.95, 1.3)):
        got, want = _draws(dev, orc, logits, cfg, [11, 12, 13], 10, past=past)
        assert np.array_equal(got, want)


def test_sampler_without_top_k_and_over_rank_major_slices(dev, orc):
    """top_k off: more than 1024 probabilities survive, so the sums are block reductions and the nucleus threshold a
    weighted radix selection (a draw can differ from the reference only when a running sum lands within rounding
    of a threshold: not in these seeds)."""
    rng = np.random.default_rng(8)
    logits = (rng.standard_normal((2, 6000)) * 2).astype(np.float32)
    for cfg in ((1.0, 0, 1.0, 1.0), (0.9, 0, 0.8, 1.0)):
        got, want = _draws(dev, orc, logits, cfg, [21, 22], 30, slices=4)
        assert np.array_equal(got, want)


def test_sampler_llama3_vocabulary(dev, orc):
    rng = np.random.default_rng(9)
    logits = (rng.standard_normal((2, 128256)) * 4).astype(np.float32)
    got, want = _draws(dev, orc, logits, (0.7, 40, 0.9, 1.0), [5, 6], 8)
    assert np.array_equal(got, want)


def test_generate_with_sampling_equals_oracle_sampler_on_the_device_logits(dev, orc):
    """generate() with temperature / top-k / top-p / repetition penalty: tokens are drawn on the device inside the
    replayed graph.  A second model instance is stepped by hand, its logits downloaded and given to the oracle's
    Sampler (same seed, same past tokens): both must produce the same tokens, draw for draw."""
    import tang_b200 as tb

    host = HostLlama(np.random.default_rng(12), n_layers=2, d=256, n_heads=4, n_kv=2, hd=128, ffn=512, vocab=1024)
    B, P, N, max_seq = 3, 2, 6, 16
    prompts = np.array([[5, 17], [44, 3], [5, 17]], np.int32)
    vals = (0.9, 30, 0.92, 1.3)
    model = host.to_device(dev, max_seq, B)
    out = model.generate(prompts, N, tb.SamplerConfig(*vals), seed=77)
    assert out.shape == (B, N) and out.min() >= 0 and out.max() < host.vocab
    assert np.array_equal(out[0], out[2])                      # same prompt, same seed: same continuation
    model.destroy()
    # by hand, with downloads
    ref = host.to_device(dev, max_seq, B)
    logits = dev.alloc(B * host.vocab, tb.F32)
    ocfg = orc.SamplerConfig(*vals)
    states = [77] * B
    seqs = [list(p) for p in prompts]
    ref.prefill(dev.upload(np.ascontiguousarray(prompts[:, :P - 1]), tb.I32), dev.upload(np.zeros(B, np.int32), tb.I32), B, P - 1, logits)
    for p in range(P - 1, P + N - 1):
        tok = np.array([s[p] for s in seqs], np.int32)
        ref.decode(dev.upload(tok, tb.I32), dev.upload(np.full(B, p, np.int32), tb.I32), B, P + N, logits)
        dev.sync()
        if p >= P - 1:
            lg = logits.to_vec().reshape(B, host.vocab)
            for b in range(B):
                t, states[b] = orc.sampler_sample(lg[b].astype(np.float64), ocfg, states[b], past=seqs[b])
                seqs[b].append(t)
    want = np.array([s[P:] for s in seqs], np.int32)
    assert np.array_equal(out, want)
    # greedy through the same path equals the argmax path
    m2 = host.to_device(dev, max_seq, B)
    g1 = m2.generate(prompts, N)
    m3 = host.to_device(dev, max_seq, B)
    g2 = m3.generate(prompts, N, tb.SamplerConfig(1.0, 1, 1.0, 1.0), seed=5)     # top_k = 1 keeps only the maximum
    assert np.array_equal(g1, g2)
    for m in (ref, m2, m3):
        m.destroy()


def test_argument_errors_of_the_newer_entry_points(dev, orc):
    """Bad arguments come back as status codes with a message (no unwinding, no device work)."""
    import ctypes as C

    import tang_b200 as tb

    x = dev.upload(np.zeros((2, 16), np.float32))
    st = dev.upload(np.zeros(2, np.uint64).view(np.float64), tb.F64)
    with pytest.raises(tb.TangqError, match="temperature"):
        dev.sample(x, 2, 16, tb.SamplerConfig(-1.0, 0, 1.0, 1.0), st)
    with pytest.raises(tb.TangqError, match="penalty"):
        dev.sample(x, 2, 16, tb.SamplerConfig(1.0, 0, 1.0, 0.0), st)
    with pytest.raises(tb.TangqError, match="LCG"):
        dev.sample(x, 2, 16, tb.SamplerConfig(1.0, 0, 1.0, 1.0), None)          # sampling without states
    assert list(dev.sample(x, 2, 16, tb.SamplerConfig(0.0, 0, 1.0, 1.0), None).to_vec()) == [0, 0]   # greedy needs none
    q = dev.alloc(2 * 3 * 128, tb.BF16)
    kv = dev.alloc(4 * 128, tb.BF16)
    with pytest.raises(tb.TangqError, match="n_heads/n_kv_heads"):
        dev.gqa_prefill(q, kv, kv, [0], 1, 2, 3, 1, 128, 4 * 128)                 # group of 3
    with pytest.raises(tb.TangqError, match="head_dim"):
        dev.gqa_prefill(q, kv, kv, [0], 1, 2, 2, 2, 64, 4 * 128)
    w = dev.upload(np.zeros((4, 32), np.float32))
    with pytest.raises(tb.TangqError, match="kind"):
        dev.quantize_matrix(w, 4, 32, tb.Q4_F16)                                  # the reference has f32 scales only
    with pytest.raises(tb.TangqError, match="empty"):
        dev.quantize_matrix(w, 0, 32, tb.Q4_F32)
    # a workspace that would have to grow inside a capture is refused with an explanation, and the capture still ends
    big = dev.upload(np.zeros((8, 300000), np.float32))          # 19 MB of f64 workspace: more than anything before it
    st4 = dev.upload(np.zeros(8, np.uint64).view(np.float64), tb.F64)
    out4 = dev.alloc(8, tb.I32)
    cfg = tb.SamplerConfig(1.0, 5, 1.0, 1.0)
    dev.begin_capture()
    rc = dev._L.tq_sample(dev._ctx, C.c_void_p(big.ptr), 1, 8, 300000, C.byref(cfg), C.c_void_p(st4.ptr), None, None, 0,
                          C.c_void_p(out4.ptr))
    msg = dev._L.tq_last_error(dev._ctx).decode()
    g = dev.end_capture()
    g.free()
    assert rc == tb._lib.TQ_EINVAL and "graph capture" in msg
    dev.sample(big, 8, 300000, cfg, st4)         # outside a capture the workspace simply grows
    dev.sync()
