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
