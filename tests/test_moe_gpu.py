"""GPU parity of the MoE FFN layer against the oracle composition (parity unpinned: the reference has
no MoE).  Expert selection must be bit-exact; outputs are f32-accumulated."""
import numpy as np
import pytest

from moe_util import HostMoe
from util import bf16_round, rel_err, rel_err_profile

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import tang_b200

    d = tang_b200.QuantComputeDevice(0)
    yield d
    d.close()


def assert_moe_close(got, want, T):
    """The f32 bar, 1e-3 against max(|ref|, rms(ref)), with one stated exception.  The SwiGLU output is rounded to bf16
    on both sides (the oracle defines the layer that way); where that value lies within an f32-vs-f64 difference of a
    rounding tie, the two sides round it to neighbouring bf16 numbers, and ONE such flip of a large activation moves
    the whole output row of that token by up to 0.3 % of the rms (seen: one token of 130, 58 of 33 280 elements between
    1e-3 and 2.6e-3).  So: at most 0.5 % of the elements may exceed 1e-3, and none may exceed 1e-2 (half the bf16
    bar).  Small batches, which see few activations, must meet 1e-3 everywhere."""
    worst, frac = rel_err_profile(got, want, floor_frac=1.0)
    assert worst < (1e-3 if T < 24 else 1e-2), (T, worst)
    assert frac < 5e-3, (T, frac)


def check(dev, orc, host, T, seed):
    import tang_b200 as tb

    rng = np.random.default_rng(seed)
    hb, hf = bf16_round(rng.standard_normal((T, host.d)).astype(np.float32))
    want, idx_o, w_o, lg_o = host.oracle(orc, hf)
    hbuf = dev.upload(hb, tb.BF16)
    idx_d, w_d, lg_d = tb.moe_router(dev, hbuf, dev.upload(host.wg_bits, tb.BF16), T, host.d, host.E, host.k, host.renorm)
    assert np.array_equal(lg_d, lg_o)                 # f64, same order of additions: bit-identical logits
    assert np.array_equal(idx_d, idx_o)               # so the selection (and its order) is identical
    assert rel_err(w_d, w_o) < 1e-6
    layer = host.to_device(dev)
    out, idx, w = layer.forward(hbuf, T, want_routing=True)
    dev.sync()
    assert np.array_equal(idx.to_vec().reshape(T, host.k), idx_o)
    got = out.to_vec().reshape(T, host.d)
    assert_moe_close(got, want, T)
    layer.destroy()


@pytest.mark.parametrize("T", [1, 5, 70, 200])
def test_small_moe(dev, orc, T):
    host = HostMoe(np.random.default_rng(5), d=256, ffn=256, n_experts=8, top_k=2, n_shared=1)
    check(dev, orc, host, T, seed=T)


def test_router_ties_pick_lower_index(dev, orc):
    import tang_b200 as tb

    d, E, k = 128, 8, 3
    wg = np.zeros((E, d), np.float32)
    wg[[1, 4, 6], 0] = 1.0            # experts 1, 4, 6 tie exactly; the rest tie at zero
    wg[2, 0] = 2.0
    h = np.zeros((1, d), np.float32)
    h[0, 0] = 1.0
    idx, w, lg = tb.moe_router(dev, dev.upload(bf16_round(h)[0], tb.BF16), dev.upload(bf16_round(wg)[0], tb.BF16), 1, d, E, k)
    oi, ow, _ = orc.router_f64(h[0].astype(np.float64), wg.astype(np.float64), E, k)
    assert list(idx[0]) == [2, 1, 4] == list(oi)


def test_router_rows_that_round(dev, orc):
    """Rows whose additions DO round (tiny products beside large ones, cancellation, a huge term): the logits must still
    be the reference's sequential f64 sum bit for bit, which the kernel gets by joining runs of the row in order."""
    import tang_b200 as tb

    rng = np.random.default_rng(77)
    T, d, E, k = 12, 2048, 64, 6
    h = rng.standard_normal((T, d)).astype(np.float32)
    wg = (rng.standard_normal((E, d)) * 0.05).astype(np.float32)
    h[0, 5] = 3e-30
    h[1, [0, 1000, 2047]] = [1e-25, -2e-31, 7e-28]
    h[2, :] = 0.0
    h[2, [3, 900]] = [1e-20, 1.0]
    h[3, 100:140] *= 1e-22                      # a whole run of tiny terms
    h[4, [10, 11]] = [3e4, -3e4]                # cancellation: the sum returns to a finer last place
    wg[:, 10] = 1.0
    wg[:, 11] = 1.0
    h[5, 77] = 1e30                             # one huge term: everything after it rounds
    h[6, ::2] = 0.0
    wg[7, :] *= 1e-18
    wg[9, 1234] = 1e-33
    hb, hf = bf16_round(h)
    wb, wf = bf16_round(wg)
    idx, w, lg = tb.moe_router(dev, dev.upload(hb, tb.BF16), dev.upload(wb, tb.BF16), T, d, E, k)
    for t in range(T):
        oi, ow, ol = orc.router_f64(hf[t].astype(np.float64), wf.astype(np.float64), E, k)
        assert np.array_equal(lg[t], ol), t
        assert list(idx[t]) == list(oi), t


def test_renormalised_weights(dev, orc):
    host = HostMoe(np.random.default_rng(6), d=256, ffn=128, n_experts=16, top_k=4, n_shared=0, renorm=True)
    check(dev, orc, host, 9, seed=3)


@pytest.mark.parametrize("T", [1, 64])
def test_deepseek_v2_lite_shape(dev, orc, T):
    """d_model 2048, 64 routed + 2 shared experts of width 1408, top-6."""
    host = HostMoe(np.random.default_rng(7), d=2048, ffn=1408, n_experts=64, top_k=6, n_shared=2)
    check(dev, orc, host, T, seed=100 + T)


@pytest.mark.parametrize("T", [1, 7, 40, 130])
def test_dispatch_variant_on_one_rank_equals_the_oracle(dev, orc, T):
    """tq_moe_ffn_dispatch with a single rank: both exchanges are local copies, everything else is the same code
    the multi-rank path runs (places, buckets, scatter back, combine)."""
    import tang_b200 as tb

    host = HostMoe(np.random.default_rng(15), d=256, ffn=256, n_experts=8, top_k=2, n_shared=1)
    rng = np.random.default_rng(T)
    hb, hf = bf16_round(rng.standard_normal((T, host.d)).astype(np.float32))
    want, idx_o, _, _ = host.oracle(orc, hf)
    layer = host.to_device(dev)
    out, idx, _w = layer.forward_dispatch(dev.upload(hb, tb.BF16), T, want_routing=True)
    dev.sync()
    assert np.array_equal(idx.to_vec().reshape(T, host.k), idx_o)
    assert_moe_close(out.to_vec().reshape(T, host.d), want, T)
    layer.destroy()


@pytest.mark.parametrize("T", [256, 4096])
def test_deepseek_v2_lite_shape_large_batches(dev, orc, T):
    """The benchmark's larger token batches at the DeepSeek-V2-Lite shape: the router's selection is compared for EVERY
    token (bit-exact logits and choices), the layer output on a seeded sample of tokens (the oracle is a per-token
    loop)."""
    import tang_b200 as tb

    host = HostMoe(np.random.default_rng(7), d=2048, ffn=1408, n_experts=64, top_k=6, n_shared=2)
    rng = np.random.default_rng(500 + T)
    hb, hf = bf16_round(rng.standard_normal((T, host.d)).astype(np.float32))
    hbuf = dev.upload(hb, tb.BF16)
    idx_d, w_d, lg_d = tb.moe_router(dev, hbuf, dev.upload(host.wg_bits, tb.BF16), T, host.d, host.E, host.k, host.renorm)
    wg64 = host.wg.astype(np.float64)
    for t in range(T):
        idx_o, w_o, lg_o = orc.router_f64(hf[t].astype(np.float64), wg64, host.E, host.k, host.renorm)
        assert np.array_equal(lg_d[t], lg_o) and np.array_equal(idx_d[t], idx_o), t
    layer = host.to_device(dev)
    out, idx, w = layer.forward(hbuf, T, want_routing=True)
    dev.sync()
    assert np.array_equal(idx.to_vec().reshape(T, host.k), idx_d)
    got = out.to_vec().reshape(T, host.d)
    assert np.all(np.isfinite(got))
    sample = np.sort(rng.choice(T, 6, replace=False))
    want, _, _, _ = host.oracle(orc, hf[sample])
    assert_moe_close(got[sample], want, T)
    layer.destroy()
