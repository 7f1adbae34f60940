"""The allocation-free decode-attention entry point, tq_gqa_decode_noalloc, checked through the C
ABI against tq_gqa_decode on the same inputs.

Some callers of this library are not allowed to allocate device memory once they are running (a
serving loop with a frozen memory pool, a callback that is only lent a stream).  For them the
library keeps the attention partials in a fixed array of its own.  The test makes two calls in a row
with different data, so the second call runs over whatever the first left in that array, and then
asks for more than the array holds to see the refusal.  This file sorts last on purpose: a run
that stops at the first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from util import bf16_round, rel_err

pytestmark = pytest.mark.gpu


def _call(dev, fn, q, k, v, lens, B, nh, nkv, hd, stride, max_len):
    import tang_b200 as tb

    out = dev.alloc(B * nh * hd, tb.F32)
    st = fn(dev._ctx, C.c_void_p(q.ptr), C.c_void_p(k.ptr), C.c_void_p(v.ptr), C.c_void_p(lens.ptr), B, nh, nkv, hd,
            stride, max_len, C.c_void_p(out.ptr), tb.F32)
    return st, out


def test_noalloc_matches_allocating_entry_point_twice():
    import tang_b200 as tb

    dev = tb.QuantComputeDevice(0)
    L = dev._L
    rng = np.random.default_rng(2024)
    hd = 128
    # two different shapes back to back: the second call reuses the array the first one filled
    for (B, nh, nkv, lens) in [(3, 32, 8, [2049, 700, 1]), (8, 8, 2, [300, 64, 65, 1000, 5, 1024, 999, 128])]:
        max_seq = max(lens) + 1
        kv_dim = nkv * hd
        q = dev.upload(bf16_round(rng.standard_normal((B, nh * hd)).astype(np.float32))[0], tb.BF16)
        k = dev.upload(bf16_round(rng.standard_normal((B, max_seq, kv_dim)).astype(np.float32))[0], tb.BF16)
        v = dev.upload(bf16_round(rng.standard_normal((B, max_seq, kv_dim)).astype(np.float32))[0], tb.BF16)
        ln = dev.upload(np.array(lens, np.int32), tb.I32)
        st0, ref = _call(dev, L.tq_gqa_decode, q, k, v, ln, B, nh, nkv, hd, max_seq * kv_dim, max(lens))
        st1, got = _call(dev, L.tq_gqa_decode_noalloc, q, k, v, ln, B, nh, nkv, hd, max_seq * kv_dim, max(lens))
        assert st0 == 0 and st1 == 0, L.tq_last_error(dev._ctx)
        dev.sync()
        a, b = got.to_vec(), ref.to_vec()
        assert np.all(np.isfinite(a))
        assert rel_err(a, b) < 1e-3          # same kernels, same split rule: in practice bit-identical
    # A request whose partials do not fit the fixed array is refused with a message, not served.  The number of
    # splits follows the GPU's SM count (the library aims at four CTAs per SM), so the test recomputes it with the
    # library's rule and picks a batch that needs at least two splits on any GPU with 98 SMs or more:
    # 390 sequences x 8 heads x >= 2 splits x 520 B >= 3.24 MB > 3 MiB.
    import torch

    B, nh, nkv, max_len = 390, 8, 1, 256
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    tiles = (max_len + 63) // 64
    want = max(1, -(-4 * sms // (B * nkv)))
    n_splits = min(want, max(1, (tiles + 1) // 2))
    per_split = -(-tiles // n_splits)
    n_splits = -(-tiles // per_split)
    assert n_splits >= 2 and B * nh * n_splits * (hd + 2) * 4 > 3 << 20, (sms, n_splits)
    q = dev.alloc(B * nh * hd, tb.BF16)
    kv = dev.alloc(B * max_len * nkv * hd, tb.BF16)
    dev.memset(q)
    dev.memset(kv)
    ln = dev.upload(np.full(B, max_len, np.int32), tb.I32)
    st, _ = _call(dev, L.tq_gqa_decode_noalloc, q, kv, kv, ln, B, nh, nkv, hd, max_len * nkv * hd, max_len)
    assert st == tb._lib.TQ_EINVAL and b"static" in L.tq_last_error(dev._ctx)
    dev.sync()
    st, _ = _call(dev, L.tq_gqa_decode, q, kv, kv, ln, B, nh, nkv, hd, max_len * nkv * hd, max_len)
    assert st == 0                             # the allocating entry point serves the same request
    dev.sync()
    st, _ = _call(dev, L.tq_gqa_decode_noalloc, q, kv, kv, ln, B, nh, nkv, 64, 0, 16)
    assert st == tb._lib.TQ_EINVAL            # wrong head_dim: same argument checks as the original
    dev.close()
