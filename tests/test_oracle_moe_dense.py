"""A second, independently written formulation of the MoE layer, checked against the oracle's per-token one (CPU only).

The reference has no MoE, so the oracle's composition (oracle/tang_oracle_models.cpp: router -> top-k -> weighted
sum of the chosen experts, token by token) is pinned by nothing outside itself.  This file states the same layer the
other way round — expert-major and dense: every expert is applied to EVERY token with the batched quantised matmul,
the routing becomes a [tokens, experts] gate matrix that is zero outside each token's top-k (built with numpy's
sort, not the oracle's selection), and the layer is one masked sum over experts.  The dequantised weights, the
softmax, the top-k rule (value descending, lower index first), the bf16 rounding point after SwiGLU and the shared
experts all have to agree for the two to meet.
"""
import numpy as np

from moe_util import HostMoe, KIND
from util import bf16_round


def dense_moe(orc, host, h):
    """h [T, d] f64 (bf16-exact).  Returns (out [T, d], chosen [T, k])."""
    T = h.shape[0]
    logits = np.zeros((T, host.E))
    wg = host.wg.astype(np.float64)
    for k in range(host.d):                                   # ascending k, like the layer's router
        logits += np.outer(h[:, k], wg[:, k])
    order = np.lexsort((np.arange(host.E)[None, :].repeat(T, 0), -logits), axis=1)   # value descending, index ascending
    chosen = order[:, :host.k]
    p = np.exp(logits - logits.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)                         # softmax over ALL routed experts
    gate = np.zeros((T, host.E))
    np.put_along_axis(gate, chosen, np.take_along_axis(p, chosen, 1), 1)
    if host.renorm:
        gate /= gate.sum(axis=1, keepdims=True)
    out = np.zeros((T, host.d))
    for e, ex in enumerate(host.experts):
        mm = lambda w, x: orc.qmatmul(KIND, w[0], w[1], w[2], w[3], x)
        g, u = mm(ex["gate"], h), mm(ex["up"], h)
        act = g / (1.0 + np.exp(-g)) * u                      # silu(gate) * up
        act = bf16_round(act.astype(np.float32))[1].astype(np.float64)   # bf16 activation entering the down projection
        y = mm(ex["down"], act)
        out += y * (gate[:, e:e + 1] if e < host.E else 1.0)  # shared experts: every token, weight 1
    return out, chosen


def test_dense_expert_major_form_equals_the_per_token_oracle(orc):
    for renorm, n_shared, T in ((False, 1, 7), (True, 0, 5), (False, 2, 12)):
        host = HostMoe(np.random.default_rng(40 + T), d=128, ffn=96, n_experts=8, top_k=3, n_shared=n_shared, renorm=renorm)
        h = bf16_round(np.random.default_rng(T).standard_normal((T, host.d)).astype(np.float32))[1]
        want, idx, w, lg = host.oracle(orc, h)
        got, chosen = dense_moe(orc, host, h.astype(np.float64))
        assert np.array_equal(chosen, idx)
        scale = float(np.sqrt(np.mean(want * want)))
        # The two differ only where an f64 rounding ahead of the bf16 rounding of the SwiGLU output flips an element by
        # one bf16 ulp (sigmoid written two ways): a handful of elements at the 1e-3 level of the rms, most identical.
        assert np.max(np.abs(got - want)) < 2e-3 * scale
        assert np.median(np.abs(got - want)) < 1e-12 * scale


def test_tie_rule_of_the_dense_form(orc):
    """Equal logits: the lower expert index wins in both formulations."""
    host = HostMoe(np.random.default_rng(1), d=128, ffn=32, n_experts=8, top_k=3, n_shared=0)
    host.wg[:] = 0.0
    host.wg[[1, 4, 6], 0] = 1.0
    host.wg[2, 0] = 2.0
    h = np.zeros((1, 128))
    h[0, 0] = 1.0
    _, chosen = dense_moe(orc, host, h)
    idx, _, _ = orc.router_f64(h[0], host.wg.astype(np.float64), 8, 3)
    assert list(chosen[0]) == [2, 1, 4] == list(idx)
