"""Host model of the MoE router's run-wise summation (tang_b200/csrc/moe.cu, router_ordered_sum and the certificate
in router_kernel): the reference adds the 2048 products of a gate row one after the other in f64; the kernel adds
runs of consecutive products in parallel and joins them in order, taking a run in one step only when every partial sum
on the way is representable.  This file restates that rule in Python floats (IEEE binary64, no contraction) and checks
it against the plain sequential loop on inputs built to round: tiny terms beside large ones, cancellation, huge terms,
zeros.  No GPU, no oracle: pure arithmetic."""
import math

import numpy as np


def bf16_bits(a):
    u = np.asarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint32)


def bf16_value(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def ulp_code(bits):
    """Biased exponent of the last place of a bf16 (at least 1: subnormals), 0x2000 for a zero."""
    e = (bits >> 7) & 0xFF
    return np.where((bits & 0x7FFF) == 0, 0x2000, np.maximum(e, 1)).astype(np.int64)


def sequential(p):
    acc = 0.0
    for x in p:
        acc += float(x)
    return acc


def fast_path_is_exact(hb, wb):
    """The warp-parallel certificate: every non-zero product is a multiple of 2^(q - 268) and the sum of magnitudes
    stays below 2^52 of those units (and no product lies below the normal range of f32)."""
    p = bf16_value(hb) * bf16_value(wb)
    q = int(np.min(ulp_code(hb) + ulp_code(wb)))
    if q >= 0x2000:
        return True
    sabs = float(np.sum(np.abs(p).astype(np.float32), dtype=np.float32))
    return q >= 140 and sabs < math.ldexp(1.0, 52 + q - 268)


def run_wise(hb, wb, lanes=32):
    d = len(hb)
    ch = ((d + 255) >> 8) << 3
    p = bf16_value(hb) * bf16_value(wb)            # exact: 16 significant bits
    codes = ulp_code(hb) + ulp_code(wb)
    any_q = 1 << 20
    s, qs = 0.0, any_q
    for c in range(lanes):
        lo, hi = c * ch, min(d, (c + 1) * ch)
        if lo >= d:
            continue
        cq = int(np.min(codes[lo:hi]))
        if cq >= 0x2000:
            continue                                # zeros only
        cs = sequential(p[lo:hi])
        ca = sequential(np.abs(p[lo:hi]))
        qq = min(qs, cq - 268)
        bound = math.ldexp(1.0, 53 + qq) if 53 + qq < 1024 else math.inf
        if (abs(s) + ca) * (1.0 + 2.0 ** -30) < bound:
            s += cs
            qs = any_q if s == 0.0 else qq
        else:
            for x in p[lo:hi]:
                s += float(x)
            if s == 0.0:
                qs = any_q
            elif math.isfinite(s):
                qs = math.frexp(s)[1] - 1 - 52      # ilogb(s) - 52
            else:
                qs = -(1 << 20)
    return s


def rows():
    rng = np.random.default_rng(2024)
    d = 2048
    out = []
    for _ in range(40):                             # plain data: mostly certified as a whole
        out.append((rng.standard_normal(d), rng.standard_normal(d) * 0.05))
    for _ in range(60):                             # magnitudes spread over 60 binades
        h = rng.standard_normal(d) * np.exp2(rng.integers(-40, 10, d))
        w = rng.standard_normal(d) * np.exp2(rng.integers(-30, 4, d))
        out.append((h, w))
    for _ in range(40):                             # large terms that cancel, with tiny ones in between
        h = rng.standard_normal(d) * 1e-12
        w = np.ones(d)
        k = rng.integers(0, d - 1, 20)
        big = rng.standard_normal(20) * 1e6
        h[k] = big
        h[k + 1] = -big
        out.append((h, w))
    for _ in range(20):                             # sparse rows and runs of zeros
        h = rng.standard_normal(d) * (rng.random(d) < 0.1)
        h[512:1024] = 0.0
        w = rng.standard_normal(d) * np.exp2(rng.integers(-60, 0, d))
        out.append((h, w))
    h = rng.standard_normal(d)
    h[77] = 1e30                                    # one huge term: everything after it rounds
    out.append((h, rng.standard_normal(d)))
    out.append((np.zeros(d), rng.standard_normal(d)))
    return out


def test_run_wise_join_equals_the_sequential_sum():
    took_runs = 0
    for h, w in rows():
        hb, wb = bf16_bits(h), bf16_bits(w)
        want = sequential(bf16_value(hb) * bf16_value(wb))
        got = run_wise(hb, wb)
        assert got == want or (math.isnan(got) and math.isnan(want))
        if not fast_path_is_exact(hb, wb):
            took_runs += 1
    assert took_runs > 50                           # the inputs do exercise the ordered path


def test_certified_rows_sum_exactly_in_any_order():
    """Where the certificate holds, the order of the additions cannot matter: a pairwise (tree) sum gives the bits of the
    sequential one."""
    rng = np.random.default_rng(7)
    d, seen = 2048, 0
    for _ in range(60):
        hb, wb = bf16_bits(rng.standard_normal(d)), bf16_bits(rng.standard_normal(d) * 0.05)
        if not fast_path_is_exact(hb, wb):
            continue
        seen += 1
        p = bf16_value(hb) * bf16_value(wb)
        t = p.copy()
        while len(t) > 1:
            t = t[0::2] + t[1::2]
        assert float(t[0]) == sequential(p)
    assert seen > 30


def test_short_rows_fuzz():
    """Many short rows (8 to 16 terms per run) with wide exponent spreads and exact cancellations: the joins cross
    binades and fall back term by term often."""
    rng = np.random.default_rng(99)
    for trial in range(1500):
        d = int(rng.choice([64, 256, 264, 512]))
        spread = int(rng.choice([2, 8, 30, 70]))
        h = rng.standard_normal(d) * np.exp2(rng.integers(-spread, spread, d))
        w = rng.standard_normal(d) * np.exp2(rng.integers(-spread, 1, d))
        if trial % 3 == 0:                          # pairs that cancel exactly
            k = rng.integers(0, d - 1, 6)
            h[k + 1] = -h[k]
            w[k + 1] = w[k]
        if trial % 5 == 0:
            h[rng.integers(0, d, d // 4)] = 0.0
        hb, wb = bf16_bits(h), bf16_bits(w)
        assert run_wise(hb, wb) == sequential(bf16_value(hb) * bf16_value(wb)), trial
