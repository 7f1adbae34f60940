"""Helpers shared by the GPU parity tests."""
import numpy as np


def rel_err(got, want, floor_frac=1e-2):
    """max_i |got-want| / max(|want_i|, floor_frac * rms(want)).

    The floor keeps outputs that happen to land near zero (sums of +- terms) from turning an
    absolute error of a few f32 ulps of the typical magnitude into a huge ratio."""
    got = np.asarray(got, np.float64).reshape(-1)
    want = np.asarray(want, np.float64).reshape(-1)
    rms = float(np.sqrt(np.mean(want * want))) or 1.0
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), floor_frac * rms)))


def bf16_round(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    r = ((u + (0x7FFF + lsb).astype(np.uint32)) >> 16).astype(np.uint16)
    return r, (r.astype(np.uint32) << 16).view(np.float32)


def make_weight(rng, kind, rows, cols):
    """Random quantised weight in the value ranges of the benchmark configurations.
    Returns (scales, payload) in the oracle's structure-of-arrays form."""
    bpr = (cols + 31) // 32
    if kind in (0, 1):
        packed = rng.integers(0, 256, (rows, bpr * 16), dtype=np.uint8)
        sc = rng.uniform(0.002, 0.02, (rows, bpr)).astype(np.float32)
        if kind == 1:
            sc = sc.astype(np.float16).view(np.uint16)
        return sc, packed
    if kind == 2:
        vals = rng.integers(-128, 128, (rows, bpr * 32), dtype=np.int8)
        sc = rng.uniform(0.001, 0.01, (rows, bpr)).astype(np.float32)
        return sc, vals
    vals = rng.integers(-127, 128, (rows, cols), dtype=np.int8)
    sc = rng.uniform(0.001, 0.01, rows).astype(np.float32)
    return sc, vals


def rel_err_profile(got, want, floor_frac=1.0):
    """(max, fraction of elements above 1e-3) of |got-want| / max(|want_i|, floor_frac * rms(want))."""
    got = np.asarray(got, np.float64).reshape(-1)
    want = np.asarray(want, np.float64).reshape(-1)
    rms = float(np.sqrt(np.mean(want * want))) or 1.0
    e = np.abs(got - want) / np.maximum(np.abs(want), floor_frac * rms)
    return float(e.max()), float(np.mean(e > 1e-3))
