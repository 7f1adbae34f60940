"""Writes quantize_kat.json: known answers for the block quantiser and the quantised matvec.

The reference (Rust) cannot be built here, so these vectors do not come from running it.  They
come from a SECOND, independent restatement of crates/tang-infer/src/quantize.rs written with
numpy scalar float32 arithmetic and Python integers (no code shared with oracle/), evaluated on
the inputs of the reference's own unit tests (quantize.rs:297-354) plus edge cases the source
defines: an all-zero block (scale 1.0), a ragged tail, a value that clamps, and a tie that must
round away from zero.  tests/test_oracle_pins.py checks the C oracle against this file bit for bit.

Run:  python tests/golden/make_quantize_kat.py
"""
import json
import math
import os
import struct

import numpy as np

F = np.float32


def f32_hex(x):
    return struct.pack("<f", float(x)).hex()


def round_half_away(v):
    v = float(v)
    return math.floor(v + 0.5) if v >= 0 else -math.floor(-v + 0.5)


def quant_block(chunk, qmax, lo, hi):
    amax = F(0)
    for v in chunk:
        a = abs(F(v))
        if a > amax:                      # f32::max(acc, NaN) keeps acc: a NaN never becomes the maximum
            amax = a
    scale = F(1.0) if amax == 0 else F(amax / F(qmax))
    inv = F(F(1.0) / scale)
    q = []
    for v in chunk:
        with np.errstate(invalid="ignore"):
            pr = F(F(v) * inv)
        if pr != pr:                      # `NaN.round().clamp(lo, hi) as i8` is 0 in Rust (a NaN weight, or inf * 0)
            q.append(0)
        elif math.isinf(pr):
            q.append(hi if pr > 0 else lo)
        else:
            q.append(int(min(max(round_half_away(pr), lo), hi)))
    return scale, q


def quantize(data, bits):
    qmax, lo, hi = (127, -128, 127) if bits == 8 else (7, -8, 7)
    scales, payload = [], []
    for s in range(0, len(data), 32):
        chunk = data[s:s + 32]
        scale, q = quant_block(chunk, qmax, lo, hi)
        q = q + [0] * (32 - len(q))
        scales.append(scale)
        if bits == 8:
            payload += [v & 0xFF for v in q]
        else:
            payload += [((q[2 * i] + 8) & 0xF) | (((q[2 * i + 1] + 8) & 0xF) << 4) for i in range(16)]
    return scales, payload


def matvec(data, rows, cols, x, bits):
    y = []
    for r in range(rows):
        scales, payload = quantize(data[r * cols:(r + 1) * cols], bits)
        s = 0.0
        for b, sc in enumerate(scales):
            for i in range(32):
                k = b * 32 + i
                if k >= cols:
                    continue
                if bits == 8:
                    v = payload[b * 32 + i]
                    v = v - 256 if v > 127 else v
                else:
                    byte = payload[b * 16 + i // 2]
                    v = ((byte >> 4) if i % 2 else (byte & 0xF)) - 8
                s += float(v) * float(sc) * x[k]
        y.append(s)
    return y


def main():
    cases = {
        "ref_roundtrip": [0.5, -1.0, 2.0, -3.0, 0.0, 1.5, -0.7, 0.3],            # quantize.rs:298,313
        "zero_block": [0.0] * 32,                                               # scale must be 1.0
        "ragged_40": [math.sin(0.37 * i) * (1 + i % 5) for i in range(40)],      # second block has 8 values
        "tie_and_clamp": [7.0, 3.5, -3.5, 0.5, -0.5, 2.5, -7.0, 6.5] + [0.25 * i - 3 for i in range(24)],
        "nan_in_block": [1.0, float("nan"), -2.0, 3.5] + [0.5 * i - 4 for i in range(28)],      # NaN -> code 0, scale from the rest
        "inf_in_block": [1.0, float("inf"), -2.0, float("-inf")] + [0.5 * i - 4 for i in range(28)],  # scale inf: finite -> 0, inf*0 = NaN -> 0
    }
    out = {"quantize": {}, "matvec": {}}
    for name, data in cases.items():
        data = [float(F(v)) for v in data]
        for bits in (8, 4):
            scales, payload = quantize(data, bits)
            out["quantize"][f"{name}_q{bits}"] = {
                "data_f32_hex": [f32_hex(v) for v in data],
                "scales_f32_hex": [f32_hex(s) for s in scales],
                "payload_u8": payload,
            }
    mv = {
        "ref_2x3": ([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], 2, 3, [1.0, 0.5, -1.0]),     # quantize.rs:329-333,344-347
        "ragged_3x40": ([math.cos(0.11 * i) * 2 for i in range(120)], 3, 40, [math.sin(0.5 * i) for i in range(40)]),
    }
    for name, (w, rows, cols, x) in mv.items():
        w = [float(F(v)) for v in w]
        for bits in (8, 4):
            y = matvec(w, rows, cols, x, bits)
            out["matvec"][f"{name}_q{bits}"] = {
                "w_f32_hex": [f32_hex(v) for v in w], "rows": rows, "cols": cols,
                "x_f64_hex": [struct.pack("<d", v).hex() for v in x],
                "y_f64_hex": [struct.pack("<d", v).hex() for v in y],
            }
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quantize_kat.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", path)


if __name__ == "__main__":
    main()
