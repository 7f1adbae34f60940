"""The safetensors reader (host) and the loader that quantises on the device
(crates/tang-safetensors/src/lib.rs:11-75; crates/tang-infer/src/quantize.rs:193-220)."""
import json
import struct

import numpy as np
import pytest

from util import bf16_round


def _ck():
    import tang_b200.checkpoint as ck

    return ck


def test_round_trip_of_every_supported_dtype(tmp_path):
    ck = _ck()
    rng = np.random.default_rng(1)
    a64 = rng.standard_normal((3, 5))
    a32 = rng.standard_normal((4, 32)).astype(np.float32)
    b16 = bf16_round(rng.standard_normal((2, 64)).astype(np.float32))[0]
    f16 = rng.standard_normal((7,)).astype(np.float16)
    path = tmp_path / "m.safetensors"
    ck.write_safetensors(path, {"a": ("F64", a64.shape, a64.ravel()), "b": ("F32", a32.shape, a32.ravel()),
                                "c": ("BF16", b16.shape, b16.ravel()), "d": ("F16", f16.shape, f16.view(np.uint16))})
    t = ck.read_safetensors(path)
    assert set(t) == {"a", "b", "c", "d"}
    assert t["a"].shape == (3, 5) and np.array_equal(t["a"].data, a64.ravel())
    assert np.array_equal(t["b"].data.view(np.uint32), a32.ravel().view(np.uint32))
    assert np.array_equal(t["c"].data, b16.ravel())
    # widening is exact (lib.rs:262-297): bf16 = the top half of an f32, f16 by value
    assert np.array_equal(t["c"].to_f32().view(np.uint32), b16.ravel().astype(np.uint32) << 16)
    assert np.array_equal(t["d"].to_f32(), f16.astype(np.float32))
    assert np.array_equal(t["a"].to_f32(), a64.ravel().astype(np.float32))


def test_metadata_entry_is_skipped_and_bad_files_are_refused(tmp_path):
    ck = _ck()

    def write(header, payload=b""):
        hj = json.dumps(header).encode()
        p = tmp_path / "x.safetensors"
        p.write_bytes(struct.pack("<Q", len(hj)) + hj + payload)
        return p

    ok = write({"__metadata__": {"format": "pt"}, "w": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8)
    assert list(ck.read_safetensors(ok)) == ["w"]
    with pytest.raises(ck.SafetensorsError, match="UnsupportedDtype"):
        ck.read_safetensors(write({"w": {"dtype": "I64", "shape": [1], "data_offsets": [0, 8]}}, b"\0" * 8))
    with pytest.raises(ck.SafetensorsError, match="data_offsets"):
        ck.read_safetensors(write({"w": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8))
    with pytest.raises(ck.SafetensorsError, match="data_offsets"):
        ck.read_safetensors(write({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8))
    bad = tmp_path / "y.safetensors"
    bad.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ck.SafetensorsError, match="header length"):
        ck.read_safetensors(bad)
    bad.write_bytes(b"\1\2\3")
    with pytest.raises(ck.SafetensorsError):
        ck.read_safetensors(bad)


@pytest.mark.gpu
def test_checkpoint_to_quantised_weight(tmp_path, orc):
    """BF16 and F32 tensors of a file become Q4 / Q8 weights in HBM with the reference quantiser's exact codes."""
    import tang_b200 as tb

    ck = _ck()
    rng = np.random.default_rng(2)
    w32 = rng.standard_normal((48, 160)).astype(np.float32)
    wb_bits, wb = bf16_round(rng.standard_normal((32, 96)).astype(np.float32))
    path = tmp_path / "m.safetensors"
    ck.write_safetensors(path, {"l0.w": ("F32", w32.shape, w32.ravel()), "l1.w": ("BF16", wb.shape, wb_bits.ravel())})
    t = ck.read_safetensors(path)
    dev = tb.QuantComputeDevice(0)
    for name, ref, kind in (("l0.w", w32, tb.Q4_F32), ("l1.w", wb, tb.Q8_F32)):
        qw = ck.quantize_linear(dev, t[name], kind)
        deq, ints = dev.dequantize(qw)
        for r in range(ref.shape[0]):
            if kind == tb.Q4_F32:
                sc, packed = orc.quantize_q4(ref[r])
                want_i, want_v = orc.unpack_q4(packed)[:ref.shape[1]], orc.dequantize_q4(sc, packed)[:ref.shape[1]]
            else:
                sc, vals = orc.quantize_q8(ref[r])
                want_i, want_v = vals[:ref.shape[1]], orc.dequantize_q8(sc, vals)[:ref.shape[1]]
            assert np.array_equal(ints[r], want_i) and np.array_equal(deq[r].view(np.uint32), want_v.view(np.uint32))
    dev.close()
