"""Reading checkpoints for the quantised path: the safetensors container on the host, the quantiser on the device.

Mirrors ``tang_safetensors::load`` (crates/tang-safetensors/src/lib.rs:11-75): the same dtypes are accepted
(F64, F32, F16, BF16; anything else is an ``UnsupportedDtype`` error) and 16-bit floats widen exactly
(lib.rs:262-297).  The reference leaves the container format itself to the ``safetensors`` crate; this is a
reader of that public format: 8 bytes little-endian header length, a JSON object mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the header, an optional
``"__metadata__"`` entry), then the tensors' bytes.  Tensors are memory-mapped, not copied.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass

import numpy as np

from . import _lib

_DTYPES = {"F64": (np.float64, 8), "F32": (np.float32, 4), "F16": (np.uint16, 2), "BF16": (np.uint16, 2)}


class SafetensorsError(ValueError):
    """Malformed container or a dtype the reference does not load either."""


@dataclass
class TensorView:
    dtype: str              # "F64" | "F32" | "F16" | "BF16"
    shape: tuple
    data: np.ndarray        # flat; 16-bit floats as their bit patterns (uint16)

    def to_f32(self) -> np.ndarray:
        """The values as f32, widened exactly as the reference does (f64 is narrowed, as `as f32` would)."""
        if self.dtype == "F32":
            return np.asarray(self.data, np.float32)
        if self.dtype == "F64":
            return np.asarray(self.data, np.float64).astype(np.float32)
        if self.dtype == "BF16":
            return (np.asarray(self.data, np.uint16).astype(np.uint32) << 16).view(np.float32)
        return np.asarray(self.data, np.uint16).view(np.float16).astype(np.float32)


def read_safetensors(path) -> dict:
    """name -> TensorView for every tensor of the file."""
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise SafetensorsError("file shorter than its header length field")
        (n,) = struct.unpack("<Q", head)
        f.seek(0, 2)
        size = f.tell()
        if n > size - 8:
            raise SafetensorsError(f"header length {n} exceeds the file ({size} bytes)")
        f.seek(8)
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"header is not JSON: {e}") from None
    if not isinstance(header, dict):
        raise SafetensorsError("header is not a JSON object")
    base = 8 + n
    mm = np.memmap(path, dtype=np.uint8, mode="r") if size > base else np.zeros(0, np.uint8)
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        try:
            dt, shape, (b, e) = info["dtype"], tuple(int(x) for x in info["shape"]), info["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"tensor {name!r}: malformed entry") from None
        if dt not in _DTYPES:
            raise SafetensorsError(f"UnsupportedDtype({dt})")
        np_dt, es = _DTYPES[dt]
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if not (0 <= b <= e <= size - base) or e - b != count * es:
            raise SafetensorsError(f"tensor {name!r}: data_offsets [{b}, {e}) do not match shape {shape} of {dt}")
        out[name] = TensorView(dt, shape, mm[base + b:base + e].view(np_dt))
    return out


def write_safetensors(path, tensors: dict) -> None:
    """tensors: name -> (dtype string, shape, flat array of that dtype's storage type).  ``tang_safetensors::save``
    writes F64 only (lib.rs:78-120); the other dtypes are accepted here so that tests can build checkpoints."""
    header, blobs, off = {}, [], 0
    for name, (dt, shape, data) in tensors.items():
        if dt not in _DTYPES:
            raise SafetensorsError(f"UnsupportedDtype({dt})")
        raw = np.ascontiguousarray(data, _DTYPES[dt][0]).tobytes()
        header[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def quantize_linear(dev, view: TensorView, kind: int):
    """[out, in] weight of a checkpoint -> quantised weight in HBM: the raw bits are uploaded once and
    ``quantize_matrix_q4`` / ``quantize_matrix_q8`` (crates/tang-infer/src/quantize.rs:193-220) runs on the device."""
    if len(view.shape) != 2:
        raise SafetensorsError(f"a linear weight is two-dimensional, got shape {view.shape}")
    rows, cols = view.shape
    if view.dtype == "BF16":
        buf = dev.upload(np.asarray(view.data, np.uint16), _lib.BF16)
    elif view.dtype == "F16":
        buf = dev.upload(np.asarray(view.data, np.uint16), _lib.F16)
    else:
        buf = dev.upload(view.to_f32(), _lib.F32)
    w = dev.quantize_matrix(buf, rows, cols, kind)
    buf.free()
    return w
