"""Host-side mirror of the reference interfaces this library stands in for.

Names and argument meaning follow the reference (paths relative to the ecto/tang repository):
  * ``QuantizedQ4`` / ``QuantizedQ8`` — crates/tang-infer/src/quantize.rs:34-44
  * ``q4_matvec`` / ``q8_matvec``     — quantize.rs:227-289
  * ``upload`` / ``download`` / ``sync`` and the operator methods — the ``ComputeDevice`` trait,
    crates/tang-compute/src/device.rs:19-180
Everything here is a thin wrapper over the C ABI in include/tangq.h; no arithmetic happens in
Python and nothing falls back to the CPU.  Where the reference panics (shape asserts) these
raise ``TangqError``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import BF16, F32, F64, I8, I8_ROW, Q4_F16, Q4_F32, Q8_F32, TangqError

_NP_OF = {F32: np.float32, BF16: np.uint16, I8: np.int8, F64: np.float64, _lib.I32: np.int32, _lib.U8: np.uint8,
          _lib.F16: np.uint16}
_SIZE_OF = {F32: 4, BF16: 2, I8: 1, F64: 8, _lib.I32: 4, _lib.U8: 1, _lib.F16: 2}


@dataclass
class QuantizedQ4:
    """Blocks of a Q4 tensor: ``scales`` f32 [n_blocks], ``packed`` u8 [n_blocks*16], ``shape`` [rows, cols]."""
    scales: np.ndarray
    packed: np.ndarray
    shape: tuple

    def to_wire(self) -> np.ndarray:
        """Array-of-structs wire form: per block LE f32 scale + 16 payload bytes (20 bytes)."""
        nb = self.scales.size
        out = np.empty((nb, 20), np.uint8)
        out[:, :4] = np.ascontiguousarray(self.scales, "<f4").reshape(nb, 1).view(np.uint8)
        out[:, 4:] = np.ascontiguousarray(self.packed, np.uint8).reshape(nb, 16)
        return out.reshape(-1)


@dataclass
class QuantizedQ8:
    """Blocks of a Q8 tensor: ``scales`` f32 [n_blocks], ``values`` i8 [n_blocks*32], ``shape`` [rows, cols]."""
    scales: np.ndarray
    values: np.ndarray
    shape: tuple

    def to_wire(self) -> np.ndarray:
        nb = self.scales.size
        out = np.empty((nb, 36), np.uint8)
        out[:, :4] = np.ascontiguousarray(self.scales, "<f4").reshape(nb, 1).view(np.uint8)
        out[:, 4:] = np.ascontiguousarray(self.values, np.int8).reshape(nb, 32).view(np.uint8)
        return out.reshape(-1)


class Buffer:
    """Device buffer (``ComputeBuffer``, device.rs:7-16): ``len()`` counts elements."""

    def __init__(self, dev: "QuantComputeDevice", ptr: int, n: int, dtype: int, owns: bool = True):
        self.dev, self.ptr, self.n, self.dtype, self.owns = dev, ptr, n, dtype, owns

    def __len__(self) -> int:
        return self.n

    @property
    def nbytes(self) -> int:
        return self.n * _SIZE_OF[self.dtype]

    def to_vec(self) -> np.ndarray:
        return self.dev.download(self)

    def free(self) -> None:
        if self.owns and self.ptr:
            self.dev._check(self.dev._L.tq_buf_free(self.dev._ctx, C.c_void_p(self.ptr)))
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class QBuffer:
    """A quantised weight matrix resident on the device."""

    def __init__(self, dev: "QuantComputeDevice", handle: int, rows: int, cols: int, kind: int, keep=None):
        self.dev, self.handle, self.rows, self.cols, self.kind = dev, handle, rows, cols, kind
        self._keep = keep  # device arrays a wrapped handle points into

    @property
    def stream_bytes(self) -> int:
        return int(self.dev._L.tq_qweight_bytes(C.c_void_p(self.handle)))

    def free(self) -> None:
        if self.handle:
            self.dev._check(self.dev._L.tq_qweight_free(self.dev._ctx, C.c_void_p(self.handle)))
            self.handle = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _host(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


class QuantComputeDevice:
    """One GPU, one stream (``CudaComputeDevice::new``, crates/tang-compute/src/cuda.rs:151-179)."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self._L = _lib.load()
        ctx = C.c_void_p()
        st = self._L.tq_ctx_create(device, C.c_void_p(stream or 0), C.byref(ctx))
        if st != _lib.TQ_OK:
            raise TangqError(st, f"tq_ctx_create(device={device}) failed: no usable sm_100 CUDA device; "
                                 "this library has no CPU fallback")
        self._ctx = ctx
        self.device = device

    def close(self) -> None:
        if getattr(self, "_ctx", None):
            self._L.tq_ctx_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st: int) -> None:
        if st != _lib.TQ_OK:
            raise TangqError(st, self._L.tq_last_error(self._ctx).decode())

    # ------------------------------------------------------------------ buffers
    @property
    def stream(self) -> int:
        return int(self._L.tq_ctx_stream(self._ctx) or 0)

    def sync(self) -> None:
        self._check(self._L.tq_sync(self._ctx))

    def alloc(self, n: int, dtype: int = F32) -> Buffer:
        ptr = C.c_void_p()
        self._check(self._L.tq_buf_alloc(self._ctx, n * _SIZE_OF[dtype], C.byref(ptr)))
        return Buffer(self, ptr.value, n, dtype)

    def upload(self, data, dtype: int = F32) -> Buffer:
        """``upload(&[f32])`` (device.rs:37).  ``dtype=BF16`` takes bf16 bit patterns (uint16)."""
        a = _host(data, _NP_OF[dtype]).reshape(-1)
        buf = self.alloc(a.size, dtype)
        self._check(self._L.tq_upload(self._ctx, C.c_void_p(buf.ptr), C.c_void_p(a.ctypes.data), a.nbytes))
        return buf

    def upload_into(self, buf: Buffer, data) -> None:
        """``copy_from_slice`` into an existing buffer of the same element type."""
        a = _host(data, _NP_OF[buf.dtype]).reshape(-1)
        if a.size > buf.n:
            raise TangqError(_lib.TQ_EINVAL, f"upload_into: {a.size} elements into a buffer of {buf.n}")
        self._check(self._L.tq_upload(self._ctx, C.c_void_p(buf.ptr), C.c_void_p(a.ctypes.data), a.nbytes))

    def argmax_rows(self, x: Buffer, rows: int, cols: int, slices: int = 1) -> Buffer:
        """Greedy ``Sampler::sample`` (sampling.rs:108-111): first maximum of each f32 row, int32 [rows]."""
        out = self.alloc(rows, _lib.I32)
        self._check(self._L.tq_argmax_rows(self._ctx, C.c_void_p(x.ptr), slices, rows, cols, C.c_void_p(out.ptr)))
        return out

    def sample(self, logits: Buffer, rows: int, cols: int, cfg: "SamplerConfig", rng_states: Buffer | None = None,
               past: Buffer | None = None, past_lens: Buffer | None = None, past_ld: int = 0, slices: int = 1) -> Buffer:
        """``Sampler::sample`` (sampling.rs:86-158) for `rows` sequences; rng_states is a U64 buffer [rows] that the
        call advances.  Returns int32 [rows]."""
        out = self.alloc(rows, _lib.I32)
        self._check(self._L.tq_sample(self._ctx, C.c_void_p(logits.ptr), slices, rows, cols, C.byref(cfg),
                                      _opt_ptr(rng_states), _opt_ptr(past), _opt_ptr(past_lens), past_ld, C.c_void_p(out.ptr)))
        return out

    def upload_bf16(self, data_f32) -> Buffer:
        """Uploads f32 data and narrows it to bf16 on the device (round to nearest even)."""
        tmp = self.upload(data_f32, F32)
        out = self.alloc(tmp.n, BF16)
        self.convert(tmp, out)
        self.sync()
        tmp.free()
        return out

    def download(self, buf: Buffer) -> np.ndarray:
        out = np.empty(buf.n, _NP_OF[buf.dtype])
        self._check(self._L.tq_download(self._ctx, C.c_void_p(out.ctypes.data), C.c_void_p(buf.ptr), out.nbytes))
        return out

    def convert(self, src: Buffer, dst: Buffer) -> None:
        assert src.n == dst.n
        self._check(self._L.tq_convert(self._ctx, C.c_void_p(src.ptr), src.dtype, C.c_void_p(dst.ptr), dst.dtype, src.n))

    def memset(self, buf: Buffer, byte: int = 0) -> None:
        self._check(self._L.tq_memset(self._ctx, C.c_void_p(buf.ptr), byte, buf.nbytes))

    # ------------------------------------------------------------------ quantised weights
    def _wrap_q(self, h: C.c_void_p, keep=None) -> QBuffer:
        rows, cols, kind = C.c_size_t(), C.c_size_t(), C.c_int()
        self._L.tq_qweight_shape(h, C.byref(rows), C.byref(cols), C.byref(kind))
        return QBuffer(self, h.value, rows.value, cols.value, kind.value, keep)

    def upload_q4(self, q: QuantizedQ4, scale_dtype: str = "f32") -> QBuffer:
        """Uploads a ``QuantizedQ4``.  ``scale_dtype='f16'`` narrows the block scales to half first."""
        rows, cols = q.shape
        h = C.c_void_p()
        if scale_dtype == "f32":
            wire = q.to_wire()
            self._check(self._L.tq_qweight_from_blocks(self._ctx, Q4_F32, C.c_void_p(wire.ctypes.data), rows, cols,
                                                       C.byref(h)))
        else:
            sc = _host(q.scales, np.float32).astype(np.float16).view(np.uint16)
            pk = _host(q.packed, np.uint8)
            self._check(self._L.tq_qweight_from_arrays(self._ctx, Q4_F16, C.c_void_p(pk.ctypes.data),
                                                       C.c_void_p(sc.ctypes.data), rows, cols, C.byref(h)))
        return self._wrap_q(h)

    def upload_q8(self, q: QuantizedQ8) -> QBuffer:
        rows, cols = q.shape
        h = C.c_void_p()
        wire = q.to_wire()
        self._check(self._L.tq_qweight_from_blocks(self._ctx, Q8_F32, C.c_void_p(wire.ctypes.data), rows, cols,
                                                   C.byref(h)))
        return self._wrap_q(h)

    def upload_qarrays(self, kind: int, payload, scales, rows: int, cols: int) -> QBuffer:
        """Structure-of-arrays upload (see ``tq_qweight_from_arrays``)."""
        pdt = np.int8 if kind in (Q8_F32, I8_ROW) else np.uint8
        sdt = np.uint16 if kind == Q4_F16 else np.float32
        pk, sc = _host(payload, pdt), _host(scales, sdt)
        h = C.c_void_p()
        self._check(self._L.tq_qweight_from_arrays(self._ctx, kind, C.c_void_p(pk.ctypes.data),
                                                   C.c_void_p(sc.ctypes.data), rows, cols, C.byref(h)))
        return self._wrap_q(h)

    def qweight_from_device(self, kind: int, payload_ptr: int, scales_ptr: int, rows: int, cols: int) -> QBuffer:
        """Builds a weight from plain block arrays that already live in HBM (read once, see
        ``tq_qweight_from_device_arrays``)."""
        h = C.c_void_p()
        self._check(self._L.tq_qweight_from_device_arrays(self._ctx, kind, C.c_void_p(payload_ptr),
                                                          C.c_void_p(scales_ptr), rows, cols, C.byref(h)))
        return self._wrap_q(h)

    def quantize_matrix(self, src: Buffer, rows: int, cols: int, kind: int) -> QBuffer:
        """``quantize_matrix_q4`` / ``quantize_matrix_q8`` (quantize.rs:193-220) on the device, bit-exact."""
        h = C.c_void_p()
        self._check(self._L.tq_quantize_matrix(self._ctx, C.c_void_p(src.ptr), src.dtype, 0, rows, cols, kind, C.byref(h)))
        return self._wrap_q(h)

    def dequantize(self, w: QBuffer):
        """``dequantize_q4`` / ``dequantize_q8``: returns (f32 [rows, cols], signed integers i8 [rows, cols])."""
        out = self.alloc(w.rows * w.cols, F32)
        ints = self.alloc(w.rows * w.cols, I8)
        self._check(self._L.tq_dequantize(self._ctx, C.c_void_p(w.handle), C.c_void_p(out.ptr), C.c_void_p(ints.ptr)))
        return out.to_vec().reshape(w.rows, w.cols), ints.to_vec().reshape(w.rows, w.cols)

    # ------------------------------------------------------------------ quantised linear
    def qlinear(self, x: Buffer, w: QBuffer, m: int, out_dtype: int = F32, out: Buffer | None = None,
                residual: Buffer | None = None) -> Buffer:
        """``Linear::forward_2d`` with a quantised weight: y[m, rows] = x[m, cols] . W^T."""
        if x.n != m * w.cols:
            raise TangqError(_lib.TQ_EINVAL, f"qlinear: x has {x.n} elements, expected {m}*{w.cols}")
        if out is None:
            out = self.alloc(m * w.rows, out_dtype)
        self._check(self._L.tq_qlinear(self._ctx, C.c_void_p(w.handle), C.c_void_p(x.ptr), x.dtype, 0, m,
                                       C.c_void_p(out.ptr), out.dtype, 0,
                                       C.c_void_p(residual.ptr if residual is not None else 0)))
        return out

    def _matvec_host(self, w: QBuffer, x, m: int):
        x = np.asarray(x)
        if x.dtype == np.float64:
            dt = F64
        elif x.dtype == np.float32:
            dt = F32
        elif x.dtype == np.uint16:
            dt = BF16
        else:
            raise TangqError(_lib.TQ_EINVAL, "matvec input must be f64, f32 or bf16 bit patterns (uint16)")
        x = np.ascontiguousarray(x).reshape(-1)
        if x.size != m * w.cols:  # quantize.rs:230-231 / 259-260 assert_eq!(x.len(), in_dim)
            raise TangqError(_lib.TQ_EINVAL, f"matvec: x has {x.size} elements, expected {m}*{w.cols}")
        y = np.empty(m * w.rows, x.dtype)
        self._check(self._L.tq_q_matvec_host(self._ctx, C.c_void_p(w.handle), C.c_void_p(x.ctypes.data),
                                             C.c_void_p(y.ctypes.data), dt, m))
        return y

    def q_matvec_host_async(self, w: QBuffer, x_ptr: int, y_ptr: int, dtype: int, m: int = 1) -> None:
        """Queues a host-vector matvec without waiting (``tq_q_matvec_host_async``): ``x_ptr`` / ``y_ptr`` are addresses
        of pinned host vectors of ``dtype`` (F64, F32 or BF16) that must stay alive and untouched until ``sync()``."""
        self._check(self._L.tq_q_matvec_host_async(self._ctx, C.c_void_p(w.handle), C.c_void_p(x_ptr), C.c_void_p(y_ptr), dtype, m))

    def q4_matvec(self, w: QBuffer, x) -> np.ndarray:
        """``q4_matvec(&QuantizedQ4, &[f64]) -> Vec<f64>`` (quantize.rs:256-289), host vectors."""
        if w.kind not in (Q4_F32, Q4_F16):
            raise TangqError(_lib.TQ_EINVAL, "q4_matvec needs a Q4 weight")
        return self._matvec_host(w, x, 1)

    def q8_matvec(self, w: QBuffer, x) -> np.ndarray:
        """``q8_matvec(&QuantizedQ8, &[f64]) -> Vec<f64>`` (quantize.rs:227-253), host vectors."""
        if w.kind not in (Q8_F32, I8_ROW):
            raise TangqError(_lib.TQ_EINVAL, "q8_matvec needs a Q8 / int8 weight")
        return self._matvec_host(w, x, 1)

    def q_matmul_host(self, w: QBuffer, x, m: int) -> np.ndarray:
        """m stacked matvecs with host arrays: x [m, cols] -> y [m, rows]."""
        return self._matvec_host(w, x, m).reshape(m, w.rows)

    # ------------------------------------------------------------------ CUDA graphs
    def begin_capture(self) -> None:
        """``begin_capture`` (crates/tang-compute/src/cuda.rs:344)."""
        self._check(self._L.tq_graph_begin(self._ctx))

    def end_capture(self) -> "Graph":
        """``end_capture`` (cuda.rs:350): returns a replayable graph."""
        g = C.c_void_p()
        self._check(self._L.tq_graph_end(self._ctx, C.byref(g)))
        return Graph(self, g.value)

    @property
    def launch_count(self) -> int:
        return int(self._L.tq_launch_count(self._ctx))


class SamplerConfig(C.Structure):
    """``SamplingConfig`` (crates/tang-infer/src/sampling.rs:6-20): temperature, top_k (0 = off), top_p (1 = off),
    repetition_penalty (1 = off)."""
    _fields_ = [("temperature", C.c_double), ("top_k", C.c_uint64), ("top_p", C.c_double), ("repetition_penalty", C.c_double)]


class Graph:
    def __init__(self, dev: QuantComputeDevice, handle: int):
        self.dev, self.handle = dev, handle

    def launch(self) -> None:
        self.dev._check(self.dev._L.tq_graph_launch(self.dev._ctx, C.c_void_p(self.handle)))

    def free(self) -> None:
        if self.handle:
            self.dev._L.tq_graph_free(self.dev._ctx, C.c_void_p(self.handle))
            self.handle = 0


# ---------------------------------------------------------------------- operators of the decode step
def _opt_ptr(buf) -> C.c_void_p:
    return C.c_void_p(buf.ptr if buf is not None else 0)


def _add_ops(cls):
    def rms_norm(self, data: Buffer, weight: Buffer, n_groups: int, dim: int, eps: float, out_dtype: int = F32) -> Buffer:
        """``ComputeDevice::rms_norm(data, weight, n_groups, dim, eps)`` (device.rs:121-128)."""
        out = self.alloc(n_groups * dim, out_dtype)
        self._check(self._L.tq_rms_norm(self._ctx, C.c_void_p(data.ptr), data.dtype, None, C.c_void_p(weight.ptr),
                                        weight.dtype, n_groups, dim, eps, C.c_void_p(out.ptr), out_dtype, None))
        return out

    def rms_norm_residual(self, inp: Buffer, residual: Buffer, weight: Buffer, n_groups: int, dim: int, eps: float,
                          out_dtype: int = F32):
        """``rms_norm_residual`` (device.rs:546-575): returns (normed, input + residual)."""
        out = self.alloc(n_groups * dim, out_dtype)
        s = self.alloc(n_groups * dim, F32)
        self._check(self._L.tq_rms_norm(self._ctx, C.c_void_p(inp.ptr), inp.dtype, C.c_void_p(residual.ptr),
                                        C.c_void_p(weight.ptr), weight.dtype, n_groups, dim, eps, C.c_void_p(out.ptr),
                                        out_dtype, C.c_void_p(s.ptr)))
        return out, s

    def rope_tables(self, head_dim: int, max_seq_len: int, base: float):
        """``InterleavedRoPE::new`` (modules.rs:495-510): device cos / sin tables."""
        half = head_dim // 2
        cos, sin = self.alloc(max_seq_len * half, F32), self.alloc(max_seq_len * half, F32)
        self._check(self._L.tq_rope_tables(self._ctx, head_dim, max_seq_len, base, C.c_void_p(cos.ptr), C.c_void_p(sin.ptr)))
        return cos, sin

    def rope_forward(self, x: Buffer, cos: Buffer, sin: Buffer, seq_len: int, n_heads: int, head_dim: int,
                     start_pos: int = 0, positions: Buffer | None = None, out_dtype: int | None = None) -> Buffer:
        """``rope_forward`` (device.rs:582-610)."""
        out = self.alloc(x.n, x.dtype if out_dtype is None else out_dtype)
        self._check(self._L.tq_rope_forward(self._ctx, C.c_void_p(x.ptr), x.dtype, C.c_void_p(cos.ptr), C.c_void_p(sin.ptr),
                                            _opt_ptr(positions), seq_len, n_heads, head_dim, start_pos, C.c_void_p(out.ptr),
                                            out.dtype))
        return out

    def swiglu_fused(self, gate: Buffer, up: Buffer, out_dtype: int = F32) -> Buffer:
        """``swiglu_fused_buf`` (device.rs:727-736)."""
        out = self.alloc(gate.n, out_dtype)
        self._check(self._L.tq_swiglu(self._ctx, C.c_void_p(gate.ptr), C.c_void_p(up.ptr), gate.dtype, 0, 1, gate.n,
                                      C.c_void_p(out.ptr), out_dtype))
        return out

    def embedding(self, weight: Buffer, ids, seq_len: int, dim: int, out_dtype: int = F32) -> Buffer:
        """``embedding(weight, ids, seq_len, dim)`` (device.rs:131-138); ids: int array or I32 Buffer."""
        idb = ids if isinstance(ids, Buffer) else self.upload(np.asarray(ids, np.int32), _lib.I32)
        out = self.alloc(seq_len * dim, out_dtype)
        self._check(self._L.tq_embedding(self._ctx, C.c_void_p(weight.ptr), weight.dtype, C.c_void_p(idb.ptr), seq_len, dim,
                                         weight.n // dim, C.c_void_p(out.ptr), out_dtype))
        return out

    def kv_attention(self, q: Buffer, k_cache: Buffer, v_cache: Buffer, cache_start: int, q_len: int, n_heads: int,
                     n_kv_heads: int, head_dim: int) -> Buffer:
        """``ComputeDevice::kv_attention`` (device.rs:161-180), f32 buffers."""
        if q.dtype != F32 or k_cache.dtype != F32 or v_cache.dtype != F32:
            raise TangqError(_lib.TQ_EINVAL, "kv_attention takes f32 buffers; use gqa_decode for the bf16 cache")
        if q.n != q_len * n_heads * head_dim or k_cache.n < (cache_start + q_len) * n_kv_heads * head_dim:
            raise TangqError(_lib.TQ_EINVAL, "kv_attention: buffer sizes do not match the shapes")
        out = self.alloc(q.n, F32)
        self._check(self._L.tq_kv_attention(self._ctx, C.c_void_p(q.ptr), C.c_void_p(k_cache.ptr), C.c_void_p(v_cache.ptr),
                                            cache_start, q_len, n_heads, n_kv_heads, head_dim, C.c_void_p(out.ptr)))
        return out

    def gqa_decode(self, q: Buffer, k_cache: Buffer, v_cache: Buffer, lens, batch: int, n_heads: int, n_kv_heads: int,
                   head_dim: int, seq_stride: int, max_len: int, out_dtype: int = BF16) -> Buffer:
        """Batched single-token decode attention over bf16 caches (``tq_gqa_decode``)."""
        lb = lens if isinstance(lens, Buffer) else self.upload(np.asarray(lens, np.int32), _lib.I32)
        out = self.alloc(batch * n_heads * head_dim, out_dtype)
        self._check(self._L.tq_gqa_decode(self._ctx, C.c_void_p(q.ptr), C.c_void_p(k_cache.ptr), C.c_void_p(v_cache.ptr),
                                          C.c_void_p(lb.ptr), batch, n_heads, n_kv_heads, head_dim, seq_stride, max_len,
                                          C.c_void_p(out.ptr), out_dtype))
        return out

    def gqa_prefill(self, q: Buffer, k_cache: Buffer, v_cache: Buffer, cache_start, batch: int, q_len: int, n_heads: int,
                    n_kv_heads: int, head_dim: int, seq_stride: int, out_dtype: int = BF16) -> Buffer:
        """``kv_attention`` with q_len > 1 (device.rs:161-180) over bf16 caches, batched: query i of sequence b attends
        positions 0 .. cache_start[b] + i (``tq_gqa_prefill``)."""
        cb = cache_start if isinstance(cache_start, Buffer) else self.upload(np.asarray(cache_start, np.int32), _lib.I32)
        out = self.alloc(batch * q_len * n_heads * head_dim, out_dtype)
        self._check(self._L.tq_gqa_prefill(self._ctx, C.c_void_p(q.ptr), C.c_void_p(k_cache.ptr), C.c_void_p(v_cache.ptr),
                                           C.c_void_p(cb.ptr), batch, q_len, n_heads, n_kv_heads, head_dim, seq_stride,
                                           C.c_void_p(out.ptr), out_dtype))
        out._keep = cb
        return out

    def concat_rows(self, parts) -> QBuffer:
        arr = (C.c_void_p * len(parts))(*[p.handle for p in parts])
        h = C.c_void_p()
        self._check(self._L.tq_qweight_concat_rows(self._ctx, arr, len(parts), C.byref(h)))
        return self._wrap_q(h)

    def interleave_gate_up(self, w: QBuffer, free_source: bool = True) -> QBuffer:
        """A fused [gate; up] weight regrouped for the in-kernel SwiGLU (``tq_qweight_interleave_gate_up``)."""
        h = C.c_void_p()
        self._check(self._L.tq_qweight_interleave_gate_up(self._ctx, C.c_void_p(w.handle), C.byref(h)))
        out = self._wrap_q(h)
        if free_source:
            self.sync()
            w.free()
        return out

    for f in (rms_norm, rms_norm_residual, rope_tables, rope_forward, swiglu_fused, embedding, kv_attention, gqa_decode,
              gqa_prefill, concat_rows, interleave_gate_up):
        setattr(cls, f.__name__, f)


_add_ops(QuantComputeDevice)
