"""Host-side driver of the MLA decode attention (``tq_mla_*`` in include/tangq.h).  The reference has
no MLA; this mirrors its operator style (buffers + explicit dimensions, like ``kv_attention``,
crates/tang-compute/src/device.rs:161-180)."""
from __future__ import annotations

import ctypes as C
import math

import numpy as np

from . import _lib
from .device import Buffer, QBuffer, QuantComputeDevice

KV_LORA, ROPE = 512, 64


def mla_decode(dev: QuantComputeDevice, w_qk: QBuffer, w_uv: QBuffer, q_nope: Buffer, q_rope: Buffer, cache: Buffer, lens,
               batch: int, n_heads: int, nope_dim: int, v_dim: int, seq_stride: int, max_len: int,
               out_dtype: int = _lib.F32) -> Buffer:
    """Absorb q, attend over the latent cache, un-absorb: returns o [batch, n_heads, v_dim]."""
    L = dev._L
    lb = lens if isinstance(lens, Buffer) else dev.upload(np.asarray(lens, np.int32), _lib.I32)
    q_full = dev.alloc(batch * n_heads * (KV_LORA + ROPE), _lib.BF16)
    o_lat = dev.alloc(batch * n_heads * KV_LORA, _lib.BF16)
    out = dev.alloc(batch * n_heads * v_dim, out_dtype)
    dev._check(L.tq_mla_absorb_q(dev._ctx, C.c_void_p(w_qk.handle), C.c_void_p(q_nope.ptr), C.c_void_p(q_rope.ptr), batch,
                                 n_heads, nope_dim, C.c_void_p(q_full.ptr)))
    dev._check(L.tq_mla_decode(dev._ctx, C.c_void_p(q_full.ptr), C.c_void_p(cache.ptr), C.c_void_p(lb.ptr), batch, n_heads,
                               KV_LORA, ROPE, seq_stride, max_len, 1.0 / math.sqrt(nope_dim + ROPE), C.c_void_p(o_lat.ptr)))
    dev._check(L.tq_mla_unabsorb(dev._ctx, C.c_void_p(w_uv.handle), C.c_void_p(o_lat.ptr), batch, n_heads, v_dim,
                                 C.c_void_p(out.ptr), out_dtype))
    out._keep = (q_full, o_lat, lb)
    return out


class MlaConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("d_model", "n_heads", "q_lora", "kv_lora", "nope_dim", "rope_dim", "v_dim", "max_batch",
                                          "max_pos")] + [("norm_eps", C.c_float)]


class MlaLayer:
    """One MLA attention layer of a decode step (``tq_mla_create`` / ``tq_mla_layer_decode``): hidden rows ->
    q_a -> RMSNorm -> q_b -> RoPE on the 64 rope dimensions -> absorbed attention over the latent cache -> W_UV ->
    row-parallel W_O (+ the sum over the ranks).  ``cfg.n_heads`` is this rank's head count."""

    def __init__(self, dev: QuantComputeDevice, cfg: MlaConfig, q_a: QBuffer, q_norm_gain: Buffer | None, q_b: QBuffer,
                 w_qk: QBuffer, w_uv: QBuffer, w_o: QBuffer, rope_base: float = 10000.0):
        self.dev, self.cfg = dev, cfg
        self.cos = dev.alloc(cfg.max_pos * (cfg.rope_dim // 2), _lib.F32)
        self.sin = dev.alloc(cfg.max_pos * (cfg.rope_dim // 2), _lib.F32)
        dev._check(dev._L.tq_rope_tables(dev._ctx, cfg.rope_dim, cfg.max_pos, C.c_double(rope_base), C.c_void_p(self.cos.ptr),
                                         C.c_void_p(self.sin.ptr)))
        self._keep = (q_a, q_norm_gain, q_b, w_qk, w_uv, w_o)
        h = C.c_void_p()
        dev._check(dev._L.tq_mla_create(dev._ctx, C.byref(cfg), C.c_void_p(q_a.handle), C.c_void_p(q_norm_gain.ptr if q_norm_gain else 0),
                                        C.c_void_p(q_b.handle), C.c_void_p(w_qk.handle), C.c_void_p(w_uv.handle),
                                        C.c_void_p(w_o.handle), C.c_void_p(self.cos.ptr), C.c_void_p(self.sin.ptr), C.byref(h)))
        self.handle = h.value

    def decode(self, h: Buffer, cache: Buffer, lens: Buffer, batch: int, seq_stride: int, max_len: int, comm=None,
               out: Buffer | None = None) -> Buffer:
        """h bf16 [batch, d_model], cache bf16 [batch][seq_stride], lens int32 [batch] -> f32 [batch, d_model]."""
        out = out or self.dev.alloc(batch * self.cfg.d_model, _lib.F32)
        self.dev._check(self.dev._L.tq_mla_layer_decode(C.c_void_p(self.handle), C.c_void_p(h.ptr), C.c_void_p(cache.ptr),
                                                        C.c_void_p(lens.ptr), batch, seq_stride, max_len,
                                                        C.c_void_p(comm.handle if comm else 0), C.c_void_p(out.ptr)))
        return out

    def destroy(self) -> None:
        if self.handle:
            self.dev._L.tq_mla_destroy(C.c_void_p(self.handle))
            self.handle = 0
