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
