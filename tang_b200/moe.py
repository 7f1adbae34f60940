"""Host-side driver of the mixture-of-experts FFN layer (``tq_moe_*`` in include/tangq.h).  The
reference has no MoE; names follow its operator style (router, expert FFN, top-k as in
crates/tang-infer/src/sampling.rs)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .device import Buffer, QBuffer, QuantComputeDevice


class MoeConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("d_model", "ffn", "n_experts", "top_k", "n_shared", "renormalize", "ep_rank",
                                          "ep_size")]


def moe_router(dev: QuantComputeDevice, h: Buffer, wg: Buffer, n_tokens: int, d_model: int, n_experts: int, top_k: int,
               renormalize: bool = False):
    """Returns (idx int32 [T, k], weights f32 [T, k], logits f64 [T, E]) as numpy arrays."""
    idx = dev.alloc(n_tokens * top_k, _lib.I32)
    w = dev.alloc(n_tokens * top_k, _lib.F32)
    lg = dev.alloc(n_tokens * n_experts, _lib.F64)
    dev._check(dev._L.tq_moe_router(dev._ctx, C.c_void_p(h.ptr), C.c_void_p(wg.ptr), n_tokens, d_model, n_experts, top_k,
                                    int(renormalize), C.c_void_p(idx.ptr), C.c_void_p(w.ptr), C.c_void_p(lg.ptr)))
    dev.sync()
    return (idx.to_vec().reshape(n_tokens, top_k), w.to_vec().reshape(n_tokens, top_k),
            lg.to_vec().reshape(n_tokens, n_experts))


class MoeLayer:
    def __init__(self, dev: QuantComputeDevice, cfg: MoeConfig, wg: Buffer, gate_up_stacked: QBuffer, down_stacked: QBuffer,
                 shared_gate_up=(), shared_down=()):
        self.dev, self.cfg = dev, cfg
        self._keep = (wg, gate_up_stacked, down_stacked, list(shared_gate_up), list(shared_down))
        n = len(shared_gate_up)
        a = (C.c_void_p * max(n, 1))(*[w.handle for w in shared_gate_up])
        b = (C.c_void_p * max(n, 1))(*[w.handle for w in shared_down])
        h = C.c_void_p()
        dev._check(dev._L.tq_moe_create(dev._ctx, C.byref(cfg), C.c_void_p(wg.ptr), C.c_void_p(gate_up_stacked.handle),
                                        C.c_void_p(down_stacked.handle), a, b, C.byref(h)))
        self.handle = h.value

    def forward(self, h: Buffer, n_tokens: int, out: Buffer | None = None, comm=None, want_routing: bool = False):
        """h bf16 [T, d_model] -> f32 [T, d_model]; with want_routing also (idx, weights) buffers."""
        k = self.cfg.top_k
        out = out or self.dev.alloc(n_tokens * self.cfg.d_model, _lib.F32)
        idx = self.dev.alloc(n_tokens * k, _lib.I32) if want_routing else None
        w = self.dev.alloc(n_tokens * k, _lib.F32) if want_routing else None
        self.dev._check(self.dev._L.tq_moe_ffn(C.c_void_p(self.handle), C.c_void_p(h.ptr), n_tokens, C.c_void_p(out.ptr),
                                               C.c_void_p(comm.handle if comm else 0), C.c_void_p(idx.ptr if idx else 0),
                                               C.c_void_p(w.ptr if w else 0)))
        return (out, idx, w) if want_routing else out

    def forward_dispatch(self, h_local: Buffer, n_tokens: int, comm=None, out: Buffer | None = None, want_routing: bool = False):
        """Tokens sharded over the expert-parallel ranks: h_local holds THIS rank's bf16 [n_tokens, d_model] rows;
        all-to-all dispatch to the experts' owners, all-to-all combine back (``tq_moe_ffn_dispatch``)."""
        k = self.cfg.top_k
        out = out or self.dev.alloc(n_tokens * self.cfg.d_model, _lib.F32)
        idx = self.dev.alloc(n_tokens * k, _lib.I32) if want_routing else None
        w = self.dev.alloc(n_tokens * k, _lib.F32) if want_routing else None
        self.dev._check(self.dev._L.tq_moe_ffn_dispatch(C.c_void_p(self.handle), C.c_void_p(h_local.ptr), n_tokens,
                                                        C.c_void_p(out.ptr), C.c_void_p(comm.handle if comm else 0),
                                                        C.c_void_p(idx.ptr if idx else 0), C.c_void_p(w.ptr if w else 0)))
        return (out, idx, w) if want_routing else out

    def destroy(self) -> None:
        if self.handle:
            self.dev._L.tq_moe_destroy(C.c_void_p(self.handle))
            self.handle = 0
