"""Host-side driver of the Llama-shaped decode step (``tq_llama_*`` in include/tangq.h), mirroring
the reference's decode loop, crates/tang-train/examples/smollm.rs:255-296 (``LlamaModel::forward``
for one new token per sequence) and its use of ``tang_infer::KVCache``."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from .device import Buffer, QBuffer, QuantComputeDevice


class LlamaConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab",
                                          "max_seq", "max_batch")] + [("eps", C.c_float), ("rope_base", C.c_double)]


class Comm:
    """NCCL communicator bound to a device context (``tq_comm_*``)."""

    def __init__(self, dev: QuantComputeDevice, unique_id: bytes, rank: int, world: int):
        self.dev = dev
        h = C.c_void_p()
        buf = C.create_string_buffer(unique_id, 128)
        dev._check(dev._L.tq_comm_create(dev._ctx, buf, rank, world, C.byref(h)))
        self.handle, self.rank, self.world = h.value, rank, world

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        st = _lib.load().tq_comm_unique_id(buf)
        if st != _lib.TQ_OK:
            raise _lib.TangqError(st, "tq_comm_unique_id failed (NCCL not loadable?)")
        return buf.raw

    def enable_peer(self, max_elems: int) -> None:
        """Peer-memory path for all-reduces of up to `max_elems` floats (``tq_comm_enable_peer``); collective."""
        self.dev._check(self.dev._L.tq_comm_enable_peer(self.dev._ctx, C.c_void_p(self.handle), max_elems))

    @classmethod
    def peer_local(cls, dev: QuantComputeDevice, rank: int, world: int, bufs, max_elems: int) -> "Comm":
        """A communicator over buffers already visible to this GPU (``tq_comm_peer_local``): `bufs[r]` is rank r's."""
        self = cls.__new__(cls)
        self.dev = dev
        arr = (C.c_void_p * world)(*[b.ptr for b in bufs])
        h = C.c_void_p()
        dev._check(dev._L.tq_comm_peer_local(dev._ctx, rank, world, arr, max_elems, C.byref(h)))
        self.handle, self.rank, self.world = h.value, rank, world
        return self

    def set_wait_limit(self, polls: int) -> None:
        st = self.dev._L.tq_comm_set_wait_limit(C.c_void_p(self.handle), polls)
        if st != _lib.TQ_OK:
            raise _lib.TangqError(st, "tq_comm_set_wait_limit: no peer path on this communicator")

    def all_reduce(self, buf: Buffer) -> None:
        self.dev._check(self.dev._L.tq_all_reduce_f32(self.dev._ctx, C.c_void_p(self.handle), C.c_void_p(buf.ptr), buf.n))

    def destroy(self) -> None:
        if self.handle:
            self.dev._L.tq_comm_destroy(self.dev._ctx, C.c_void_p(self.handle))
            self.handle = 0


@dataclass
class LlamaLayerWeights:
    """One block's device weights in the fused form the kernels take (shard shapes under TP)."""
    wqkv: QBuffer
    wo: QBuffer
    wgate_up: QBuffer
    wdown: QBuffer
    attn_norm: Buffer   # bf16 [d_model]
    ffn_norm: Buffer    # bf16 [d_model]


class LlamaModel:
    def __init__(self, dev: QuantComputeDevice, cfg: LlamaConfig, comm: Comm | None = None):
        self.dev, self.cfg, self.comm = dev, cfg, comm
        self.tp = comm.world if comm else 1
        h = C.c_void_p()
        dev._check(dev._L.tq_llama_create(dev._ctx, C.byref(cfg), C.c_void_p(comm.handle if comm else 0), C.byref(h)))
        self.handle = h.value
        self._keep = []

    def set_layer(self, layer: int, w: LlamaLayerWeights) -> None:
        self._keep.append(w)
        self.dev._check(self.dev._L.tq_llama_set_layer(
            C.c_void_p(self.handle), layer, C.c_void_p(w.wqkv.handle), C.c_void_p(w.wo.handle),
            C.c_void_p(w.wgate_up.handle), C.c_void_p(w.wdown.handle), C.c_void_p(w.attn_norm.ptr),
            C.c_void_p(w.ffn_norm.ptr)))

    def set_head(self, embed: Buffer, final_norm: Buffer, lm_head: QBuffer) -> None:
        self._keep.append((embed, final_norm, lm_head))
        self.dev._check(self.dev._L.tq_llama_set_head(C.c_void_p(self.handle), C.c_void_p(embed.ptr),
                                                      C.c_void_p(final_norm.ptr), C.c_void_p(lm_head.handle)))

    def kv_cache(self, layer: int):
        """(k_ptr, v_ptr, seq_stride_elems) of this rank's bf16 cache for `layer`."""
        k, v, s = C.c_void_p(), C.c_void_p(), C.c_size_t()
        self.dev._check(self.dev._L.tq_llama_kv_cache(C.c_void_p(self.handle), layer, C.byref(k), C.byref(v), C.byref(s)))
        return k.value, v.value, s.value

    def kv_buffers(self, layer: int):
        k, v, s = self.kv_cache(layer)
        n = self.cfg.max_batch * s
        return (Buffer(self.dev, k, n, _lib.BF16, owns=False), Buffer(self.dev, v, n, _lib.BF16, owns=False), s)

    def trim_to(self, seq_lens: Buffer, batch: int, keep: int) -> None:
        """``KVCache::trim_to(keep)`` (crates/tang-infer/src/kv_cache.rs:138-149) for `batch` sequences: each keeps its
        last `keep` positions (moved to the front of its cache rows); `seq_lens` (int32, device) is updated in place."""
        self.dev._check(self.dev._L.tq_llama_kv_trim(C.c_void_p(self.handle), C.c_void_p(seq_lens.ptr), batch, keep))

    def decode(self, token_ids: Buffer, positions: Buffer, batch: int, max_len: int, logits: Buffer,
               rope_positions: Buffer | None = None) -> None:
        """``model.forward(&[tok], cache, pos)`` for `batch` sequences (smollm.rs:535); asynchronous.  `positions` are the
        cache rows the new tokens are appended at; `rope_positions` the positions their rotation uses when that differs
        (a trimmed cache)."""
        self.dev._check(self.dev._L.tq_llama_decode_at(C.c_void_p(self.handle), C.c_void_p(token_ids.ptr), C.c_void_p(positions.ptr),
                                                       C.c_void_p(rope_positions.ptr if rope_positions is not None else 0),
                                                       batch, max_len, C.c_void_p(logits.ptr)))

    def prefill(self, token_ids: Buffer, cache_start: Buffer, batch: int, q_len: int, logits: Buffer) -> None:
        """``model.forward(&tokens, cache, pos)`` for a chunk of `q_len` tokens per sequence (prompt processing): appends the
        chunk to the cache and leaves the logits of each sequence's last chunk position; asynchronous."""
        self.dev._check(self.dev._L.tq_llama_prefill(C.c_void_p(self.handle), C.c_void_p(token_ids.ptr), C.c_void_p(cache_start.ptr),
                                                     batch, q_len, C.c_void_p(logits.ptr)))

    def generate(self, prompts, n_new: int, sampling=None, seed: int = 42, comm_world: int = 1) -> np.ndarray:
        """``generate`` (crates/tang-infer/src/sampling.rs:229-256) for a batch of equal-length prompts.  The prompt
        goes through one prefill chunk (all tokens but the last); then decode -> ``Sampler::sample`` -> advance is captured
        once as a CUDA graph and replayed `n_new` times, the logits never leaving the device.  `sampling` is a
        ``SamplerConfig`` (None or temperature 0: greedy, the first maximum); every sequence owns an LCG seeded
        with `seed` (as ``Sampler::with_seed`` per call of ``generate``); the repetition penalty sees the prompt and
        everything generated so far.  Returns int32 [batch, n_new]; the caller cuts at its stop token (what is
        drawn before a stop token does not depend on what follows)."""
        from .device import SamplerConfig

        dev, L = self.dev, self.dev._L
        prompts = np.asarray(prompts, np.int32)
        B, P = prompts.shape
        if P < 1 or n_new < 1:
            raise _lib.TangqError(_lib.TQ_EINVAL, "generate: need at least one prompt token and one new token")
        if P + n_new > self.cfg.max_seq:
            raise _lib.TangqError(_lib.TQ_EINVAL, "generate: prompt + new tokens exceed max_seq")
        cfg = sampling if sampling is not None else SamplerConfig(0.0, 0, 1.0, 1.0)
        vocab, ld = self.cfg.vocab, P + n_new
        logits = dev.alloc(B * vocab, _lib.F32)
        tok, pos = dev.alloc(B, _lib.I32), dev.alloc(B, _lib.I32)
        chosen = dev.alloc(B, _lib.I32)
        step = dev.upload(np.full(1, P, np.int32), _lib.I32)            # column of the history the next token goes to
        hist = np.zeros((B, ld), np.int32)
        hist[:, :P] = prompts
        hist_d = dev.upload(hist, _lib.I32)                             # prompt + generated tokens: the penalty's past
        lens = dev.upload(np.full(B, P, np.int32), _lib.I32)
        rng = dev.upload(np.full(B, seed, np.uint64).view(np.float64), _lib.F64)
        if P > 1:                                   # all prompt tokens but the last: one prefill chunk fills the cache
            self.prefill(dev.upload(np.ascontiguousarray(prompts[:, :P - 1]), _lib.I32), dev.upload(np.zeros(B, np.int32), _lib.I32),
                         B, P - 1, logits)
        dev.upload_into(tok, prompts[:, P - 1].copy())
        dev.upload_into(pos, np.full(B, P - 1, np.int32))

        def one():
            self.decode(tok, pos, B, P + n_new, logits)
            dev._check(L.tq_sample(dev._ctx, C.c_void_p(logits.ptr), comm_world, B, vocab // comm_world, C.byref(cfg),
                                   C.c_void_p(rng.ptr), C.c_void_p(hist_d.ptr), C.c_void_p(lens.ptr), ld, C.c_void_p(chosen.ptr)))
            dev._check(L.tq_generate_advance(dev._ctx, C.c_void_p(chosen.ptr), B, C.c_void_p(tok.ptr), C.c_void_p(pos.ptr),
                                             C.c_void_p(hist_d.ptr), ld, C.c_void_p(step.ptr), C.c_void_p(lens.ptr)))
        one()                                       # eager once (workspaces), then the remaining steps from a graph
        if n_new > 1:
            dev.sync()
            dev.begin_capture()
            one()
            graph = dev.end_capture()
            for _ in range(n_new - 1):
                graph.launch()
            dev.sync()
            graph.free()
        dev.sync()
        return hist_d.to_vec().reshape(B, ld)[:, P:].copy()

    def generate_greedy(self, prompts, n_new: int, comm_world: int = 1) -> np.ndarray:
        """``generate`` with ``SamplingConfig::greedy()``."""
        return self.generate(prompts, n_new, None, comm_world=comm_world)

    def destroy(self) -> None:
        if self.handle:
            self.dev._L.tq_llama_destroy(C.c_void_p(self.handle))
            self.handle = 0
