"""Builds one random Llama-shaped model twice — as oracle structs and as device weights — from the
same host arrays, and runs the oracle's decode step."""
import numpy as np

from util import bf16_round, make_weight

KIND = 1  # int4 group-32 with f16 scales (the benchmark configuration)


class HostLlama:
    def __init__(self, rng, n_layers, d, n_heads, n_kv, hd, ffn, vocab, eps=1e-5, rope_base=500000.0):
        self.n_layers, self.d, self.n_heads, self.n_kv, self.hd, self.ffn, self.vocab = n_layers, d, n_heads, n_kv, hd, ffn, vocab
        self.eps, self.rope_base = eps, rope_base
        q_dim, kv_dim = n_heads * hd, n_kv * hd
        self.layers = []
        for _ in range(n_layers):
            L = {}
            for name, (r, c) in dict(wq=(q_dim, d), wk=(kv_dim, d), wv=(kv_dim, d), wo=(d, q_dim), gate=(ffn, d),
                                     up=(ffn, d), down=(d, ffn)).items():
                L[name] = make_weight(rng, KIND, r, c) + (r, c)
            L["attn_norm"] = bf16_round(rng.normal(0, 0.02, d).astype(np.float32))[0]
            L["ffn_norm"] = bf16_round(rng.normal(0, 0.02, d).astype(np.float32))[0]
            self.layers.append(L)
        self.embed = bf16_round(rng.normal(0, 0.02, (vocab, d)).astype(np.float32))[0]
        self.final_norm = bf16_round(rng.normal(0, 0.02, d).astype(np.float32))[0]
        self.lm_head = make_weight(rng, KIND, vocab, d) + (vocab, d)

    # ------------------------------------------------------------------ oracle side
    def oracle_decode(self, orc, token, k_caches, v_caches, pos, threads=0, rope_pos=None):
        """k_caches / v_caches: per layer uint16 [max_seq, kv_dim] (updated in place).  Returns f64 logits.
        `pos` is the cache row of the new token; `rope_pos` its position for the rotation when that differs."""
        dims = orc.LlamaDims(self.d, self.n_heads, self.n_kv, self.hd, self.ffn, self.rope_base, self.eps)
        hidden = ((self.embed[token].astype(np.uint32) << 16).view(np.float32)).astype(np.float64)
        for li, L in enumerate(self.layers):
            ol = orc.LlamaLayer()
            for name in ("wq", "wk", "wv", "wo", "gate", "up", "down"):
                sc, pay, r, c = L[name]
                setattr(ol, name, orc.qweight(KIND, sc, pay, r, c))
            ol.attn_norm_bf16 = L["attn_norm"].ctypes.data
            ol.ffn_norm_bf16 = L["ffn_norm"].ctypes.data
            orc.llama_layer_f64(dims, ol, hidden, k_caches[li], v_caches[li], pos, threads, rope_pos)
        sc, pay, r, c = self.lm_head
        return orc.llama_head_f64(dims, self.final_norm, orc.qweight(KIND, sc, pay, r, c), hidden, threads)

    # ------------------------------------------------------------------ device side
    def shard(self, rank, tp):
        """Plain arrays of this rank's shard in the fused forms the device takes."""
        hd, d = self.hd, self.d
        hl, kl, fl, vl = self.n_heads // tp, self.n_kv // tp, self.ffn // tp, self.vocab // tp
        out = []

        def rows(w, lo, hi):
            sc, pay, r, c = w
            return sc[lo:hi], pay[lo:hi]

        def cols(w, lo, hi):           # K slice on 32-block boundaries
            sc, pay, r, c = w
            return np.ascontiguousarray(sc[:, lo // 32:hi // 32]), np.ascontiguousarray(pay[:, lo // 2:hi // 2])

        def cat(parts):
            return np.concatenate([p[0] for p in parts]), np.concatenate([p[1] for p in parts])

        for L in self.layers:
            qkv = cat([rows(L["wq"], rank * hl * hd, (rank + 1) * hl * hd), rows(L["wk"], rank * kl * hd, (rank + 1) * kl * hd),
                       rows(L["wv"], rank * kl * hd, (rank + 1) * kl * hd)])
            gu = cat([rows(L["gate"], rank * fl, (rank + 1) * fl), rows(L["up"], rank * fl, (rank + 1) * fl)])
            out.append(dict(wqkv=qkv + ((hl + 2 * kl) * hd, d), wo=cols(L["wo"], rank * hl * hd, (rank + 1) * hl * hd) + (d, hl * hd),
                            wgu=gu + (2 * fl, d), wdown=cols(L["down"], rank * fl, (rank + 1) * fl) + (d, fl),
                            attn_norm=L["attn_norm"], ffn_norm=L["ffn_norm"]))
        head = rows(self.lm_head, rank * vl, (rank + 1) * vl) + (vl, d)
        return out, head

    def to_device(self, dev, max_seq, max_batch, comm=None, interleave=True):
        """`interleave`: hand the gate/up weight over in the interleaved row order (SwiGLU fused into the projection);
        False keeps the reference's [gate; up] order and the separate SwiGLU operator."""
        import tang_b200 as tb

        tp = comm.world if comm else 1
        rank = comm.rank if comm else 0
        cfg = tb.LlamaConfig(self.n_layers, self.d, self.n_heads, self.n_kv, self.hd, self.ffn, self.vocab, max_seq,
                             max_batch, self.eps, self.rope_base)
        model = tb.LlamaModel(dev, cfg, comm)
        layers, head = self.shard(rank, tp)
        for i, L in enumerate(layers):
            up = lambda w: dev.upload_qarrays(KIND, w[1], w[0], w[2], w[3])
            wgu = dev.interleave_gate_up(up(L["wgu"])) if interleave else up(L["wgu"])
            model.set_layer(i, tb.LlamaLayerWeights(up(L["wqkv"]), up(L["wo"]), wgu, up(L["wdown"]),
                                                    dev.upload(L["attn_norm"], tb.BF16), dev.upload(L["ffn_norm"], tb.BF16)))
        model.set_head(dev.upload(self.embed, tb.BF16), dev.upload(self.final_norm, tb.BF16),
                       dev.upload_qarrays(KIND, head[1], head[0], head[2], head[3]))
        return model
