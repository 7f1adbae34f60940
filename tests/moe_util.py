"""Random MoE layer on the host (oracle form) and on the device, from the same arrays."""
import numpy as np

from util import bf16_round, make_weight

KIND = 1


class HostMoe:
    def __init__(self, rng, d, ffn, n_experts, top_k, n_shared, renorm=False):
        self.d, self.ffn, self.E, self.k, self.n_shared, self.renorm = d, ffn, n_experts, top_k, n_shared, renorm
        self.wg_bits, self.wg = bf16_round(rng.normal(0, 0.02, (n_experts, d)).astype(np.float32))
        mk = lambda r, c: make_weight(rng, KIND, r, c) + (r, c)
        self.experts = [dict(gate=mk(ffn, d), up=mk(ffn, d), down=mk(d, ffn)) for _ in range(n_experts + n_shared)]

    def oracle(self, orc, h_f32):
        """h_f32 [T, d] (bf16-exact values).  Returns (out f64 [T, d], idx [T, k], weights [T, k], logits [T, E])."""
        T = h_f32.shape[0]
        out = np.zeros((T, self.d))
        idxs, ws, lgs = [], [], []
        qw = lambda w: orc.qweight(KIND, w[0], w[1], w[2], w[3])
        for t in range(T):
            x = h_f32[t].astype(np.float64)
            idx, w, lg = orc.router_f64(x, self.wg.astype(np.float64), self.E, self.k, self.renorm)
            for e, p in zip(idx, w):
                ex = self.experts[e]
                out[t] += p * orc.expert_ffn_f64(qw(ex["gate"]), qw(ex["up"]), qw(ex["down"]), x)
            for s in range(self.n_shared):
                ex = self.experts[self.E + s]
                out[t] += orc.expert_ffn_f64(qw(ex["gate"]), qw(ex["up"]), qw(ex["down"]), x)
            idxs.append(idx)
            ws.append(w)
            lgs.append(lg)
        return out, np.array(idxs), np.array(ws), np.array(lgs)

    def to_device(self, dev, ep_rank=0, ep_size=1):
        import tang_b200 as tb

        nl = self.E // ep_size
        lo = ep_rank * nl
        cat = lambda ws: (np.concatenate([w[0] for w in ws]), np.concatenate([w[1] for w in ws]))
        gu = cat([w for e in self.experts[lo:lo + nl] for w in (e["gate"], e["up"])])
        dn = cat([e["down"] for e in self.experts[lo:lo + nl]])
        w_gu = dev.upload_qarrays(KIND, gu[1], gu[0], nl * 2 * self.ffn, self.d)
        w_dn = dev.upload_qarrays(KIND, dn[1], dn[0], nl * self.d, self.ffn)
        sh_gu, sh_dn = [], []
        for e in self.experts[self.E:]:
            g = cat([e["gate"], e["up"]])
            sh_gu.append(dev.upload_qarrays(KIND, g[1], g[0], 2 * self.ffn, self.d))
            sh_dn.append(dev.upload_qarrays(KIND, e["down"][1], e["down"][0], self.d, self.ffn))
        cfg = tb.MoeConfig(self.d, self.ffn, self.E, self.k, self.n_shared, int(self.renorm), ep_rank, ep_size)
        return tb.MoeLayer(dev, cfg, dev.upload(self.wg_bits, tb.BF16), w_gu, w_dn, sh_gu, sh_dn)
