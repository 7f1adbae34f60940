"""Worker of the tensor-parallel decode tests: one process per rank.

    torchrun --nproc-per-node N tests/tp_worker.py gpu     # NCCL, libtangq on N GPUs
    torchrun --nproc-per-node N tests/tp_worker.py cpu     # gloo, the oracle's arithmetic, no GPU

Both modes build the same seeded Llama-shaped model on every rank, shard it with
HostLlama.shard, run one decode step over the shards with the collectives of the device path
(all-reduce after o_proj and down, all-gather of the vocabulary slices), and rank 0 compares the
logits with the unsharded oracle.  Exit code 0 = parity.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

import oracle as orc  # noqa: E402
from llama_util import KIND, HostLlama  # noqa: E402
from util import bf16_round, rel_err  # noqa: E402


def f32_of(bits):
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def make_case():
    host = HostLlama(np.random.default_rng(7), n_layers=2, d=512, n_heads=8, n_kv=4, hd=128, ffn=1024, vocab=2048)
    rng = np.random.default_rng(8)
    B, max_seq = 2, 96
    ctx = [40, 77]
    kv_dim = host.n_kv * host.hd
    caches = [(bf16_round(rng.standard_normal((B, max_seq, kv_dim)).astype(np.float32))[0],
               bf16_round(rng.standard_normal((B, max_seq, kv_dim)).astype(np.float32))[0]) for _ in range(host.n_layers)]
    tokens = rng.integers(0, host.vocab, B).astype(np.int32)
    return host, B, max_seq, ctx, caches, tokens


def oracle_logits(host, B, ctx, caches, tokens):
    out = []
    for b in range(B):
        ks = [c[0][b].copy() for c in caches]
        vs = [c[1][b].copy() for c in caches]
        out.append(host.oracle_decode(orc, int(tokens[b]), ks, vs, ctx[b]))
    return np.stack(out)


def cpu_rank_decode(host, rank, tp, dist, torch, b, token, caches, pos):
    """One sequence through this rank's shards with the oracle's arithmetic (f64, bf16 rounding points)."""
    layers, head = host.shard(rank, tp)
    hd, d = host.hd, host.d
    hl, kl, fl = host.n_heads // tp, host.n_kv // tp, host.ffn // tp
    rb = lambda v: orc.round_bf16(np.asarray(v, np.float32)).astype(np.float64)

    def allreduce(v):
        t = torch.from_numpy(np.ascontiguousarray(v))
        dist.all_reduce(t)
        return t.numpy()

    h = f32_of(host.embed[token]).astype(np.float64)
    for li, L in enumerate(layers):
        xn = rb(orc.rms_norm_f64(h, f32_of(L["attn_norm"]).astype(np.float64), host.eps))
        sc, pay, r, c = L["wqkv"]
        qkv = orc.qmatmul(KIND, sc, pay, r, c, xn)
        q, k, v = qkv[:hl * hd], qkv[hl * hd:(hl + kl) * hd], qkv[(hl + kl) * hd:]
        q = rb(orc.rope_heads_f64(q, hl, hd, pos, host.rope_base))
        k = orc.rope_heads_f64(k, kl, hd, pos, host.rope_base)
        kc = caches[li][0][b][:, rank * kl * hd:(rank + 1) * kl * hd].copy()
        vc = caches[li][1][b][:, rank * kl * hd:(rank + 1) * kl * hd].copy()
        kc[pos], vc[pos] = bf16_round(k.astype(np.float32))[0], bf16_round(v.astype(np.float32))[0]
        attn = rb(orc.attention_decode_f64(q, f32_of(kc[:pos + 1]).astype(np.float64), f32_of(vc[:pos + 1]).astype(np.float64),
                                           pos + 1, hl, kl, hd))
        sc, pay, r, c = L["wo"]
        h = h + allreduce(orc.qmatmul(KIND, sc, pay, r, c, attn))
        xn = rb(orc.rms_norm_f64(h, f32_of(L["ffn_norm"]).astype(np.float64), host.eps))
        sc, pay, r, c = L["wgu"]
        gu = orc.qmatmul(KIND, sc, pay, r, c, xn)
        act = rb(orc.swiglu_f64(gu[:fl], gu[fl:]))
        sc, pay, r, c = L["wdown"]
        h = h + allreduce(orc.qmatmul(KIND, sc, pay, r, c, act))
    xn = rb(orc.rms_norm_f64(h, f32_of(host.final_norm).astype(np.float64), host.eps))
    sc, pay, r, c = head
    local = torch.from_numpy(orc.qmatmul(KIND, sc, pay, r, c, xn))
    parts = [torch.empty_like(local) for _ in range(tp)]
    dist.all_gather(parts, local)
    return np.concatenate([p.numpy() for p in parts])


def main():
    import torch
    import torch.distributed as dist

    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    host, B, max_seq, ctx, caches, tokens = make_case()
    if mode == "cpu":
        dist.init_process_group("gloo")
        got = np.stack([cpu_rank_decode(host, rank, world, dist, torch, b, int(tokens[b]), caches, ctx[b]) for b in range(B)])
        tol = 1e-9
    else:
        import tang_b200 as tb

        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        dev = tb.QuantComputeDevice(local)
        ids = [tb.Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = tb.Comm(dev, ids[0], rank, world)
        if mode == "gpu_peer":      # the row-parallel sums through the one-shot peer-memory all-reduce instead of NCCL
            comm.enable_peer(B * host.d)
        model = host.to_device(dev, max_seq, B, comm)
        kl = host.n_kv // world
        sl = slice(rank * kl * host.hd, (rank + 1) * kl * host.hd)
        for li in range(host.n_layers):
            kbuf, vbuf, _ = model.kv_buffers(li)
            for buf, src in ((kbuf, caches[li][0]), (vbuf, caches[li][1])):
                a = np.ascontiguousarray(src[:, :, sl])
                dev._check(dev._L.tq_upload(dev._ctx, buf.ptr, a.ctypes.data, a.nbytes))
        logits = dev.alloc(B * host.vocab, tb.F32)
        model.decode(dev.upload(tokens, tb.I32), dev.upload(np.array(ctx, np.int32), tb.I32), B, max(ctx) + 1, logits)
        dev.sync()
        if mode == "gpu_peer":      # and once more from a recorded graph: the sequence number lives on the device
            first = logits.to_vec().copy()
            for li in range(host.n_layers):      # (the step appended K/V rows: put the caches back)
                kbuf, vbuf, _ = model.kv_buffers(li)
                for buf, src in ((kbuf, caches[li][0]), (vbuf, caches[li][1])):
                    a = np.ascontiguousarray(src[:, :, sl])
                    dev._check(dev._L.tq_upload(dev._ctx, buf.ptr, a.ctypes.data, a.nbytes))
            tok_d, pos_d = dev.upload(tokens, tb.I32), dev.upload(np.array(ctx, np.int32), tb.I32)
            dev.begin_capture()
            model.decode(tok_d, pos_d, B, max(ctx) + 1, logits)
            g = dev.end_capture()
            for _ in range(3):
                g.launch()
            dev.sync()
            assert np.array_equal(logits.to_vec(), first), "graph replay of the peer all-reduce differs"
        got = logits.to_vec().reshape(world, B, host.vocab // world).transpose(1, 0, 2).reshape(B, host.vocab)
        tol = 2e-2
    ok = True
    if rank == 0:
        want = oracle_logits(host, B, ctx, caches, tokens)
        err = max(rel_err(got[b], want[b], floor_frac=1.0) for b in range(B))
        print(f"tp={world} mode={mode} max err {err:.3e} (tol {tol})", flush=True)
        ok = err < tol
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
