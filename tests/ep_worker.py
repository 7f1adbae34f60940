"""Worker of the expert-parallel MoE tests with token dispatch: one process per rank, tokens sharded.

    torchrun --nproc-per-node N tests/ep_worker.py gpu     # NCCL, tq_moe_ffn_dispatch on N GPUs (gpu_big: counts-first exchange)
    torchrun --nproc-per-node N tests/ep_worker.py cpu     # gloo, the same protocol in numpy + the oracle

Protocol (both modes): every rank routes its own tokens; each (token, choice) row goes to the block of the
send buffer addressed to the expert's owner (padded to the worst case T*k rows per peer, -1 = padding);
all-to-all; owners run their experts on what arrived; all-to-all back; the token's rank weights and sums
its k results and adds the shared experts.  Every rank then compares its tokens with the unsharded oracle.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

import oracle as orc  # noqa: E402
from moe_util import KIND, HostMoe  # noqa: E402
from util import bf16_round, rel_err  # noqa: E402


def make_case(world, big=False):
    host = HostMoe(np.random.default_rng(21), d=256, ffn=256, n_experts=8, top_k=2, n_shared=1)
    rng = np.random.default_rng(22)
    # ragged on purpose; the large case has T * top_k >= 256 rows per rank, from where tq_moe_ffn_dispatch exchanges
    # the row counts first and sends rows, ids and results with their true sizes
    T_loc = ([150, 131, 140, 129] if big else [5, 3, 4, 6])[:world]
    hb, hf = bf16_round(rng.standard_normal((sum(T_loc), host.d)).astype(np.float32))
    return host, T_loc, hb, hf


def exchange(dist, torch, blocks, rank, world):
    """blocks[p] goes to rank p; returns what every rank sent to this one.  gloo has no all-to-all, so the
    whole send buffers are gathered and the column addressed to this rank is kept."""
    t = torch.from_numpy(np.ascontiguousarray(np.stack(blocks)))
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t)
    return [p.numpy()[rank] for p in parts]


def cpu_rank(host, rank, world, dist, torch, h_loc):
    T, k, E, nl = h_loc.shape[0], host.k, host.E, host.E // world
    qw = lambda w: orc.qweight(KIND, w[0], w[1], w[2], w[3])
    cap = max_cap = None
    # capacity must be the same on every rank for a fixed-size exchange: the largest T*k
    caps = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(caps, torch.tensor([T * k], dtype=torch.int64))
    cap = int(max(c.item() for c in caps))
    idxs, ws = [], []
    send_x = [np.zeros((cap, host.d)) for _ in range(world)]
    send_e = [np.full(cap, -1, np.int64) for _ in range(world)]
    fill = [0] * world
    place = {}
    for t in range(T):
        idx, w, _ = orc.router_f64(h_loc[t].astype(np.float64), host.wg.astype(np.float64), E, k, host.renorm)
        idxs.append(idx)
        ws.append(w)
        for s, e in enumerate(idx):
            owner = int(e) // nl
            send_x[owner][fill[owner]] = h_loc[t]
            send_e[owner][fill[owner]] = int(e) - owner * nl
            place[(t, s)] = (owner, fill[owner])
            fill[owner] += 1
    recv_x = exchange(dist, torch, send_x, rank, world)
    recv_e = exchange(dist, torch, send_e, rank, world)
    back = []
    for src in range(world):
        y = np.zeros((cap, host.d))
        for j in range(cap):
            e = int(recv_e[src][j])
            if e >= 0:
                ex = host.experts[rank * nl + e]
                y[j] = orc.expert_ffn_f64(qw(ex["gate"]), qw(ex["up"]), qw(ex["down"]), recv_x[src][j])
        back.append(y)
    ret = exchange(dist, torch, back, rank, world)
    out = np.zeros((T, host.d))
    for t in range(T):
        for s in range(k):
            owner, pos = place[(t, s)]
            out[t] += ws[t][s] * ret[owner][pos]
        for sx in range(host.n_shared):
            ex = host.experts[E + sx]
            out[t] += orc.expert_ffn_f64(qw(ex["gate"]), qw(ex["up"]), qw(ex["down"]), h_loc[t].astype(np.float64))
    return out


def main():
    import torch
    import torch.distributed as dist

    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    host, T_loc, hb, hf = make_case(world, big=mode == "gpu_big")
    lo = sum(T_loc[:rank])
    h_bits, h_f32 = hb[lo:lo + T_loc[rank]], hf[lo:lo + T_loc[rank]]
    want, idx_o, _, _ = host.oracle(orc, h_f32)
    if mode == "cpu":
        dist.init_process_group("gloo")
        got = cpu_rank(host, rank, world, dist, torch, h_f32)
        err, tol = float(np.max(np.abs(got - want))), 1e-12
    else:
        import tang_b200 as tb

        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        dev = tb.QuantComputeDevice(local)
        ids = [tb.Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = tb.Comm(dev, ids[0], rank, world)
        # the fixed-size exchange needs the same rows-per-peer capacity everywhere: pad every rank to the largest shard
        T_max = max(T_loc)
        pad = np.zeros((T_max, host.d), np.uint16)
        pad[:T_loc[rank]] = h_bits
        layer = host.to_device(dev, ep_rank=rank, ep_size=world)
        out, idx, _w = layer.forward_dispatch(dev.upload(pad, tb.BF16), T_max, comm, want_routing=True)
        dev.sync()
        got = out.to_vec().reshape(T_max, host.d)[:T_loc[rank]]
        assert np.array_equal(idx.to_vec().reshape(T_max, host.k)[:T_loc[rank]], idx_o)
        err, tol = rel_err(got, want, floor_frac=1.0), 1e-3
        layer.destroy()
        comm.destroy()
    print(f"ep={world} rank={rank} mode={mode} err {err:.3e} (tol {tol})", flush=True)
    flag = torch.tensor([1 if err < tol else 0])
    if mode != "cpu":
        flag = flag.cuda()
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
