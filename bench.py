#!/usr/bin/env python
"""Headline benchmark: int4 group-32 dequant-GEMV, K=4096 -> N=14336 (Llama-3-8B FFN up-projection
shape), f16 block scales, bf16 activations, M decode tokens (default 1).

A *step* is one decode pass over LAYERS distinct weight matrices of that shape (default 32, about
1.06 GB, so every launch streams weights that are not in the 126 MB L2), replayed from one CUDA
graph.  `value` is the whole-job HBM stream rate in TB/s: algorithmic bytes (packed nibbles + f16
scales + activations in + bf16 results out) divided by device time.  With N GPUs every rank owns
its own LAYERS matrices (column-parallel shards never exchange data on this path), so scaling is
weak and the aggregate is the sum over ranks.

    python bench.py --gpus 1 --steps 50 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference        # the CPU restatement of tang-infer on the host cores

The JSON line also carries: `e2e` (the same rate through the reference-shaped call q4_matvec with
HOST vectors, copies inside the timed region), `roofline` (dominant kernel vs measured HBM peak),
`cpu_baseline` (the oracle port on a bounded sample), `decode` (Llama-3-8B-shaped decode step,
tokens/s, when --decode is given), `clocks`, `gpu_launches`.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_OUT, K_IN, GROUP = 14336, 4096, 32
METRIC, UNIT = "int4_gemv_hbm_tbps", "TB/s"

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from one ncu
# capture of this command with 8 layers and 1 step (33.10 MB read; the 28 KB of results stay in L2).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 33_104_640


def algorithmic_bytes(m: int) -> int:
    """Bytes one launch has to move: nibbles + f16 scales + bf16 activations in + bf16 results out."""
    return N_OUT * K_IN // 2 + N_OUT * (K_IN // GROUP) * 2 + m * K_IN * 2 + m * N_OUT * 2


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.lines, self.proc, self.thread = gpu_index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [l for (t, l) in self.lines if t0 <= t <= t1 + 0.2] or [l for (_, l) in self.lines]
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in rows:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_matvec_rate(weights, m_x, threads: int, budget_s: float):
    """Times the oracle's q4 matvec (f16 scales) on the host over `weights`, a list of distinct (scales, packed)
    matrices visited in turn (four of them are 132 MB, more than the host's caches): returns (TB/s, reps, seconds)."""
    import oracle

    oracle.build()
    x = m_x.astype(np.float64)
    for sc, pk in weights:
        oracle.qmatmul(oracle.KIND_Q4_F16, sc, pk, N_OUT, K_IN, x, threads)  # warm
    reps, t0 = 0, time.perf_counter()
    while True:
        sc, pk = weights[reps % len(weights)]
        oracle.qmatmul(oracle.KIND_Q4_F16, sc, pk, N_OUT, K_IN, x, threads)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s:
            break
    return algorithmic_bytes(x.shape[0]) * reps / dt / 1e12, reps, dt


def host_weight(seed: int):
    rng = np.random.default_rng(seed)
    packed = rng.integers(0, 256, (N_OUT, K_IN // 2), dtype=np.uint8)
    scales = rng.uniform(0.002, 0.02, (N_OUT, K_IN // GROUP)).astype(np.float16).view(np.uint16)
    return scales, packed


def run_reference(args, rank: int) -> None:
    """The reference's CPU implementation of the path (its restatement in oracle/, since the Rust
    crate cannot be built here) on all host threads.  One step = --ref-sample matvecs."""
    if rank != 0:
        return
    import oracle

    oracle.build()
    threads = oracle.max_threads()
    per_step = args.ref_sample
    weights = [host_weight(43 + i) for i in range(per_step)]      # distinct matrices: the step streams them, as the GPU arm does
    rng = np.random.default_rng(44)
    x = rng.standard_normal((args.m, K_IN)).astype(np.float32).astype(np.float64)
    for _ in range(max(args.warmup, 1)):
        for sc, pk in weights:
            oracle.qmatmul(oracle.KIND_Q4_F16, sc, pk, N_OUT, K_IN, x, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for sc, pk in weights:
            oracle.qmatmul(oracle.KIND_Q4_F16, sc, pk, N_OUT, K_IN, x, threads)
    dt = time.perf_counter() - t0
    value = algorithmic_bytes(args.m) * args.steps * per_step / dt / 1e12
    sample = (f"each timed step = {per_step} distinct matrices ({per_step * algorithmic_bytes(args.m) / 1e6:.0f} MB) of the "
              f"{args.layers} a full step streams, M={args.m}, {threads} threads; the reference itself is single-threaded")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(args) -> dict:
    return {"workload": f"int4-g32/f16-scale dequant-GEMV K={K_IN} N={N_OUT} M={args.m} (the headline int4 GEMM configuration)",
            "layers_per_step": args.layers, "m": args.m,
            "l2": f"{args.layers} distinct weight matrices per step ({args.layers * algorithmic_bytes(args.m) / 1e6:.0f} MB) >> 126 MB L2",
            "parallelism": f"replicated column shards x{args.gpus}, no data-path collective"}


def run_ours(args, rank: int, world: int, local_rank: int) -> None:
    import torch

    import tang_b200 as tb

    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    # The context owns its stream (on a stream of its own the library may let independent matvecs overlap);
    # torch sees the same stream, so CUDA events recorded through torch time the library's launches.
    dev = tb.QuantComputeDevice(local_rank)
    stream = torch.cuda.ExternalStream(dev.stream, device=torch.device("cuda", local_rank))
    L, m = args.layers, args.m

    with torch.cuda.stream(stream):
        gen = torch.Generator(device="cuda").manual_seed(43 + rank)
        packed = torch.randint(0, 256, (L, N_OUT, K_IN // 2), dtype=torch.uint8, device="cuda", generator=gen)
        scales = (torch.rand((L, N_OUT, K_IN // GROUP), device="cuda", generator=gen) * 0.018 + 0.002).half()
        x = torch.randn((m, K_IN), device="cuda", generator=gen).bfloat16()
        y = torch.empty((L, m, N_OUT), dtype=torch.bfloat16, device="cuda")
    stream.synchronize()
    L_ = dev._L
    import ctypes as C

    handles = []
    for i in range(L):
        h = C.c_void_p()
        dev._check(L_.tq_qweight_from_device_arrays(dev._ctx, tb.Q4_F16, C.c_void_p(packed[i].data_ptr()),
                                             C.c_void_p(scales[i].data_ptr()), N_OUT, K_IN, C.byref(h)))
        handles.append(h)

    def one_pass():
        for i in range(L):
            dev._check(L_.tq_qlinear(dev._ctx, handles[i], C.c_void_p(x.data_ptr()), tb.BF16, 0, m,
                                     C.c_void_p(y[i].data_ptr()), tb.BF16, 0, None))

    one_pass()          # eager once: sizes workspaces, sets kernel attributes
    dev.sync()
    dev.begin_capture()
    one_pass()
    graph = dev.end_capture()

    # parity spot check against the oracle on rank 0 (256 output rows of layer 0)
    parity = None
    if rank == 0:
        import oracle

        oracle.build()
        rows = 256
        sc_h = scales[0, :rows].cpu().numpy().view(np.uint16)
        pk_h = packed[0, :rows].cpu().numpy()
        x_h = x.float().cpu().numpy().astype(np.float64)
        want = oracle.qmatmul(oracle.KIND_Q4_F16, sc_h, pk_h, rows, K_IN, x_h, 0)
        got = y[0, :, :rows].float().cpu().numpy().astype(np.float64)
        rms = float(np.sqrt(np.mean(want * want)))
        parity = float(np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-2 * rms)))

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    for _ in range(args.warmup):
        graph.launch()
    barrier()
    launches0 = dev.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.perf_counter()
    with torch.cuda.stream(stream):
        ev0.record(stream)
        for _ in range(args.steps):
            graph.launch()
        ev1.record(stream)
    barrier()
    t_wall1 = time.perf_counter()
    ms = ev0.elapsed_time(ev1)
    gpu_launches = dev.launch_count - launches0

    # ---- end to end: the reference-shaped host call, pinned host vectors, copies inside the timing.  A step queues
    # the L matvecs (upload of x, kernel, result written to its own pinned vector) and waits once for all of them;
    # the second timing waits after every call, as a loop over the reference's q4_matvec does.
    # Every matrix of the step gets its own pinned input vector (a layer's input differs from the next one's).
    xh = torch.empty((L, m, K_IN), dtype=torch.bfloat16).pin_memory()
    xh.copy_(torch.randn((L, m, K_IN), generator=torch.Generator().manual_seed(7 + rank)).bfloat16())
    yh = torch.empty((L, m, N_OUT), dtype=torch.bfloat16).pin_memory()

    x_ptrs = [C.c_void_p(xh[i].data_ptr()) for i in range(L)]      # (a caller has its pointers at hand)
    y_ptrs = [C.c_void_p(yh[i].data_ptr()) for i in range(L)]

    def e2e_pass(call):
        for i in range(L):
            dev._check(call(dev._ctx, handles[i], x_ptrs[i], y_ptrs[i], tb.BF16, m))

    # Timed on the host clock, from the first call to the return of the last wait (the clock an end-to-end caller
    # sees); the CUDA-event time of the same region is kept beside it.
    e2e_steps = max(1, min(args.steps, 20))
    e2e_times, e2e_event_times = [], []
    for call, wait in ((L_.tq_q_matvec_host, False), (L_.tq_q_matvec_host_async, True)):
        e2e_pass(call)
        dev.sync()
        barrier()
        with torch.cuda.stream(stream):
            ev0.record(stream)
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                e2e_pass(call)
                if wait:
                    dev.sync()          # the step's results are read here: one wait per step
            t1 = time.perf_counter()
            ev1.record(stream)
        barrier()
        e2e_times.append((t1 - t0) * 1e3)
        e2e_event_times.append(ev0.elapsed_time(ev1))
    e2e_sync_ms, e2e_async_ms = e2e_times
    # The same step recorded once (tq_graph_begin .. tq_graph_end around the L calls) and replayed: every replay reads
    # the pinned input vectors again and writes the pinned results; per step the host launches one graph and waits once.
    yh_calls = yh.clone()                    # what the call-by-call loop above produced
    dev.begin_capture()
    e2e_pass(L_.tq_q_matvec_host_async)
    e2e_graph = dev.end_capture()
    yh.zero_()
    e2e_graph.launch()
    dev.sync()
    e2e_graph_ok = bool(torch.equal(yh.view(torch.int16), yh_calls.view(torch.int16)))
    barrier()
    with torch.cuda.stream(stream):
        ev0.record(stream)
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_graph.launch()
            dev.sync()
        t1 = time.perf_counter()
        ev1.record(stream)
    barrier()
    e2e_ms = (t1 - t0) * 1e3
    e2e_event_times.append(ev0.elapsed_time(ev1))
    e2e_graph.free()
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None

    t = torch.tensor([ms, e2e_ms, e2e_sync_ms, e2e_async_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, e2e_sync_ms, e2e_async_ms = float(t[0]), float(t[1]), float(t[2]), float(t[3])

    host_w = None   # layer 0 on the host, for the CPU baseline leg
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        host_w = (scales[0].cpu().numpy().view(np.uint16), packed[0].cpu().numpy(), x.float().cpu().numpy())

    # ---- Llama-3-8B-shaped decode step, tensor parallel over the ranks of this job
    decode = None
    comm = None
    if world > 1 and not (args.no_decode and args.no_extras):
        import torch.distributed as dist

        ids = [tb.Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = tb.Comm(dev, ids[0], rank, world)
        comm.enable_peer(64 * 7168)      # the row-parallel sums of a decode step (<= 64 rows of d_model f32) go over peer memory
    if not args.no_decode:
        graph.free()
        graph = None
        for h in handles:
            L_.tq_qweight_free(dev._ctx, h)
        del packed, scales, y
        torch.cuda.empty_cache()
        decode = run_decode(dev, tb, torch, stream, comm, rank, world, args, barrier)

    extras = None
    if not args.no_extras:
        if graph is not None:
            graph.free()
            graph = None
        torch.cuda.empty_cache()
        peak_gbs = measured_peaks()[0]
        extras = run_extras(dev, tb, torch, stream, peak_gbs) if world == 1 else {}
        extras.update(run_sharded_extras(dev, tb, torch, stream, peak_gbs, comm, rank, world, barrier))
    if comm:
        comm.destroy()

    if rank == 0:
        bytes_launch = algorithmic_bytes(m)
        ms_per_step = ms / args.steps
        value = world * L * bytes_launch / (ms_per_step * 1e-3) / 1e12
        e2e_value = world * L * bytes_launch / (e2e_ms / e2e_steps * 1e-3) / 1e12
        peak, peak_kind = measured_peaks()
        achieved = bytes_launch / (ms_per_step * 1e-3 / L) / 1e9
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            import oracle

            threads = oracle.max_threads()
            weights = [(host_w[0], host_w[1])] + [host_weight(900 + i) for i in range(3)]
            v, reps, dt = cpu_matvec_rate(weights, host_w[2], threads, args.cpu_budget)
            # the reference runs this loop on one thread (README: "single-threaded"): that figure beside the all-core one
            v1, reps1, dt1 = cpu_matvec_rate(weights, host_w[2], 1, args.cpu_budget)
            cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                   "sample": f"{reps} matvecs over 4 distinct K={K_IN} N={N_OUT} matrices, M={m}, in {dt:.1f} s",
                   "single_thread": {"value": v1, "unit": UNIT, "cores": 1,
                                     "sample": f"{reps1} matvecs over the same 4 matrices in {dt1:.1f} s"}}
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int4 weights x bf16 activations, f32 accumulate", "data": "synthetic",
            "config": workload_config(args),
            "pct_of_8tbps_nominal": 100.0 * value / world / 8.0,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_kind, "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                         "kernel": "qgemv_sk_kernel<Q4_F16> (persistent GEMV)" if m == 1 else "qgemm_sk_kernel (2..8 rows) / qgemm_mma_kernel / qgemm_umma_kernel", "algorithmic_bytes_per_launch": bytes_launch,
                         "avg_launch_us": ms_per_step * 1e3 / L},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": L * m * K_IN * 2,
                    "d2h_bytes_per_step": L * m * N_OUT * 2, "steps": e2e_steps,
                    "call": "tq_graph_launch of a recorded step (L x tq_q_matvec_host_async: pinned host vectors, one per matrix, read "
                            "again by every replay; results written to pinned host vectors) + one tq_sync per step",
                    "clock": "host wall clock around the calls and their final wait",
                    "graph_result_equals_call_by_call": e2e_graph_ok,
                    "value_cuda_events": world * L * bytes_launch / (e2e_event_times[2] / e2e_steps * 1e-3) / 1e12,
                    "value_async_calls": world * L * bytes_launch / (e2e_async_ms / e2e_steps * 1e-3) / 1e12,
                    "call_async_calls": "tq_q_matvec_host_async per matrix + one tq_sync per step, no graph",
                    "value_wait_per_call": world * L * bytes_launch / (e2e_sync_ms / e2e_steps * 1e-3) / 1e12,
                    "call_wait_per_call": "tq_q_matvec_host (q4_matvec: returns when the result is on the host)"},
            "cpu_baseline": cpu, "gpu_launches": int(gpu_launches), "clocks": clocks,
            "parity_max_rel_err_vs_oracle": parity,
            "decode": None if decode is None else {
                "metric": "llama3_8b_shape_decode_tokens_per_s", "peak_gbs": peak,
                "results": [dict(r, frac_of_hbm_peak=r["gbs_per_gpu"] / peak) for r in decode if "batch" in r],
                "prefill": [r for r in decode if "prefill_tokens" in r]},
            "extras": extras,
        }
        print(json.dumps(out))
    if graph is not None:
        graph.free()
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------
# Llama-3-8B-shaped decode step (the decode configuration): 32 layers, d 4096, 32/8 heads of 128, FFN
# 14336, vocab 128256, int4-g32/f16 weights, bf16 KV cache prefilled to 2048 positions; tensor
# parallel over the ranks of this job.  Random-init weights generated on the device.
# ----------------------------------------------------------------------------------------------
LLAMA = dict(n_layers=32, d=4096, n_heads=32, n_kv=8, hd=128, ffn=14336, vocab=128256, ctx=2048)


def decode_bytes_per_gpu(batch: int, tp: int, n_layers: int) -> int:
    """Algorithmic bytes one GPU streams per step: its weight shards (nibbles + f16 scales) + its KV heads."""
    c = LLAMA
    per_layer_w = (c["d"] * (c["n_heads"] + 2 * c["n_kv"]) * c["hd"] + c["d"] * c["n_heads"] * c["hd"] + 3 * c["d"] * c["ffn"])
    w = n_layers * per_layer_w + c["vocab"] * c["d"]
    wbytes = w // 2 + w // 32 * 2
    kv = n_layers * 2 * batch * (c["ctx"] + 1) * c["n_kv"] * c["hd"] * 2
    return (wbytes + kv) // tp


def build_llama(dev, tb, torch, stream, comm, rank, world, n_layers, max_batch):
    import ctypes as C

    c = LLAMA
    tp = world
    hl, kl, fl, vl = c["n_heads"] // tp, c["n_kv"] // tp, c["ffn"] // tp, c["vocab"] // tp
    d, hd = c["d"], c["hd"]
    cfg = tb.LlamaConfig(n_layers, d, c["n_heads"], c["n_kv"], hd, c["ffn"], c["vocab"], c["ctx"] + 1, max_batch, 1e-5, 500000.0)
    model = tb.LlamaModel(dev, cfg, comm)
    gen = torch.Generator(device="cuda").manual_seed(1000 + rank)
    keep = []

    def qw(rows, cols):
        with torch.cuda.stream(stream):
            pay = torch.randint(0, 256, (rows, cols // 2), dtype=torch.uint8, device="cuda", generator=gen)
            sc = (torch.rand((rows, cols // 32), device="cuda", generator=gen) * 0.018 + 0.002).half()
        stream.synchronize()
        w = dev.qweight_from_device(tb.Q4_F16, pay.data_ptr(), sc.data_ptr(), rows, cols)
        dev.sync()
        return w

    def bf16_vec(n, std=0.02):
        with torch.cuda.stream(stream):
            t = (torch.randn(n, device="cuda", generator=gen) * std).bfloat16()
        stream.synchronize()
        keep.append(t)
        return tb.Buffer(dev, t.data_ptr(), t.numel(), tb.BF16, owns=False)

    for l in range(n_layers):
        # gate/up in the interleaved row order: the SwiGLU becomes the projection's epilogue
        model.set_layer(l, tb.LlamaLayerWeights(qw((hl + 2 * kl) * hd, d), qw(d, hl * hd), dev.interleave_gate_up(qw(2 * fl, d)), qw(d, fl),
                                                bf16_vec(d), bf16_vec(d)))
        kbuf, vbuf, _ = model.kv_buffers(l)
        with torch.cuda.stream(stream):     # prefill the cache with bf16 N(0,1), in slices to bound the temporary
            step = 1 << 26
            for buf in (kbuf, vbuf):
                for off in range(0, buf.n, step):
                    n = min(step, buf.n - off)
                    t = torch.randn(n, device="cuda", generator=gen).bfloat16()
                    dev._check(dev._L.tq_convert(dev._ctx, C.c_void_p(t.data_ptr()), tb.BF16, C.c_void_p(buf.ptr + 2 * off), tb.BF16, n))
                    stream.synchronize()
    model.set_head(bf16_vec(c["vocab"] * d), bf16_vec(d), qw(vl, d))
    model._bench_keep = keep
    return model


def run_decode(dev, tb, torch, stream, comm, rank, world, args, barrier):
    """Times the decode step at each batch size; returns a list of result dicts (rank 0 uses them)."""
    c = LLAMA
    batches = [int(b) for b in args.decode_batches.split(",") if b]
    model = build_llama(dev, tb, torch, stream, comm, rank, world, args.decode_layers, max(batches))
    out = []
    for B in batches:
        with torch.cuda.stream(stream):
            tok = torch.randint(0, c["vocab"], (B,), dtype=torch.int32, device="cuda")
            pos = torch.full((B,), c["ctx"], dtype=torch.int32, device="cuda")
            logits = torch.empty((world, B, c["vocab"] // world), dtype=torch.float32, device="cuda")
        stream.synchronize()
        tbuf = tb.Buffer(dev, tok.data_ptr(), B, tb.I32, owns=False)
        pbuf = tb.Buffer(dev, pos.data_ptr(), B, tb.I32, owns=False)
        lbuf = tb.Buffer(dev, logits.data_ptr(), logits.numel(), tb.F32, owns=False)
        model.decode(tbuf, pbuf, B, c["ctx"] + 1, lbuf)      # eager once (workspaces, attributes, NCCL warm-up)
        dev.sync()
        l0 = dev.launch_count
        dev.begin_capture()
        model.decode(tbuf, pbuf, B, c["ctx"] + 1, lbuf)
        graph = dev.end_capture()
        for _ in range(max(args.warmup, 3)):
            graph.launch()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        steps = args.decode_steps
        with torch.cuda.stream(stream):
            ev0.record(stream)
            for _ in range(steps):
                graph.launch()
            ev1.record(stream)
        barrier()
        ms = ev0.elapsed_time(ev1) / steps
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        if world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
        finite = bool(torch.isfinite(logits).all().item())
        graph.free()
        byt = decode_bytes_per_gpu(B, world, args.decode_layers)
        out.append({"batch": B, "tp": world, "layers": args.decode_layers, "ms_per_step": ms, "tokens_per_s": B / (ms * 1e-3),
                    "bytes_per_gpu": byt, "gbs_per_gpu": byt / (ms * 1e-3) / 1e9, "logits_finite": finite,
                    "kernels_per_step": int((dev.launch_count - l0) // (steps + max(args.warmup, 3)))})
    # prompt processing with the same model: one sequence, a 2048-token chunk from an empty cache
    q_len = min(2048, c["ctx"])
    with torch.cuda.stream(stream):
        ptok = torch.randint(0, c["vocab"], (q_len,), dtype=torch.int32, device="cuda")
        start0 = torch.zeros((1,), dtype=torch.int32, device="cuda")
        plog = torch.empty((world, 1, c["vocab"] // world), dtype=torch.float32, device="cuda")
    stream.synchronize()
    mk = lambda t, dt: tb.Buffer(dev, t.data_ptr(), t.numel(), dt, owns=False)
    model.prefill(mk(ptok, tb.I32), mk(start0, tb.I32), 1, q_len, mk(plog, tb.F32))      # sizes the workspaces
    dev.sync()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 3
    with torch.cuda.stream(stream):
        ev0.record(stream)
        for _ in range(reps):
            model.prefill(mk(ptok, tb.I32), mk(start0, tb.I32), 1, q_len, mk(plog, tb.F32))
        ev1.record(stream)
    barrier()
    pms = ev0.elapsed_time(ev1) / reps
    t = torch.tensor([pms], dtype=torch.float64, device="cuda")
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    pms = float(t[0])
    w_params = args.decode_layers * (c["d"] * (c["n_heads"] + 2 * c["n_kv"]) * c["hd"] + c["d"] * c["n_heads"] * c["hd"] + 3 * c["d"] * c["ffn"])
    out.append({"prefill_tokens": q_len, "tp": world, "layers": args.decode_layers, "ms": pms, "tokens_per_s": q_len / (pms * 1e-3),
                "tflops_per_gpu": 2.0 * q_len * w_params / world / (pms * 1e-3) / 1e12, "logits_finite": bool(torch.isfinite(plog).all().item())})
    model.destroy()
    return out


# ----------------------------------------------------------------------------------------------
# The other benchmark configurations, timed briefly at N=1 and reported under "extras": the M sweep of
# the int4 GEMM, the DeepSeek-V2-Lite-shaped MoE layer and the DeepSeek-V3-shaped MLA decode
# attention.  Seeded synthetic inputs generated on the device.
# ----------------------------------------------------------------------------------------------
def _time_ms(torch, stream, dev, fn, reps, warm=2):
    for _ in range(warm):
        fn()
    dev.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(reps):
            fn()
        e1.record(stream)
    dev.sync()
    return e0.elapsed_time(e1) / reps


def run_extras(dev, tb, torch, stream, peak_gbs):
    import ctypes as C

    L_ = dev._L
    gen = torch.Generator(device="cuda").manual_seed(77)
    out = {}

    def q4(rows, cols):
        with torch.cuda.stream(stream):
            pay = torch.randint(0, 256, (rows, cols // 2), dtype=torch.uint8, device="cuda", generator=gen)
            sc = (torch.rand((rows, cols // 32), device="cuda", generator=gen) * 0.018 + 0.002).half()
        stream.synchronize()
        w = dev.qweight_from_device(tb.Q4_F16, pay.data_ptr(), sc.data_ptr(), rows, cols)
        dev.sync()
        return w

    def i8(rows, cols):
        with torch.cuda.stream(stream):
            pay = torch.randint(-127, 128, (rows, cols), dtype=torch.int8, device="cuda", generator=gen)
            sc = torch.rand(rows, device="cuda", generator=gen) * 0.009 + 0.001
        stream.synchronize()
        w = dev.qweight_from_device(tb.I8_ROW, pay.data_ptr(), sc.data_ptr(), rows, cols)
        dev.sync()
        return w

    def bf16(shape, std=1.0):
        with torch.cuda.stream(stream):
            t = (torch.randn(shape, device="cuda", generator=gen) * std).bfloat16()
        stream.synchronize()
        return t

    # ---- the int8 GEMV of the CPU-runnable configuration: [4096, 4096] int8, one f32 scale per output row (and the same
    # integers as tang-infer's native Q8 blocks, one f32 scale per 32 weights), f32 activations, f32 results;
    # 16 distinct matrices per graph (268 MB > L2)
    def q8_blocks(rows, cols):
        with torch.cuda.stream(stream):
            pay = torch.randint(-127, 128, (rows, cols), dtype=torch.int8, device="cuda", generator=gen)
            sc = (torch.rand((rows, cols // 32), device="cuda", generator=gen) * 0.009 + 0.001)
        stream.synchronize()
        w = dev.qweight_from_device(tb.Q8_F32, pay.data_ptr(), sc.data_ptr(), rows, cols)
        dev.sync()
        return w

    int8 = []
    n8 = 16
    for name, make, byt in (("int8 per-row scale", i8, 4096 * 4096 + 4096 * 4 + 4096 * 4 + 4096 * 4),
                            ("Q8 blocks (f32 scale per 32)", q8_blocks, 4096 * 4096 + 4096 * 128 * 4 + 4096 * 4 + 4096 * 4)):
        w8 = [make(4096, 4096) for _ in range(n8)]
        with torch.cuda.stream(stream):
            x32 = torch.randn((1, 4096), device="cuda", generator=gen)
        xb16 = x32.bfloat16()
        y32 = torch.empty((n8, 1, 4096), dtype=torch.float32, device="cuda")
        stream.synchronize()
        row = {"layout": name, "algorithmic_bytes": byt}
        for tag, xt, xdt in (("f32_x", x32, tb.F32), ("bf16_x", xb16, tb.BF16)):
            def one8():
                for i, w in enumerate(w8):
                    dev._check(L_.tq_qlinear(dev._ctx, C.c_void_p(w.handle), C.c_void_p(xt.data_ptr()), xdt, 0, 1,
                                             C.c_void_p(y32[i].data_ptr()), tb.F32, 0, None))
            one8()
            dev.sync()
            dev.begin_capture()
            one8()
            g = dev.end_capture()
            us = _time_ms(torch, stream, dev, g.launch, 10, 3) * 1e3 / n8
            g.free()
            row[tag] = {"us_per_launch": us, "gbs": byt / us / 1e3, "frac_of_hbm_peak": byt / us / 1e3 / peak_gbs}
        # the same weights against many rows (the tcgen05 GEMM): bf16 activations, f32 results
        for m in (64, 2048):
            xm = bf16((m, 4096))
            ym = torch.empty((n8, m, 4096), dtype=torch.float32, device="cuda")
            stream.synchronize()

            def many8():
                for i, w in enumerate(w8):
                    dev._check(L_.tq_qlinear(dev._ctx, C.c_void_p(w.handle), C.c_void_p(xm.data_ptr()), tb.BF16, 0, m,
                                             C.c_void_p(ym[i].data_ptr()), tb.F32, 0, None))
            many8()
            dev.sync()
            dev.begin_capture()
            many8()
            g = dev.end_capture()
            us = _time_ms(torch, stream, dev, g.launch, 10, 3) * 1e3 / n8
            g.free()
            row["m%d_bf16_x" % m] = {"us_per_launch": us, "tflops": 2.0 * m * 4096 * 4096 / us / 1e6}
            del xm, ym
        int8.append(row)
        for w in w8:
            w.free()
    out["int8_gemv_4096"] = int8

    # ---- the reference's one published number for this path: quantize/q8_matvec_576x576, 207 992 ns on an Apple M4 Max,
    # one thread (crates/tang-bench/benches/cpu_training.rs:267-275).  Here: the oracle port on one host thread, the
    # reference-shaped host call (f64 vectors in and out, waits), and the kernel alone from a graph.
    import oracle

    oracle.build()
    rng = np.random.default_rng(576)
    wf = (rng.standard_normal((576, 576)) * 0.05).astype(np.float32)
    s8, v8 = oracle.quantize_matrix_q8(wf, 576, 576)
    xq = rng.standard_normal(576)
    t0 = time.perf_counter()
    n_cpu = 200
    for _ in range(n_cpu):
        oracle.q8_matvec(s8, v8, 576, 576, xq, 1)
    cpu_ns = (time.perf_counter() - t0) / n_cpu * 1e9
    w576 = dev.upload_q8(tb.QuantizedQ8(s8.reshape(-1), v8.reshape(-1), (576, 576)))
    dev.q8_matvec(w576, xq)
    t0 = time.perf_counter()
    for _ in range(200):
        dev.q8_matvec(w576, xq)
    host_call_ns = (time.perf_counter() - t0) / 200 * 1e9
    with torch.cuda.stream(stream):
        x576 = torch.randn((1, 576), device="cuda", generator=gen)
    y576 = torch.empty((1, 576), dtype=torch.float32, device="cuda")
    stream.synchronize()

    def one576():
        dev._check(L_.tq_qlinear(dev._ctx, C.c_void_p(w576.handle), C.c_void_p(x576.data_ptr()), tb.F32, 0, 1,
                                 C.c_void_p(y576.data_ptr()), tb.F32, 0, None))
    one576()
    dev.sync()
    dev.begin_capture()
    for _ in range(20):
        one576()
    g = dev.end_capture()
    kern_ns = _time_ms(torch, stream, dev, g.launch, 10, 3) * 1e6 / 20
    g.free()
    out["q8_matvec_576x576"] = {"reference_published_ns_m4max_1thread": 207992, "oracle_port_1thread_ns": cpu_ns,
                                "host_call_f64_ns": host_call_ns, "device_launches_from_graph_ns": kern_ns}

    # ---- int4 GEMM: M sweep over 16 distinct matrices (528 MB > L2), bf16 results, one CUDA graph per M
    n_mat = 16
    ws = [q4(N_OUT, K_IN) for _ in range(n_mat)]
    sweep = []
    for m in (1, 8, 32, 64, 512, 2048):
        x = bf16((m, K_IN))
        y = torch.empty((n_mat, m, N_OUT), dtype=torch.bfloat16, device="cuda")   # one result per matrix, as in the headline

        def one():
            for i, w in enumerate(ws):
                dev._check(L_.tq_qlinear(dev._ctx, C.c_void_p(w.handle), C.c_void_p(x.data_ptr()), tb.BF16, 0, m,
                                         C.c_void_p(y[i].data_ptr()), tb.BF16, 0, None))
        one()
        dev.sync()
        dev.begin_capture()
        one()
        g = dev.end_capture()
        us = _time_ms(torch, stream, dev, g.launch, 10, 3) * 1e3 / n_mat
        g.free()
        byt, fl = algorithmic_bytes(m), 2.0 * m * N_OUT * K_IN
        sweep.append({"m": m, "us_per_launch": us, "gbs": byt / us / 1e3, "tflops": fl / us / 1e6,
                      "frac_of_hbm_peak": byt / us / 1e3 / peak_gbs})
    out["int4_gemm_m_sweep"] = sweep
    for w in ws:
        w.free()
    del ws
    torch.cuda.empty_cache()

    # ---- prefill attention: one sequence, Llama-3-8B heads (32 query / 8 KV heads of 128), causal chunk of q_len positions
    pre = []
    for q_len in (512, 2048):
        nh, nkv, hd = 32, 8, 128
        q = bf16((1, q_len, nh * hd))
        kc, vc = bf16((1, q_len, nkv * hd)), bf16((1, q_len, nkv * hd))
        o = torch.empty((1, q_len, nh * hd), dtype=torch.bfloat16, device="cuda")
        st0 = dev.upload(np.zeros(1, np.int32), tb.I32)

        def fn():
            dev._check(L_.tq_gqa_prefill(dev._ctx, C.c_void_p(q.data_ptr()), C.c_void_p(kc.data_ptr()), C.c_void_p(vc.data_ptr()),
                                         C.c_void_p(st0.ptr), 1, q_len, nh, nkv, hd, q_len * nkv * hd, C.c_void_p(o.data_ptr()), tb.BF16))
        ms = _time_ms(torch, stream, dev, fn, 10, 3)
        flops = 4.0 * nh * hd * q_len * (q_len + 1) / 2          # QK^T and PV over the causal half
        pre.append({"q_len": q_len, "us": ms * 1e3, "tflops": flops / ms / 1e9})
    out["gqa_prefill_llama_heads"] = pre
    return out


def run_sharded_extras(dev, tb, torch, stream, peak_gbs, comm, rank, world, barrier):
    """The MoE layer with its experts over the ranks and the MLA layer with its heads over the ranks; at N = 1 the
    same calls without a communicator.  Times are the max over the ranks."""
    import ctypes as C

    L_ = dev._L
    gen = torch.Generator(device="cuda").manual_seed(77)      # same seed on every rank: replicated tensors are equal
    out = {}

    def q4(rows, cols):
        with torch.cuda.stream(stream):
            pay = torch.randint(0, 256, (rows, cols // 2), dtype=torch.uint8, device="cuda", generator=gen)
            sc = (torch.rand((rows, cols // 32), device="cuda", generator=gen) * 0.018 + 0.002).half()
        stream.synchronize()
        w = dev.qweight_from_device(tb.Q4_F16, pay.data_ptr(), sc.data_ptr(), rows, cols)
        dev.sync()
        return w

    def i8(rows, cols):
        with torch.cuda.stream(stream):
            pay = torch.randint(-127, 128, (rows, cols), dtype=torch.int8, device="cuda", generator=gen)
            sc = torch.rand(rows, device="cuda", generator=gen) * 0.009 + 0.001
        stream.synchronize()
        w = dev.qweight_from_device(tb.I8_ROW, pay.data_ptr(), sc.data_ptr(), rows, cols)
        dev.sync()
        return w

    def bf16(shape, std=1.0):
        with torch.cuda.stream(stream):
            t = (torch.randn(shape, device="cuda", generator=gen) * std).bfloat16()
        stream.synchronize()
        return t

    def timed(fn, reps):
        fn()
        dev.sync()
        dev.begin_capture()
        fn()
        g = dev.end_capture()
        barrier()
        ms = _time_ms(torch, stream, dev, g.launch, reps)
        g.free()
        if world > 1:
            import torch.distributed as dist

            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        return ms

    # ---- MoE layer, d 2048, 64 routed + 2 shared experts of width 1408, top-6; experts over the ranks
    d, ffn, E, k, nsh = 2048, 1408, 64, 6, 2
    n_local = E // world
    wg = bf16((E, d), 0.02)
    layer = tb.MoeLayer(dev, tb.MoeConfig(d, ffn, E, k, nsh, 0, rank, world), tb.Buffer(dev, wg.data_ptr(), wg.numel(), tb.BF16, owns=False),
                        q4(n_local * 2 * ffn, d), q4(n_local * d, ffn), [q4(2 * ffn, d) for _ in range(nsh)], [q4(d, ffn) for _ in range(nsh)])
    per_expert = 3 * (ffn * d // 2 + ffn * d // 32 * 2)
    moe = []
    for T in (1, 64, 256, 4096):
        h = bf16((T, d))                                      # the same tokens on every rank
        hb = tb.Buffer(dev, h.data_ptr(), h.numel(), tb.BF16, owns=False)
        o, idx, _w = layer.forward(hb, T, comm=comm, want_routing=True)
        dev.sync()
        distinct = int(len(set(idx.to_vec().tolist())))
        ob = dev.alloc(T * d, tb.F32)
        reps = 10 if T <= 256 else 3
        ms = timed(lambda: layer.forward(hb, T, out=ob, comm=comm), reps)
        byt = (distinct + nsh) * per_expert
        row = {"tokens": T, "us": ms * 1e3, "distinct_routed_experts": distinct, "weight_bytes_touched": byt,
               "gbs": byt / ms / 1e6, "tflops": 2.0 * T * (k + nsh) * 3 * ffn * d / ms / 1e9,
               "form": "one GPU" if world == 1 else "tokens replicated, experts over the ranks, all-reduce of the outputs"}
        if world > 1 and T % world == 0:
            # tokens sharded over the ranks: all-to-all dispatch to the experts' owners and all-to-all combine back
            tl = T // world
            hl = tb.Buffer(dev, h[rank * tl:(rank + 1) * tl].data_ptr(), tl * d, tb.BF16, owns=False)
            ol = dev.alloc(tl * d, tb.F32)
            ms2 = timed(lambda: layer.forward_dispatch(hl, tl, comm=comm, out=ol), reps)
            row["dispatch"] = {"us": ms2 * 1e3, "tokens_per_rank": tl, "tflops": 2.0 * T * (k + nsh) * 3 * ffn * d / ms2 / 1e9,
                               "form": "tokens over the ranks, all-to-all dispatch and combine, peer blocks padded to the worst case "
                                       "(fixed size: replayed from a graph)"}
            if tl * k >= 256:
                # outside a graph the call exchanges the row counts first and sends true sizes (one host round trip inside)
                barrier()
                ms3 = _time_ms(torch, stream, dev, lambda: layer.forward_dispatch(hl, tl, comm=comm, out=ol), reps)
                if world > 1:
                    import torch.distributed as dist

                    t3 = torch.tensor([ms3], dtype=torch.float64, device="cuda")
                    dist.all_reduce(t3, op=dist.ReduceOp.MAX)
                    ms3 = float(t3[0])
                row["dispatch_counts_first"] = {"us": ms3 * 1e3, "tflops": 2.0 * T * (k + nsh) * 3 * ffn * d / ms3 / 1e9,
                                                "form": "the same call made eagerly: counts exchanged first, rows sent with their true sizes"}
        moe.append(row)
    out["moe_dsv2_lite_layer"] = moe
    layer.destroy()
    torch.cuda.empty_cache()

    # ---- MLA decode, 128 heads over the ranks, latent 512 + rope 64, int8 per-row weights.  The attention core
    # (absorb W_UK, attend over the latent cache, un-absorb W_UV) and the whole layer with q_a [1536, d], q_b and the
    # row-parallel W_O at d_model 7168 (an assumption: the configuration names no hidden size).
    H, NOPE, VD, CL, RP, QL, DM = 128 // world, 128, 128, 512, 64, 1536, 7168
    wq, wu = i8(H * CL, NOPE), i8(H * VD, CL)
    max_pos = 32768 + 1
    gain = bf16((QL,), 0.03)
    mlayer = tb.MlaLayer(dev, tb.MlaConfig(DM, H, QL, CL, NOPE, RP, VD, 64, max_pos, 1e-6), i8(QL, DM),
                         tb.Buffer(dev, gain.data_ptr(), QL, tb.BF16, owns=False), i8(H * (NOPE + RP), QL), wq, wu, i8(DM, H * VD))
    mla = []
    for ctx, B in ((4096, 1), (16384, 16), (32768, 64)):
        cache = torch.empty((B, ctx, CL + RP), dtype=torch.bfloat16, device="cuda")
        with torch.cuda.stream(stream):
            for b in range(B):
                cache[b].copy_(torch.randn((ctx, CL + RP), device="cuda", generator=gen))
        stream.synchronize()
        qn, qr = bf16((B, H, NOPE)), bf16((B, H, RP))
        hid = bf16((B, DM))
        lens = dev.upload(np.full(B, ctx, np.int32), tb.I32)
        q_full, o_lat, o = dev.alloc(B * H * (CL + RP), tb.BF16), dev.alloc(B * H * CL, tb.BF16), dev.alloc(B * H * VD, tb.F32)
        lo = dev.alloc(B * DM, tb.F32)
        cb = tb.Buffer(dev, cache.data_ptr(), cache.numel(), tb.BF16, owns=False)
        hb = tb.Buffer(dev, hid.data_ptr(), hid.numel(), tb.BF16, owns=False)

        def core():   # absorb W_UK into q, attend over the latent cache, un-absorb with W_UV
            dev._check(L_.tq_mla_absorb_q(dev._ctx, C.c_void_p(wq.handle), C.c_void_p(qn.data_ptr()), C.c_void_p(qr.data_ptr()),
                                          B, H, NOPE, C.c_void_p(q_full.ptr)))
            dev._check(L_.tq_mla_decode(dev._ctx, C.c_void_p(q_full.ptr), C.c_void_p(cache.data_ptr()), C.c_void_p(lens.ptr), B, H,
                                        CL, RP, ctx * (CL + RP), ctx, 1.0 / (NOPE + RP) ** 0.5, C.c_void_p(o_lat.ptr)))
            dev._check(L_.tq_mla_unabsorb(dev._ctx, C.c_void_p(wu.handle), C.c_void_p(o_lat.ptr), B, H, VD, C.c_void_p(o.ptr), tb.F32))
        ms = timed(core, 5)
        ms_layer = timed(lambda: mlayer.decode(hb, cb, lens, B, ctx * (CL + RP), ctx, comm=comm, out=lo), 5)
        byt = B * ctx * (CL + RP) * 2                       # the cache is replicated: every rank streams all of it
        mla.append({"ctx": ctx, "batch": B, "heads_per_gpu": H, "us": ms * 1e3, "layer_us": ms_layer * 1e3, "cache_bytes": byt,
                    "gbs_per_gpu": byt / ms / 1e6, "tflops": B * ctx * H * world * 2176.0 / ms / 1e9,
                    "frac_of_hbm_peak": byt / ms / 1e6 / peak_gbs})
        del cache
        torch.cuda.empty_cache()
    out["mla_dsv3_decode"] = mla
    mlayer.destroy()
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=1, help="decode tokens per GEMV (1..64)")
    ap.add_argument("--layers", type=int, default=32, help="distinct weight matrices per step")
    ap.add_argument("--cpu-budget", type=float, default=8.0, help="seconds of CPU baseline timing")
    ap.add_argument("--ref-sample", type=int, default=4, help="matvecs per step of the reference arm")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the Llama-3-8B-shaped decode step")
    ap.add_argument("--no-extras", action="store_true", help="skip the M sweep / MoE / MLA timings (N=1 only)")
    ap.add_argument("--decode-batches", default="1,16,64")
    ap.add_argument("--decode-layers", type=int, default=32)
    ap.add_argument("--decode-steps", type=int, default=10)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        sys.exit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
