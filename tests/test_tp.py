"""Tensor-parallel decode: sharding + collectives against the unsharded oracle.

CPU: two gloo ranks run the oracle's arithmetic over HostLlama.shard's shards with the same
all-reduce / all-gather pattern as the device path (exercises the N>1 host logic without a GPU).
GPU: the same case through libtangq and NCCL on two GPUs (skipped when fewer are visible)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(mode, n, port, worker="tp_worker.py"):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, worker), mode]
    env = dict(os.environ)
    env.setdefault("OMP_NUM_THREADS", "2")
    if mode.startswith("gpu"):
        env["NCCL_NVLS_ENABLE"] = "0"
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)


def test_tp2_sharding_with_gloo_on_cpu():
    r = _run("cpu", 2, 29631)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "max err" in r.stdout


@pytest.mark.gpu
def test_tp2_decode_on_two_gpus():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = _run("gpu", 2, 29632)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.gpu
def test_tp2_decode_with_peer_memory_allreduce_on_two_gpus():
    """The same decode step with the row-parallel sums going through the one-shot peer-memory all-reduce
    (plain peer stores + bounded flag waits), eagerly and replayed from a graph."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = _run("gpu_peer", 2, 29635)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def test_ep2_token_dispatch_protocol_with_gloo_on_cpu():
    """Expert parallelism with sharded tokens: route, dispatch to the experts' owners, combine back; numpy + the
    oracle's expert arithmetic over two gloo ranks must reproduce the unsharded oracle exactly."""
    r = _run("cpu", 2, 29633, "ep_worker.py")
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "err" in r.stdout


@pytest.mark.gpu
def test_ep2_token_dispatch_on_two_gpus():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = _run("gpu", 2, 29634, "ep_worker.py")
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.gpu
def test_ep2_counts_first_dispatch_on_two_gpus():
    """A batch large enough for the counts-first exchange (row counts to the owners, then rows, ids and results with
    their true sizes): same result as the unsharded oracle, and the padded rows of the ragged shard change nothing."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = _run("gpu_big", 2, 29636, "ep_worker.py")
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
