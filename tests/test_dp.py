"""Data-parallel path: world_size-2 gloo ranks on CPU (sharding + the one exchange per window),
and -- where two GPUs are visible -- the library's own exchange on one GPU per rank, both over peer
memory and through NCCL."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _launch(mode, nproc, **extra_env):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "dp_worker.py"), mode]
    env = dict(os.environ, OMP_NUM_THREADS="2", **extra_env)
    return subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)


def test_shard_range_partitions_rows(g):
    for rows, world in [(8192, 8), (37, 2), (10, 3), (5, 8), (0, 4)]:
        seen = []
        for r in range(world):
            f, c = g.shard_range(rows, r, world)
            seen.extend(range(f, f + c))
        assert seen == list(range(rows))
        counts = [g.shard_range(rows, r, world)[1] for r in range(world)]
        assert max(counts) - min(counts) <= 1


def test_two_gloo_ranks_reproduce_one_rank(oracle):
    r = _launch("cpu", 2)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.gpu
@pytest.mark.parametrize("mode,push", [("gpu", "1"), ("gpu", "0"), ("gpu_tc", "1"), ("gpu_tc", "0"), ("gpu_tc_wide", "1"),
                                       ("gpu_tc_wide", "0")])
def test_two_gpus_reproduce_one_gpu(g, mode, push):
    """push=1: the gradient exchange over peer memory (required, no silent NCCL fallback);
    push=0: one NCCL all-reduce per layer."""
    if g.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = _launch(mode, 2, GLADES_DP_PUSH=push)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.gpu
@pytest.mark.parametrize("store", ["1", "2"])
def test_two_gpus_other_ways_of_moving_the_gradient_bands(g, store):
    """GLADES_DP_STORE: the gradient product writes locally and its bands reach their owners by a copy kernel (1)
    or by the copy engines (2) on the layer's exchange stream, instead of from the product's epilogue."""
    if g.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = _launch("gpu_tc_wide", 2, GLADES_DP_PUSH="1", GLADES_DP_STORE=store)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.gpu
@pytest.mark.parametrize("ranks", [4, 8])
def test_more_gpus_reproduce_one_gpu(g, ranks):
    """The exchange over peer memory with 4 and 8 ranks (bands of 4 and 2 row tiles, the rotated walk over the
    owners' bands, four windows queued back to back) against the one-GPU run."""
    if g.device_count() < ranks:
        pytest.skip("needs %d GPUs" % ranks)
    r = _launch("gpu_tc_wide", ranks, GLADES_DP_PUSH="1")
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
