"""Data-parallel path: world_size-2 gloo ranks on CPU (sharding + the one exchange per window),
and -- where two GPUs are visible -- the library's own NCCL all-reduce on one GPU per rank."""
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


def _launch(mode, nproc):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "dp_worker.py"), mode]
    env = dict(os.environ, OMP_NUM_THREADS="2")
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
def test_two_gpus_reproduce_one_gpu(g):
    if g.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = _launch("gpu", 2)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
