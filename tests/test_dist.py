"""Multi-rank path: sharding helpers, a world-size-2 gloo run on CPU (host
logic), and on a box with at least two GPUs the NCCL all-reduce of the C ABI."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
WORKER = Path(__file__).resolve().parent / "dist_worker.py"


def test_shard_range_partitions_exactly():
    from metaphor_b200.dist import shard_range
    for n in (0, 1, 7, 64, 65536, 1000003):
        for world in (1, 2, 3, 8):
            parts = [shard_range(n, world, r) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == n
            assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in parts]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(10, 2, 2)


def free_port() -> int:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(mode, nproc, port=None):
    port = port or free_port()
    env = dict(os.environ)
    env["PYTHONPATH"] = str(ROOT) + os.pathsep + env.get("PYTHONPATH", "")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(WORKER), mode]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)


def test_two_gloo_ranks_reproduce_the_full_batch_step(orc):
    res = run_ranks("cpu", 2)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert res.stdout.count(" ok") == 2


@pytest.mark.gpu
def test_nccl_all_reduce_and_data_parallel_step_on_two_gpus(mp, orc):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = run_ranks("gpu", 2)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert res.stdout.count(" ok") == 2


def test_a_rank_whose_communicator_creation_fails_is_noticed_by_all(mp):
    res = run_ranks("fail_init", 2)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert res.stdout.count(" ok") == 2


def test_a_rank_that_leaves_between_steps_is_noticed_without_hanging(mp):
    res = run_ranks("leave", 2)
    assert res.stdout.count(" ok") == 2, res.stdout[-2000:] + res.stderr[-4000:]
