"""Two-GPU checks of the sharded path (skipped on a single-GPU box): ShardedQuantLinear.forward
under torchrun with both gather implementations against the unsharded oracle, and bench.py with
the library's peer-store all-gather, which bench.py itself verifies against NCCL's result."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("gather", ["nccl", "nvlink"])
def test_two_rank_bench_runs_and_gathers_correctly(gather):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29571" if gather == "nccl" else "29572", os.path.join(ROOT, "bench.py"),
           "--gpus", "2", "--steps", "3", "--warmup", "3", "--watchdog", "120", "--gather", gather]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-800:]
    line = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert line["n_gpus"] == 2 and line["value"] > 0
    assert ("NVLink" in line["config"]["sharding"]) == (gather == "nvlink")


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_linear_forward_matches_the_unsharded_oracle():
    """tests/sharded_worker.py on 2 ranks: gather = nccl and nvlink, M in {1, 4, 16}, both output
    layouts, three consecutive calls each; every rank compares the gathered [M, N] with the oracle."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29573", os.path.join(ROOT, "tests", "sharded_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert out.returncode == 0, (out.stdout[-1500:], out.stderr[-1500:])
    assert out.stdout.count("SHARDED_OK") == 2, out.stdout[-1500:]
