"""Context parallelism on real GPUs (needs at least two): CP result == single-GPU result."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _launch(world):
    port = 29700 + (os.getpid() % 1000)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "cp_gpu_worker.py")]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=600)


def test_context_parallel_matches_single_gpu():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 2 if n < 4 else 4
    res = _launch(world)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "cp gpu worker ok" in res.stdout
    print(res.stdout[-1500:])
