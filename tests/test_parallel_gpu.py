"""Two replicas on two GPUs: the gradient sum through peer memory inside the step's graph against
the NCCL all-reduce between two graphs (tests/dp_worker.py).  Skipped with fewer than two GPUs."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_reduce_equals_nccl_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    worker = Path(__file__).parent / "dp_worker.py"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533", str(worker)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "DP_WORKER_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
