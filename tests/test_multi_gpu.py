"""Two-GPU checks (skipped with fewer): the sharded long-context decode through NCCL
and through the peer-memory exchange kernel, run as torchrun child processes.  NVLS
is switched off for the children, and the exchange uses plain peer loads/stores."""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.timeout(600)
def test_sharded_decode_over_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533",
           str(ROOT / "tests" / "multi_gpu_worker.py")]
    run = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=540)
    assert run.returncode == 0 and "MULTI_GPU_OK" in run.stdout, run.stdout[-3000:] + run.stderr[-3000:]
