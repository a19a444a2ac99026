"""All-reduce fused into the decode GEMM over NVLink peer memory: needs at least two GPUs, runs
the ranks as child processes (one per GPU) under a hard time limit."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
def test_fused_allreduce_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29541", os.path.join(HERE, "allreduce_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert out.returncode == 0 and "ALLREDUCE_OK" in out.stdout, out.stdout[-3000:] + out.stderr[-3000:]
