"""Tensor-parallel decoder stack on two GPUs: the token-sharded prompt path (reduce-scatter +
all-gather of activation codes) against the all-reduce path of the same sharded model.  The ranks
run as child processes (one per GPU) under a hard time limit."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
def test_token_sharded_prefill_paths_equal_allreduce_prefill_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29543", os.path.join(HERE, "decoder_tp_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "DECODER_TP_OK" in out.stdout, out.stdout[-3000:] + out.stderr[-3000:]
