"""Two real ranks on two GPUs: the sharded map over NCCL all-to-all and over the peer-memory exchange against one
serial oracle table.  Skipped on machines with fewer than two GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_nccl_and_peer_exchange_match_one_table():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(HERE, "multi_gpu_worker.py")]
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    assert "multi-gpu parity ok" in done.stdout
