"""Two real ranks on two GPUs: the sharded map over NCCL all-to-all and over the peer-memory exchange against one
serial oracle table.  Skipped on machines with fewer than two GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("world,value_columns", [(2, 2), (2, 5), (4, 2), (8, 2)])
def test_ranks_on_real_gpus_match_one_table(world, value_columns):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29533 + world), os.path.join(HERE, "multi_gpu_worker.py"), str(value_columns)]
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-6000:]
    assert "multi-gpu parity ok" in done.stdout
