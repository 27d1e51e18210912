"""Multi-GPU parity: launches tests/_multirank_worker.py with one process per GPU (2 and, when
the box has them, 4 and 8 GPUs).  Skipped on a single-GPU box."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
WORKER = Path(__file__).resolve().parent / "_multirank_worker.py"


@pytest.mark.parametrize("world", [2, 4, 8])
def test_multirank_parity(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ)
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    port = 29700 + world
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           str(WORKER)]
    res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                         timeout=900)
    assert res.returncode == 0, res.stdout[-4000:]
    assert f"multirank parity ok on {world} GPUs" in res.stdout
