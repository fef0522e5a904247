"""Expert-parallel parity on 2+ GPUs: spawns one process per GPU (torchrun)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(n):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", OMOE_EP_WAIT_MS="5000")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.join(ROOT, "tests", "ep_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "ep parity ok" in p.stdout


def test_expert_parallel_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(2)


def test_expert_parallel_all_gpus():
    n = torch.cuda.device_count()
    if n < 4:
        pytest.skip("needs 4 or more GPUs")
    _run(8 if n >= 8 else 4)
