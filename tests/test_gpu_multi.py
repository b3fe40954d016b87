"""Multi-GPU checks; skipped on a single-GPU box.  Ranks are child processes (torchrun), NVLS is
switched off for them, and no rank leaves while work is in flight."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pushed_output_equals_all_gather_on_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300),
           os.path.join(ROOT, "tests", "multigpu_push_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "PUSH_EQUALS_ALLGATHER" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
