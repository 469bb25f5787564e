"""Expert parallelism over two GPUs of one box (tests/ep_worker.py under torchrun); skipped where fewer are visible."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_rank_expert_parallel_matches_one_gpu_and_reports_a_missing_rank():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29611", os.path.join(ROOT, "tests", "ep_worker.py")],
                         capture_output=True, text=True, timeout=600, env=env)
    assert "EP_WORKER_OK" in out.stdout, out.stdout[-3000:] + out.stderr[-3000:]
