"""Expert and tensor parallelism over two GPUs of one box (tests/ep_worker.py under torchrun); skipped where fewer are
visible."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(mode: str, port: int) -> None:
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "ep_worker.py"),
                          mode], capture_output=True, text=True, timeout=600, env=env)
    assert "EP_WORKER_OK" in out.stdout, out.stdout[-3000:] + out.stderr[-3000:]


def test_two_rank_expert_parallel_matches_one_gpu_and_reports_a_missing_rank():
    _run("ep", 29611)


def test_two_rank_tensor_parallel_matches_one_gpu_and_reports_a_missing_rank():
    _run("tp", 29612)
