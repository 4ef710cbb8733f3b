"""Data parallelism on real GPUs (needs at least two): child processes, one per GPU, run tests/dp_gpu_worker.py over
NCCL -- bucketed all-reduce against an all-gathered sum, the one-graph step against eager steps, the two-graph
fallback, identical parameters on every rank.  NCCL's in-switch reduction is switched off for the children and the
process group gives up after a minute, so a failure ends with an error instead of a stall."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_gpu_train_step_bucketed_allreduce_in_graph():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs (the CPU twin of this test is tests/test_dp_cpu.py)")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", AETHER_DP_TIMEOUT_S="60")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "dp_gpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "DP_GPU_OK 2" in r.stdout
