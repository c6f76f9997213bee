"""Context parallelism on real GPUs (NCCL + peer stores); needs at least two devices."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def _launch(nproc, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "_cp_gpu_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", OMP_NUM_THREADS="4")
    return subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)


def test_context_parallel_on_gpus():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if n < 2:
        pytest.skip("needs at least two GPUs")
    nproc = 4 if n >= 4 else 2
    proc = _launch(nproc, 29741)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
