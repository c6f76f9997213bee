"""World-size > 1 tests of the context-parallel host logic on CPU (gloo) ranks."""

import os
import subprocess
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
WORKER = os.path.join(ROOT, "tests", "_cp_worker.py")
_PORT = [29611]


def _run(nproc, cfg_size, up, cp_backend, mode):
    _PORT[0] += 1
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_PORT[0]), WORKER, str(cfg_size), str(up), cp_backend, mode]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]


@pytest.mark.parametrize("nproc,cfg,up,backend,mode", [
    (2, 1, 2, "ucp", "plain"),      # Ulysses-2
    (2, 1, 1, "ucp", "plain"),      # ring-2
    (2, 1, 2, "agcp", "plain"),     # all-gather-KV
    (4, 1, 2, "ucp", "plain"),      # Ulysses-2 x ring-2
    (4, 1, 2, "ucp", "batch2"),     # batch > 1 takes the unpack-copy path
    (4, 2, 2, "ucp", "plain"),      # CFG-parallel 2 x Ulysses-2: two independent CP groups
    (4, 1, 2, "ucp", "fulltxt"),    # Qwen layout, padded tail, Ulysses x ring
    (2, 1, 2, "agcp", "fulltxt"),
    (2, 1, 2, "ucp", "fused"),      # producer-callback API (falls back to the serial schedule on CPU)
    (4, 1, 2, "ucp", "imagecp_unified"),   # image-CP core: Ulysses-2 x ring-2
    (2, 1, 2, "ucp", "imagecp_ring"),
    (2, 1, 2, "ucp", "imagecp_agkv"),
    (4, 2, 2, "ucp", "dispatch"),   # token dispatch / gather with a padded tail; CFG-parallel exchange + combine
])
def test_context_parallel_layouts(nproc, cfg, up, backend, mode):
    _run(nproc, cfg, up, backend, mode)
