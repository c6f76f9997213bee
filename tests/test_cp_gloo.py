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


# one torchrun launch per (ranks, CFG size, Ulysses limit, CP backend); the worker runs the listed modes in turn
@pytest.mark.parametrize("nproc,cfg,up,backend,mode", [
    # Ulysses-2; producer-callback API (serial schedule on CPU); image-CP core in ring and all-gather-KV mode
    # every launch also replays the fixtures the reference's own CP wrapper produced for that layout ("golden:")
    (2, 1, 2, "ucp", "plain,fused,imagecp_ring,imagecp_agkv,golden:ulysses2,golden:ulysses2_bf16,golden:fulltxt_ulysses2"),
    # fixtures produced by the reference's own image-CP core ("imgolden:"), its FP8 transfer and K/V cache included
    (2, 1, 2, "ucp", "imgolden:agkv2,imgolden:ulysses2,imgolden:ring2,imgolden:agkv2_fp8,imgolden:agkv2_cache"),
    (2, 1, 1, "ucp", "plain,golden:ring2,golden:ring2_bf16,cached_ring"),  # ring-2; cached ring states
    # all-gather-KV, also with the replicated-text layout
    (2, 1, 2, "agcp", "plain,fulltxt,qwen,golden:agcp2,golden:agcp2_bf16,golden:fulltxt_agcp2"),
    # Ulysses-2 x ring-2; batch > 1 (unpack-copy path); Qwen layout with a padded tail; image-CP core, unified mode
    (4, 1, 2, "ucp", "plain,batch2,fulltxt,qwen,imagecp_unified,golden:usp_u2r2,golden:usp_u2r2_batch2,"
                     "golden:usp_u2r2_bf16,golden:fulltxt_usp_u2r2,imgolden:unified4_u2"),
    (4, 1, 4, "ucp", "golden:ulysses4"),
    # ring-4; ring attention that reuses the states of skipped source blocks
    (4, 1, 1, "ucp", "golden:ring4,golden:fulltxt_ring4,cached_ring"),
    (4, 1, 4, "agcp", "golden:agcp4"),
    # CFG-parallel 2 x Ulysses-2: two independent CP groups; token dispatch / gather; CFG exchange + combine
    (4, 2, 2, "ucp", "plain,dispatch"),
])
def test_context_parallel_layouts(nproc, cfg, up, backend, mode):
    _run(nproc, cfg, up, backend, mode)
