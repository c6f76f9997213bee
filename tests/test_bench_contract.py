"""bench.py on a machine without a GPU: the reference arm prints the agreed JSON line, the product arm refuses to run."""

import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def _run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=600, cwd=ROOT)


def test_reference_arm_line():
    proc = _run("--impl", "reference", "--steps", "1", "--warmup", "0", "--workload", "wan1.3b-480p-17f-layer")
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads([ln for ln in proc.stdout.splitlines() if ln.startswith("{")][-1])
    assert line["impl"] == "reference" and line["metric"] == "attention_tflops" and line["unit"] == "TFLOP/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["steps"] == 1
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] in ("port", "reference")
    assert line["cpu_baseline"]["cores"] >= 1 and line["e2e"]["h2d_bytes_per_step"] == 0
    assert line["config"]["workload"] == "wan1.3b-480p-17f-layer"


@pytest.mark.skipif(torch.cuda.is_available(), reason="only meaningful without a GPU")
def test_product_arm_has_no_cpu_path():
    proc = _run("--steps", "1", "--warmup", "0")
    assert proc.returncode != 0
    assert "CUDA" in proc.stderr
