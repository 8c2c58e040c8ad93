"""Sharded weights with the all-gather fused into the GEMM: 2 gloo ranks (fallback path) and 2 GPUs (peer-TMA kernel)."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(tmp_path, kind, port):
    out = tmp_path / "fg.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "_fsdp_gather_worker.py"), str(out), kind]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return json.loads(out.read_text())


@pytest.mark.timeout(600)
def test_sharded_linear_cpu():
    import tempfile
    from pathlib import Path
    with tempfile.TemporaryDirectory() as d:
        for x in _run(Path(d), "cpu", 29681):
            assert not x["fused"] and max(x["errs"]) < 1e-5, x


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_weight_gather_fused_gemm_gpu(tmp_path):
    for x in _run(tmp_path, "cuda", 29682):
        assert x["fused"] and max(x["errs"]) < 2e-2, x
