"""Fused peer-memory kernels on 2+ GPUs (skipped on smaller boxes): device barrier, ZeRO-1 step vs
NCCL + torch.optim.AdamW, RoutingTable plan pushed over NVLink."""
import json
import os
import subprocess
import sys

import pytest
import torch


def _n_gpus():
    try:
        return torch.cuda.device_count()
    except Exception:  # noqa: BLE001
        return 0


@pytest.mark.gpu
@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_fused_peer_kernels(tmp_path):
    # two ranks by default; AXON_TEST_RANKS=4 (or 8) runs the same checks on more GPUs of the box
    n = max(2, min(int(os.environ.get("AXON_TEST_RANKS", "2")), _n_gpus()))
    out = tmp_path / "res.json"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(root, "tests", "_mgpu_worker.py"), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.loads(out.read_text())
    for rank, x in enumerate(res):
        assert x["peer_values"] == [float(i + 1) for i in range(n)]
        # The first AdamW step moves every element by lr * g / (|g| + eps): where the summed gradient is within a few eps
        # of zero the order of the cross-rank sum decides the step, so the bound is 1 % of the step size (lr = 1e-2).
        assert x["zero1_norm_err"] < 1e-4 and x["zero1_param_err"] < 2e-2 and x["zero1_master_err"] < 1e-4, x
        assert x["sync_exact"] and x["status_ok"], x
        assert x["engine_fused_active"] and x["engine_replicas_equal"], x
        assert x["engine_param_diff"] < 2e-2, x                       # bf16 parameters after two updates
        n0 = x["engine_norms"]
        assert abs(n0[0] - n0[1]) / max(n0[1], 1e-9) < 1e-3 and abs(n0[2] - n0[3]) / max(n0[3], 1e-9) < 2e-2, x
    print("push GB/s:", res[0]["sync_push_gbs"])
