"""Expert-parallel MoE (tokens dispatched to the expert owners and combined back) equals the unsharded
model on every rank's tokens: log-probs, expert weight gradients on the owners, summed gradients of the
shared parameters. CPU: gloo with gathered payloads. GPU: dispatch / combine through peer memory."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(tmp_path, n, kind, port, worker="_ep_worker.py"):
    out = tmp_path / "ep.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", worker), str(out), kind]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return json.loads(out.read_text())


@pytest.mark.timeout(600)
@pytest.mark.parametrize("n", [2, 4])
def test_ep_matches_unsharded_model_cpu(tmp_path, n):
    for x in _run(tmp_path, n, "cpu", 29651):
        assert not x["fused"] and x["lp_err"] < 1e-4, x
        worst = sorted(x["grad_rel"].items(), key=lambda kv: -kv[1])[:3]
        assert worst[0][1] < 1e-4, worst


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_ep_peer_memory_kernels_match_unsharded_model_gpu(tmp_path):
    for x in _run(tmp_path, 2, "cuda", 29652):
        assert x["fused"] and x["lp_err"] < 0.25, x
        worst = sorted(x["grad_rel"].items(), key=lambda kv: -kv[1])[:3]
        assert worst[0][1] < 0.15, worst


@pytest.mark.timeout(600)
def test_tensor_plus_expert_parallel_group_matches_unsharded_model_cpu(tmp_path):
    """One group divides the attention heads (sequence-parallel rows) and the experts: local log-probs / entropy, every
    gradient shard (expert gradients on the owners), the global gradient norm, and the model's own routing."""
    for x in _run(tmp_path, 2, "cpu", 29653, "_tp_ep_worker.py"):
        assert not x["fused"] and x["lp_err"] < 1e-4 and x["ent_err"] < 1e-4 and x["norm_rel"] < 1e-5 and x["routing_equal"], x
        assert max(x["grad_rel"].values()) < 1e-4, sorted(x["grad_rel"].items(), key=lambda kv: -kv[1])[:3]


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_tensor_plus_expert_parallel_group_on_the_fused_kernels_gpu(tmp_path):
    for x in _run(tmp_path, 2, "cuda", 29654, "_tp_ep_worker.py"):
        assert x["fused"] and x["ep_fused"] and x["lp_err"] < 0.25 and x["ent_err"] < 0.2 and x["norm_rel"] < 0.05, x
        worst = sorted(x["grad_rel"].items(), key=lambda kv: -kv[1])[:3]
        assert worst[0][1] < 0.15, worst
