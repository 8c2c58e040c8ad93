"""Ulysses sequence parallelism: the exchange's index maps, and sp=2 trainers (x dp=1 and x dp=2, gloo on CPU)
that match the single-process trainer in log-probs, gradient norm and the parameters after a step."""
import numpy as np
import pytest
import torch

from test_megatron_trainer import _run


def _cfg(sp):
    return {"model_path": "tiny-qwen3", "force_cpu": True, "seed": 7, "max_token_len_per_gpu": 512,
            "optimizer_args": {"lr": 1e-3, "weight_decay": 0.0, "betas": [0.9, 0.95], "eps": 1e-8}, "grad_clip": 1.0,
            "fsdp": {"ulysses_sequence_parallel_size": sp}, "recompute": "full"}


def test_exchange_maps_are_inverse_single_rank():
    from axon_b200.parallel.ulysses import UlyssesContext
    ctx = UlyssesContext(None, "cpu", 64, 96)
    x = torch.randn(10, 96)
    segs_out = [(0, 64, 0), (64, 16, 64), (80, 16, 80)]
    y = ctx.scatter_cols(x, segs_out, 96)
    assert torch.equal(y, x)
    assert torch.equal(ctx.scatter_rows(y, segs_out, 96), x)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world,sp", [(2, 2), (4, 2)])
def test_sequence_parallel_trainer_matches_single_process(world, sp):
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(1), 1)
    got = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(sp), world)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-4


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_fused_exchange_and_model_on_two_gpus(tmp_path):
    import json, os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "ul.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29671", os.path.join(root, "tests", "_ulysses_worker.py"), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for x in json.loads(out.read_text()):
        assert x["fused"] and x["exchange_exact"] and x["status_ok"], x
        assert x["lp_err"] < 0.2 and x["ent_err"] < 0.15 and x["grad_rel"] < 0.08, x
