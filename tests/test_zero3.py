"""Parameter shards (ZeRO-3 / FSDP style): a world of 2 and of 4 ranks with different data per rank matches the
single-process trainer in log-probs, gradient norm and the parameters after a step; the HF export holds full tensors."""
import json
import os

import numpy as np
import pytest
import torch

from test_megatron_trainer import _batch, _cfg, _run


def _z3(model="tiny-qwen3"):
    c = _cfg(1, model)
    c["fsdp"] = {"param_sharding": True}
    return c


def test_layout_cuts_only_the_layer_matrices():
    from axon_b200.models.config import get_config
    from axon_b200.models.params import param_layout
    from axon_b200.parallel.zero3 import zero3_layout
    cfg = get_config("tiny-qwen2")
    full, cut = param_layout(cfg), zero3_layout(cfg, 4)
    for name, shape in full.items():
        if name.endswith(("qkv_proj.weight", "o_proj.weight", "gate_up_proj.weight", "down_proj.weight")):
            assert cut[name] == (shape[0] // 4, shape[1])
        else:
            assert cut[name] == tuple(shape), name


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world,model", [(2, "tiny-qwen3"), (4, "tiny-qwen2")])
def test_sharded_parameter_trainer_matches_single_process(world, model):
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(1, model), 1)
    got = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _z3(model), world)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-4


@pytest.mark.timeout(900)
def test_sharded_run_exports_full_hf_model(tmp_path):
    from axon_b200.models.config import get_config
    from axon_b200.models.dense import DenseModel, PackedBatch
    from axon_b200.utils.hf_model import load_hf_weights
    d = str(tmp_path / "ck")
    got = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _z3("tiny-qwen3-untied"), 2, save_dir=d)
    assert json.load(open(os.path.join(d, "model_parallel_config.json")))["param_shards"] == 2
    m = DenseModel(get_config("tiny-qwen3-untied"), device="cpu", dtype=torch.float32)
    load_hf_weights(m, os.path.join(d, "huggingface"))
    data = _batch()
    for row in range(2):
        n = int(data.batch["attention_mask"][row].sum())
        lp, _ = m.forward(PackedBatch.from_sequences([data.batch["input_ids"][row, :n].to(torch.int32)], "cpu"))
        torch.testing.assert_close(lp[: n - 1], got[3][row, 1:n].float(), rtol=2e-3, atol=2e-3)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_fused_weight_gather_model_on_two_gpus(tmp_path):
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "z3.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29675", os.path.join(root, "tests", "_zero3_worker.py"), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for x in json.loads(out.read_text()):
        assert x["fused"] and x["status_ok"], x
        assert x["lp_err"] < 0.2 and x["ent_err"] < 0.15 and x["grad_rel"] < 0.08, x


@pytest.mark.timeout(900)
def test_hybrid_sharding_matches_single_process():
    """``fsdp.fsdp_size = 2`` on four ranks: optimizer shards inside groups of two, replicas across the groups. Log-probs,
    gradient norm and the parameters after the step equal the single-process run."""
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(1, "tiny-qwen3"), 1)
    c = _cfg(1, "tiny-qwen3")
    c["fsdp"] = {"fsdp_size": 2}
    got = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", c, 4)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-4
