"""Parameter shards for the family toolkit: a family model whose decoder layers are cut into one piece per rank gives
the unsharded model's log-probs and gradients (different data per rank), gathers back to the same tensors, and trains
through the FSDP trainer worker like the single-process run."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from test_megatron_trainer import _cfg, _run

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world", [2, 3])
def test_sharded_family_model_matches_unsharded(tmp_path, world):
    out = tmp_path / "sf.json"
    presets = "tiny-gemma3,tiny-qwen3-next,tiny-deepseek-v3"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29694 + world), os.path.join(ROOT, "tests", "_sharded_family_worker.py"), str(out), presets]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=800)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for x in json.loads(out.read_text()):
        for p in presets.split(","):
            y = x[p]
            assert y["lp_err"] < 1e-5 and y["grad_rel"] < 1e-5 and y["gathered_equal"] and y["piece_grad_norm"] > 0, (p, y)
            assert y["local_numel"] < y["full_numel"], (p, y)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("model,vocab", [("tiny-gemma3", 512), ("tiny-glm4-moe", 512)])
def test_sharded_family_trainer_matches_single_process(model, vocab):
    from axon_b200.models.config import get_config
    vocab = get_config(model).vocab_size
    z3 = _cfg(1, model)
    z3["fsdp"] = {"param_sharding": True}
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(1, model), 1, vocab=vocab)
    got = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", z3, 2, vocab=vocab)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-4


@pytest.mark.timeout(900)
def test_sharded_family_run_exports_whole_model_and_resumes(tmp_path):
    from axon_b200.models.config import get_config
    from axon_b200.models.dense import PackedBatch
    from axon_b200.models.families import FamilyModel
    from axon_b200.utils.hf_model import iter_hf_weights
    from test_megatron_trainer import _batch
    model = "tiny-gemma3"
    vocab = get_config(model).vocab_size
    z3 = _cfg(1, model)
    z3["fsdp"] = {"param_sharding": True}
    d = str(tmp_path / "ck")
    got = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", z3, 2, vocab=vocab, save_dir=d)
    assert json.load(open(os.path.join(d, "fsdp_config.json"))) == {"FSDP_version": "layer-pieces", "world_size": 2}
    # the export holds whole tensors under the family's checkpoint names: an unsharded model loaded from it gives the
    # run's own post-update log-probs
    m = FamilyModel(get_config(os.path.join(d, "huggingface")), device="cpu", dtype=torch.float32)
    m.load_state_dict(dict(iter_hf_weights(os.path.join(d, "huggingface"))))
    data = _batch(vocab=vocab)
    for row in range(2):
        n = int(data.batch["attention_mask"][row].sum())
        lp, _ = m.forward(PackedBatch.from_sequences([data.batch["input_ids"][row, :n].to(torch.int32)], "cpu"))
        torch.testing.assert_close(lp[: n - 1], got[3][row, 1:n].float(), rtol=2e-3, atol=2e-3)
    again = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", z3, 2, vocab=vocab, load_dir=d)
    torch.testing.assert_close(again[0], got[3], rtol=1e-5, atol=1e-5)
    # ... and a sharded run can start from the export (streamed in layer by layer)
    z3b = dict(z3, model_path=os.path.join(d, "huggingface"))
    fresh = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", z3b, 2, vocab=vocab)
    torch.testing.assert_close(fresh[0], got[3], rtol=2e-3, atol=2e-3)
