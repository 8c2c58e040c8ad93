"""Tensor-parallel sampler group: a model sharded over the group (heads, MLP columns, whole experts) generates what
the unsharded model generates; the group's servers run in lockstep behind their first rank (requests, sleep / wake,
weight updates with full tensors, reset). CPU: 2 gloo ranks. GPU: 2 ranks, sums through the peer-memory kernel."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(tmp_path, n, kind, port, how="tp"):
    out = tmp_path / "tps.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "_tp_sampler_worker.py"), str(out), kind, how]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return json.loads(out.read_text())


def _check(res, presets, tol, exact, routed=True):
    for x in res:
        for p in presets:
            y = x[p]
            assert y["same_tokens_on_all_ranks"] and y["logprob_err"] < tol, (p, y)
            if exact:
                assert y["equals_unsharded"], (p, y)
            if x["rank"] == 0:
                assert y["server_first_len"] == [16] * 6 and y["updated"] > 0 and y["after_update_err"] < tol, (p, y)
                assert y["aborted_reason"] in ("abort", "length") and y["third_equals_second"], (p, y)
                assert y["server_first_err"] < tol, (p, y)
            else:
                assert y["follower_done"] and y["follower_error"] is None, (p, y)
        assert x["tiny-moe" if exact else "tiny-moe-gpu"]["routed"] or not routed


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world", [2, 4])
def test_sampler_group_matches_unsharded_model_cpu(tmp_path, world):
    """Groups of 2 and of 4 ranks; the models have 2 key / value heads, so in the group of 4 two ranks each hold the same one."""
    res = _run(tmp_path, world, "cpu", 29671 + world)
    _check(res, ("tiny-qwen3", "tiny-moe"), 1e-4, exact=True)
    assert not res[0]["fused"] and len(res) == world


@pytest.mark.timeout(900)
def test_pipelined_sampler_group_matches_unsharded_model_cpu(tmp_path):
    """A group of 2 ranks that holds the model by layers (each rank its slice and its share of the KV cache): the stream
    crosses the stage boundary inside every prefill / decode call, every rank computes the same logits, and the group's
    servers run in lockstep like a tensor-parallel group's (requests, sleep / wake, weight updates, reset)."""
    res = _run(tmp_path, 2, "cpu", 29679, how="pp")
    _check(res, ("tiny-qwen3", "tiny-moe"), 1e-4, exact=True, routed=False)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_tp2_sampler_group_sums_through_peer_memory_gpu(tmp_path):
    res = _run(tmp_path, 2, "cuda", 29672)
    _check(res, ("tiny-gpu", "tiny-moe-gpu"), 0.15, exact=False)
    for x in res:
        assert x["fused"] and x["reduce_calls"]["fused"] > 0 and x["status"] == 0, x
        assert x["tiny-gpu"]["graphs"] > 0, x          # the decode graph replays the peer-memory sums


def test_sampler_group_models_accept_a_checkpoint_with_a_prediction_module():
    """A multi-token-prediction module behind the decoder is a training device. A sampler stage holds none of it (its
    tensors are skipped when weights arrive); a tensor-parallel member keeps its cut like any layer's and never runs it.
    Both generate what the whole model generates."""
    import torch
    from axon_b200.models.config import get_config
    from axon_b200.models.moe import build_model_for
    from axon_b200.models.pp_infer import StagedDenseModel
    from axon_b200.models.tp_infer import Shard, ShardedDenseModel, ShardedMoEModel
    from axon_b200.sampler.engine import GenerationEngine
    from axon_b200.sampler.params import SamplingParams

    class _Alone:                     # a group of one: nothing to sum
        calls: dict = {}

        def begin_step(self):
            pass

        def __call__(self, y):
            return y
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    prompt = [[5, 6, 7, 8, 9]]
    for preset, kinds in (("tiny-qwen3-mtp", (StagedDenseModel, ShardedDenseModel)), ("tiny-moe-mtp", (ShardedMoEModel,))):
        cfg = get_config(preset)
        full = build_model_for(cfg, "cpu", torch.float32)
        full.params.init_random(std=0.08, seed=3)
        want = GenerationEngine(full, num_pages=8, max_num_seqs=4, seed=1).generate(prompt, sp)[0].token_ids
        for cls in kinds:
            part = cls(cfg, Shard(None, 0, 1, _Alone()), device="cpu", dtype=torch.float32)
            part.load_full_state(full.params.views)
            assert GenerationEngine(part, num_pages=8, max_num_seqs=4, seed=1).generate(prompt, sp)[0].token_ids == want
            if cls is StagedDenseModel:
                L = cfg.num_hidden_layers
                assert part.localize(f"model.layers.{L}.eh_proj.weight", torch.zeros(1)) is None
                assert part.localize("model.layers.0.input_layernorm.weight", torch.zeros(1))[0] == "model.layers.0.input_layernorm.weight"
