"""Model-parallel trainer worker: tp=2 x dp=2 worker groups (and the other layouts below) on CPU (gloo) give the same
losses, gradient norms and updated parameters as the single-process data-parallel trainer."""
import pytest
import torch

from axon_b200.controller.worker_group import ClassWithInitArgs, LocalWorkerGroup
from axon_b200.core.resource_pool import ResourcePool
from axon_b200.protocol import DataProto


def _cfg(tp, model="tiny-qwen3", ep=1, pp=1, vpp=1, cp=1, etp=1):
    return {"model_path": model, "force_cpu": True, "seed": 7, "max_token_len_per_gpu": 512,
            "optimizer_args": {"lr": 1e-3, "weight_decay": 0.0, "betas": [0.9, 0.95], "eps": 1e-8}, "grad_clip": 1.0,
            "megatron": {"tensor_model_parallel_size": tp, "expert_model_parallel_size": ep, "pipeline_model_parallel_size": pp,
                         "virtual_pipeline_model_parallel_size": vpp, "context_parallel_size": cp,
                         "expert_tensor_parallel_size": etp}, "recompute": "full"}


def _batch(n_rows=4, T=48, vocab=4096):
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, vocab, (n_rows, T), generator=g)
    att = torch.ones(n_rows, T, dtype=torch.long)
    att[1, 40:] = 0
    rm = att.clone().float()
    rm[:, :10] = 0
    d = DataProto.from_dict({"input_ids": ids, "attention_mask": att, "position_ids": (att.cumsum(1) - 1) * att,
                             "response_mask": rm, "advantages": torch.randn(n_rows, T, generator=g) * rm,
                             "old_log_probs": torch.zeros(n_rows, T)})
    d.meta_info["temperature"] = 1.0
    return d


def _run(cls_path, cfg, world, vocab=4096, save_dir=None, load_dir=None):
    import importlib
    mod, name = cls_path.rsplit(".", 1)
    cls = getattr(importlib.import_module(mod), name)
    wg = LocalWorkerGroup(ResourcePool([world]), ClassWithInitArgs(cls, config=cfg, name="actor"), backend="process",
                          rpc_timeout=300)
    try:
        wg.init_model()
        data = _batch(vocab=vocab)
        if load_dir is not None:                   # resume: the forward below runs on the restored parameters
            wg.load_state(load_dir)
            return (wg.forward(data).batch["log_probs"],)
        fwd = wg.forward(data)
        data.batch["old_log_probs"] = fwd.batch["log_probs"]
        from axon_b200.driver.driver_utils import process_mini_batch
        process_mini_batch(data)                   # mini-batch-global loss denominators, as the driver attaches them
        out1 = wg.forward_backward(data, loss_fn="ppo", loss_fn_args={"clip_ratio": 0.2})
        opt1 = wg.optim_step(step_lr=True)
        fwd2 = wg.forward(data)
        if save_dir is not None:
            wg.save_state(save_dir, global_step=1, save_mode="both")
            wg.wait_for_save()
        return fwd.batch["log_probs"], out1.meta_info["metrics"], opt1.meta_info["metrics"], fwd2.batch["log_probs"]
    finally:
        wg.shutdown()


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world,tp", [(4, 2)])
def test_tensor_parallel_trainer_matches_data_parallel_trainer(world, tp):
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(1), 1)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(tp), world)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)                 # log-probs before the update
    import numpy as np
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)                 # log-probs after one optimizer step
    assert (got[3] - got[0]).abs().max() > 1e-4                                      # and the step did move the model


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world,ep", [(4, 2)])
def test_expert_parallel_trainer_matches_data_parallel_trainer(world, ep):
    """ep=2 x edp=2: every rank trains on its own rows, experts are split over the group."""
    import numpy as np
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(1, "tiny-moe"), 1, vocab=2048)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(1, "tiny-moe", ep), world, vocab=2048)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-4


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world", [4])
def test_tensor_and_expert_parallel_over_one_group_matches_data_parallel_trainer(world):
    """tp = ep = 2 x dp = 2: the group divides the attention heads AND the experts; the ranks of a group see the
    same rows, each routes its own share of the tokens to the experts' owners."""
    import numpy as np
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(1, "tiny-moe"), 1, vocab=2048)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(2, "tiny-moe", 2), world, vocab=2048)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-4


@pytest.mark.timeout(900)
@pytest.mark.parametrize("kind", ["tp", "tp-bias", "ep", "pp", "tp-pp", "tp-ep", "vpp", "tp-ep-pp", "tp-etp"])
def test_model_parallel_checkpoint_exports_full_hf_model(tmp_path, kind):
    """The HF export of a tp=2 / ep=2 run holds the full tensors: an unsharded model loaded from it gives the
    run's own post-update log-probs; the sharded files and the layout note are there for resuming."""
    import json
    import os
    from axon_b200.models.config import get_config
    from axon_b200.models.dense import PackedBatch
    from axon_b200.models.moe import build_model_for
    from axon_b200.utils.hf_model import load_hf_weights
    preset, vocab = ("tiny-moe", 2048) if "ep" in kind else (("tiny-qwen2" if kind == "tp-bias" else "tiny-qwen3-untied"), 4096)
    if kind == "vpp":
        preset = "tiny-qwen3-untied-5l"
    cfg = _cfg(2 if kind.startswith("tp") else 1, preset, 2 if "ep" in kind else 1, 2 if kind.endswith("pp") else 1, 2 if kind == "vpp" else 1)
    if kind == "tp-etp":
        preset, vocab = "tiny-moe", 2048
        cfg = _cfg(2, preset, etp=2)
    world = 4 if kind in ("tp-pp", "tp-ep-pp") else 2
    d = str(tmp_path / "ck")
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", cfg, world, vocab=vocab, save_dir=d)
    assert json.load(open(os.path.join(d, "model_parallel_config.json")))["world_size"] == world
    # the sharded state is one array per parameter in full-model coordinates ...
    from axon_b200.models.params import FlatParams
    from axon_b200.utils.state.dist_checkpoint import ShardedTensor, load_sharded, read_metadata
    dist_dir = os.path.join(d, "dist_ckpt")
    meta = read_metadata(dist_dir)
    assert any(k.startswith("optimizer/") for k in meta["tensors"]) and "extra/common" in meta["objects"]
    host = FlatParams(get_config(preset), "cpu", torch.float32)
    from axon_b200.utils.state.megatron_state_manager import view2d       # the 2-D view in which shards are boxes
    load_sharded({"model/" + n: ShardedTensor("model/" + n, v, view2d(n, v.shape), [((0, 0), view2d(n, v.shape))]) for n, v in host.views.items()}, dist_dir)
    m = build_model_for(get_config(preset), device="cpu", dtype=torch.float32)
    load_hf_weights(m, os.path.join(d, "huggingface"))
    for n, v in host.views.items():              # ... which an unsharded reader assembles to the exported tensors
        torch.testing.assert_close(v, m.params.views[n].float(), rtol=0, atol=0, msg=n)
    data = _batch(vocab=vocab)
    for row in range(2):
        n = int(data.batch["attention_mask"][row].sum())
        lp, _ = m.forward(PackedBatch.from_sequences([data.batch["input_ids"][row, :n].to(torch.int32)], "cpu"))
        torch.testing.assert_close(lp[: n - 1], got[3][row, 1:n].float(), rtol=2e-3, atol=2e-3)
    # resume under the writing layout and - for the tensor-parallel run - under NO model parallelism at all
    again = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", cfg, world, vocab=vocab, load_dir=d)
    torch.testing.assert_close(again[0], got[3], rtol=1e-5, atol=1e-5)
    if kind == "tp-pp":          # written by tp 2 x pp 2, resumed by two pipeline stages without tensor parallelism
        other = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(1, preset, pp=2), 2, vocab=vocab, load_dir=d)
        torch.testing.assert_close(other[0], got[3], rtol=1e-3, atol=1e-3)
    if kind == "vpp":           # written by two ranks with two interleaved chunks each, resumed by two plain pipeline stages
        other = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(1, preset, pp=2), 2, vocab=vocab, load_dir=d)
        torch.testing.assert_close(other[0], got[3], rtol=1e-3, atol=1e-3)
    if kind == "tp-ep-pp":      # written by pipeline 2 x (tensor = expert = 2), resumed by one tensor + expert group without stages
        other = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(2, preset, 2), 2, vocab=vocab, load_dir=d)
        torch.testing.assert_close(other[0], got[3], rtol=1e-3, atol=1e-3)
    if kind == "tp-etp":        # every expert cut over two ranks when written; resumed by ranks that hold whole experts
        other = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(2, preset, 2), 2, vocab=vocab, load_dir=d)
        torch.testing.assert_close(other[0], got[3], rtol=1e-3, atol=1e-3)
    if kind == "tp-ep":         # written by one tp = ep = 2 group, resumed by two expert-parallel ranks without tensor parallelism
        other = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(1, preset, 2), 2, vocab=vocab, load_dir=d)
        torch.testing.assert_close(other[0], got[3], rtol=1e-3, atol=1e-3)
    if kind == "tp":
        single = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(1, preset), 1, vocab=vocab, load_dir=d)
        torch.testing.assert_close(single[0], got[3], rtol=1e-3, atol=1e-3)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world,pp", [(4, 2)])
def test_pipeline_parallel_trainer_matches_data_parallel_trainer(world, pp):
    """Two pipeline stages x dp=2: same log-probs, gradient norm and update as the single-process trainer."""
    import numpy as np
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(1, "tiny-qwen3-untied"), 1)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(1, "tiny-qwen3-untied", pp=pp), world)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-4


@pytest.mark.timeout(900)
def test_tensor_parallel_inside_pipeline_stages_matches_data_parallel_trainer():
    """world = 4 as pp 2 x tp 2: same log-probs, gradient norm (replicated parameters counted once across the tensor-
    parallel ranks of EACH stage) and update as the single-process trainer."""
    import numpy as np
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(1, "tiny-qwen3-untied"), 1)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(2, "tiny-qwen3-untied", pp=2), 4)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-4


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world,pp,cap", [(3, 3, 64), (3, 3, 128)])
def test_pipeline_schedule_over_several_micro_batches(world, pp, cap):
    """A token cap of 64 makes every row its own micro-batch (4 micro-batches: more than stages), 128
    gives 2 (fewer than 3 stages): the one-forward-one-backward schedule and the streamed forward match
    the single-process trainer."""
    import numpy as np
    name = "tiny-qwen3-untied-5l"        # 5 layers over 3 stages: uneven stages too
    ref_cfg, got_cfg = _cfg(1, name), _cfg(1, name, pp=pp)
    ref_cfg["max_token_len_per_gpu"] = got_cfg["max_token_len_per_gpu"] = cap
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", ref_cfg, 1)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", got_cfg, world)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(np.mean(got[1]["actor/loss"]), np.mean(ref[1]["actor/loss"]), rtol=1e-3, atol=1e-5)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)


@pytest.mark.timeout(900)
def test_tensor_parallel_trainer_with_qkv_bias_matches_data_parallel_trainer():
    """Qwen2-style q/k/v biases split with the heads of their rank; random biases make them matter."""
    import numpy as np
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(1, "tiny-qwen2"), 1)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(2, "tiny-qwen2"), 2)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world,pp,model,cap", [(2, 2, "tiny-qwen3", 512), (3, 3, "tiny-qwen3-5l", 64)])
def test_pipeline_stages_share_a_tied_embedding(world, pp, model, cap):
    """Tied embeddings: the first and the last stage both hold the table, sum its gradient, and stay equal; log-probs,
    gradient norm (the table counted once) and the update match the single-process trainer."""
    import numpy as np
    ref_cfg, got_cfg = _cfg(1, model), _cfg(1, model, pp=pp)
    ref_cfg["max_token_len_per_gpu"] = got_cfg["max_token_len_per_gpu"] = cap
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", ref_cfg, 1)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", got_cfg, world)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-4


def test_virtual_stage_schedule_runs_every_operation_once_in_dependency_order():
    """The tick table of the interleaved schedule: every (micro-batch, virtual stage) forward and backward exactly once, a
    forward only after the previous virtual stage's forward of an earlier tick, a backward only after the next virtual
    stage's backward of an earlier tick; activation memory stays within the warm-up depth when the counts divide."""
    from axon_b200.models.pp_dense import virtual_schedule
    for P, v, M in [(2, 2, 4), (2, 2, 3), (3, 2, 6), (4, 3, 5), (4, 2, 8), (2, 3, 1), (4, 1, 8)]:
        ticks = virtual_schedule(P, v, M)
        K, seen = P * v, {}
        for t, step in enumerate(ticks):
            for r, op in enumerate(step):
                if op is not None:
                    key = (op[0], op[1], op[2] * P + r)
                    assert key not in seen
                    seen[key] = t
        assert len(seen) == 2 * M * K
        for (kind, m, k), t in seen.items():
            if kind == "F" and k > 0:
                assert seen[("F", m, k - 1)] < t
            if kind == "B":
                assert seen[("F", m, k)] < t and (k == K - 1 or seen[("B", m, k + 1)] < t)
        if M % P == 0:
            for r in range(P):
                held = peak = 0
                for step in ticks:
                    if step[r] is not None:
                        held += 1 if step[r][0] == "F" else -1
                        peak = max(peak, held)
                assert peak <= ((P - r - 1) * 2 + (v - 1) * P if v > 1 else P - 1 - r) + 1
        fwd_only = virtual_schedule(P, v, M, train=False)
        assert sum(op is not None for step in fwd_only for op in step) == M * K and all(op is None or op[0] == "F" for step in fwd_only for op in step)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world,pp,vpp,cap,model", [(2, 2, 2, 64, "tiny-qwen3-untied-5l"), (2, 2, 2, 512, "tiny-qwen3-5l")])
def test_interleaved_pipeline_chunks_match_single_process(world, pp, vpp, cap, model):
    """Two ranks with two model chunks each (virtual stages 0, 2 on the first rank and 1, 3 on the second; with a token cap
    of 64 every row is its own micro-batch, with 512 there is one): log-probs, loss, gradient norm and the update equal the
    single-process trainer, also with the embedding tied between the first rank's first chunk and the last rank's last."""
    import numpy as np
    ref_cfg, got_cfg = _cfg(1, model), _cfg(1, model, pp=pp, vpp=vpp)
    ref_cfg["max_token_len_per_gpu"] = got_cfg["max_token_len_per_gpu"] = cap
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", ref_cfg, 1)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", got_cfg, world)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(np.mean(got[1]["actor/loss"]), np.mean(ref[1]["actor/loss"]), rtol=1e-3, atol=1e-5)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-4


@pytest.mark.timeout(900)
@pytest.mark.parametrize("how", ["ep", "etp"])
def test_sparse_model_with_tensor_and_expert_parallel_pipeline_stages_matches_single_process(how):
    """world = 4 as pipeline 2 x (tensor = expert = 2) - whole experts per rank, or a slice of every expert per rank (expert
    tensor parallelism) - token cap 64 so that every row is its own micro-batch and several are in flight: log-probs,
    loss, gradient norm and update equal the single-process trainer."""
    import numpy as np
    ref_cfg, got_cfg = _cfg(1, "tiny-moe"), (_cfg(2, "tiny-moe", ep=2, pp=2) if how == "ep" else _cfg(2, "tiny-moe", etp=2, pp=2))
    ref_cfg["max_token_len_per_gpu"] = got_cfg["max_token_len_per_gpu"] = 64
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", ref_cfg, 1, vocab=2048)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", got_cfg, 4, vocab=2048)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(np.mean(got[1]["actor/loss"]), np.mean(ref[1]["actor/loss"]), rtol=1e-3, atol=1e-5)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-4


@pytest.mark.timeout(900)
def test_tensor_parallel_groups_as_context_parallel_ranks_match_single_process():
    """world = 4 as context 2 x tensor 2: every sequence is cut into zigzag chunks over two tensor-parallel groups, whose
    members exchange the K|V of their own heads; log-probs, gradient norm and update equal the single-process trainer."""
    import numpy as np
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(1, "tiny-qwen3-untied"), 1)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(2, "tiny-qwen3-untied", cp=2), 4)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-4


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world", [2])
def test_expert_tensor_parallel_trainer_matches_data_parallel_trainer(world):
    """tp = etp = 2: every rank holds a slice of the intermediate units of EVERY expert and works on all the
    group's tokens; partial expert outputs are reduce-scattered back to the rows' owners."""
    import numpy as np
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(1, "tiny-moe"), 1, vocab=2048)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(2, "tiny-moe", etp=2), world, vocab=2048)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-4


@pytest.mark.timeout(900)
def test_tensor_parallel_critic_matches_single_process():
    """A value-head model (critic) under tensor parallelism: values, the value-loss update and the values after it equal the
    single-process critic."""
    import importlib

    def run(cls_path, cfg, world):
        mod, name = cls_path.rsplit(".", 1)
        from axon_b200.trainer.fsdp_trainer import ValueModel
        wg = LocalWorkerGroup(ResourcePool([world]), ClassWithInitArgs(getattr(importlib.import_module(mod), name), config=cfg, name="critic",
                                                                       model=ValueModel), backend="process", rpc_timeout=300)
        try:
            wg.init_model()
            data = _batch()
            v0 = wg.forward(data).batch["values"]
            g = torch.Generator().manual_seed(5)
            data.batch["values"] = v0
            data.batch["returns"] = (v0 + torch.randn(v0.shape, generator=g) * 0.1) * data.batch["response_mask"]
            from axon_b200.driver.driver_utils import process_mini_batch
            process_mini_batch(data)
            m = wg.forward_backward(data, loss_fn="value", loss_fn_args={"cliprange_value": 0.5})
            opt = wg.optim_step(step_lr=True)
            return v0, m.meta_info["metrics"], opt.meta_info["metrics"], wg.forward(data).batch["values"]
        finally:
            wg.shutdown()
    ref = run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(1), 1)
    got = run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(2), 2)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-5


@pytest.mark.timeout(900)
def test_tensor_parallel_trainer_with_multi_token_prediction_matches_single_process(monkeypatch):
    """The depth-1 prediction module under tensor parallelism: its own decoder layer is cut like the others, its
    projection and norms are whole on every rank; reported loss, gradient norm and update equal the single-process run."""
    import numpy as np
    monkeypatch.setenv("AXON_ENABLE_MTP", "1")       # the worker processes inherit it; another test may have switched the module off
    ref_cfg, got_cfg = _cfg(1, "tiny-qwen3-mtp"), _cfg(2, "tiny-qwen3-mtp")
    ref_cfg["mtp_loss_scaling_factor"] = got_cfg["mtp_loss_scaling_factor"] = 0.3
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", ref_cfg, 1)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", got_cfg, 2)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    assert "actor/mtp_loss" in ref[1] and abs(np.mean(got[1]["actor/mtp_loss"]) - np.mean(ref[1]["actor/mtp_loss"])) < 1e-3
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)


@pytest.mark.timeout(900)
def test_tensor_parallel_inside_interleaved_pipeline_chunks_matches_single_process():
    """world = 4 as pipeline 2 x tensor 2 with two model chunks per pipeline rank, every row its own micro-batch: equals the
    single-process trainer."""
    import numpy as np
    name = "tiny-qwen3-untied-5l"
    ref_cfg, got_cfg = _cfg(1, name), _cfg(2, name, pp=2, vpp=2)
    ref_cfg["max_token_len_per_gpu"] = got_cfg["max_token_len_per_gpu"] = 64
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", ref_cfg, 1)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", got_cfg, 4)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(np.mean(got[1]["actor/loss"]), np.mean(ref[1]["actor/loss"]), rtol=1e-3, atol=1e-5)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("kind", ["ep", "tp-ep", "tp-etp"])
def test_sparse_model_with_multi_token_prediction_matches_single_process(monkeypatch, kind):
    """The prediction module of a sparse model is a sparse layer of its own: under expert parallelism, tensor + expert
    parallelism and expert tensor parallelism its experts are divided like the decoder's; reported loss, gradient norm and
    update equal the single-process run."""
    import numpy as np
    monkeypatch.setenv("AXON_ENABLE_MTP", "1")
    name = "tiny-moe-mtp"
    got_cfg = {"ep": _cfg(1, name, ep=2), "tp-ep": _cfg(2, name, ep=2), "tp-etp": _cfg(2, name, etp=2)}[kind]
    ref_cfg = _cfg(1, name)
    ref_cfg["mtp_loss_scaling_factor"] = got_cfg["mtp_loss_scaling_factor"] = 0.3
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", ref_cfg, 1, vocab=2048)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", got_cfg, 2, vocab=2048)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    assert "actor/mtp_loss" in ref[1] and abs(np.mean(got[1]["actor/mtp_loss"]) - np.mean(ref[1]["actor/mtp_loss"])) < 1e-3
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("kind", ["tied", "untied-micro"])
def test_pipeline_trainer_with_multi_token_prediction_matches_single_process(monkeypatch, tmp_path, kind):
    """The prediction module sits on the last stage and embeds the next token there, so the table lives on both ends of
    the pipeline (tied or not) with its gradients summed; one micro-batch and one per row both equal the single process."""
    import numpy as np
    monkeypatch.setenv("AXON_ENABLE_MTP", "1")
    name = "tiny-qwen3-mtp" if kind == "tied" else "tiny-qwen3-untied-mtp"
    ref_cfg, got_cfg = _cfg(1, name), _cfg(1, name, pp=2)
    ref_cfg["mtp_loss_scaling_factor"] = got_cfg["mtp_loss_scaling_factor"] = 0.3
    if kind == "untied-micro":
        ref_cfg["max_token_len_per_gpu"] = got_cfg["max_token_len_per_gpu"] = 64
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", ref_cfg, 1)
    d = str(tmp_path / "ck") if kind == "untied-micro" else None
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", got_cfg, 2, save_dir=d)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    assert "actor/mtp_loss" in got[1] and abs(np.mean(got[1]["actor/mtp_loss"]) - np.mean(ref[1]["actor/mtp_loss"])) < 1e-3
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    if d is not None:          # the table is written once although both ends hold it; a single process reads the checkpoint back
        single = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cfg(1, name), 1, load_dir=d)
        torch.testing.assert_close(single[0], got[3], rtol=1e-3, atol=1e-3)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("kind", ["dense", "sparse"])
def test_tensor_parallel_pipeline_stages_with_multi_token_prediction_match_single_process(monkeypatch, kind):
    """world = 4 as pipeline 2 x tensor 2 (the sparse model with tensor = expert 2), every row its own micro-batch: the
    prediction module runs on the last stage's tensor-parallel group."""
    import numpy as np
    monkeypatch.setenv("AXON_ENABLE_MTP", "1")
    name, vocab = ("tiny-qwen3-untied-mtp", 4096) if kind == "dense" else ("tiny-moe-mtp", 2048)
    ref_cfg, got_cfg = _cfg(1, name), (_cfg(2, name, pp=2) if kind == "dense" else _cfg(2, name, ep=2, pp=2))
    for c in (ref_cfg, got_cfg):
        c["mtp_loss_scaling_factor"], c["max_token_len_per_gpu"] = 0.3, 64
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", ref_cfg, 1, vocab=vocab)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", got_cfg, 4, vocab=vocab)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    assert "actor/mtp_loss" in got[1] and abs(np.mean(got[1]["actor/mtp_loss"]) - np.mean(ref[1]["actor/mtp_loss"])) < 1e-3
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
