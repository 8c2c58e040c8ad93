"""End-to-end RL runs of all three driver modes on CPU with the tiny model: colocated synchronous
(in-process workers, checkpoint + resume), disaggregated asynchronous and the one-off pipelined
synchronous mode (worker processes, gloo bridge group, P2P weight push)."""
import json
import os

import pytest
import torch

from axon_b200.driver.train_agent_ppo import train_agent
from axon_b200.utils.config import compose_config
from axon_b200.utils.state import find_latest_ckpt_path, is_valid_checkpoint


def _config(tmp_path, extra):
    rows = [{"question": f"What is {i}+{i}?", "ground_truth": str(2 * i), "data_source": "toy", "reward_fn": "bernoulli"}
            for i in range(8)]
    data = tmp_path / "train.jsonl"
    with open(data, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    ov = [f"train_files={data}", "model_path=tiny-qwen3", "+force_cpu=true", "train_batch_size=2", "decoding.n=2",
          "mini_batch_size=2", "max_seq_length=256", "max_prompt_length=200", f"output_dir={tmp_path}/out",
          "advantage=grpo", "validation.before_train=false", "+sampler.num_kv_pages=64", "sampler.max_num_seqs=8",
          "max_tokens_per_step=12", "drop_zero_advantage_samples=false", "actor.max_token_len_per_gpu=512",
          "save_programs_flag=false", "logger=[file]", "resume_from_checkpoint=true"] + extra
    os.environ["AXON_FILE_LOGGER_ROOT"] = str(tmp_path)
    return compose_config(ov)


def _logged_steps(tmp_path):
    path = tmp_path / "axon-agent_ppo.jsonl"
    return [json.loads(line) for line in open(path)]


@pytest.mark.timeout(600)
def test_sync_colocated_train_checkpoint_resume(tmp_path):
    cfg = _config(tmp_path, ["num_gpus_per_node=1", "total_training_steps=2", "save_steps=1", "checkpoint_format=both",
                             f"val_files={tmp_path}/train.jsonl"])
    drv = train_agent(cfg, backend="inline", keep_alive=True)
    try:
        assert drv.global_steps == 3
        # colocated sampler generates from the trainer's own parameter buffer
        s_worker = drv.sampler_wg.workers[0].role_objects["sampler"]
        a_worker = drv.sampler_wg.workers[0].role_objects["actor"]
        assert s_worker.shares_trainer_weights and s_worker.model is a_worker.model
        sum_after = a_worker.params_checksum()
        sched = a_worker.engine.sched_step
    finally:
        drv.shutdown()
    logs = _logged_steps(tmp_path)
    assert [r["step"] for r in logs][:2] == [1, 2] and "val/reward" in logs[-1]["data"]
    first = logs[0]["data"]
    for key in ("actor/loss", "actor/grad_norm", "batch/sampler_logprobs_diff_mean", "critic/rewards/mean", "timing_s/gen",
                "timing_s/forward_backward", "response_length/mean", "perf/throughput_tokens_per_s", "engine/returned_programs"):
        assert key in first, key
    assert first["batch/sampler_logprobs_diff_mean"] < 1e-4            # sampler and trainer agree on log-probs
    ckpt_root = tmp_path / "out" / "axon" / "agent_ppo" / "checkpoints"
    latest = find_latest_ckpt_path(str(ckpt_root))
    assert latest.endswith("step_2") and is_valid_checkpoint(latest)
    assert os.path.exists(os.path.join(latest, "actor", "huggingface", "model.safetensors"))
    # resume: one more step; parameters and schedule continue from the checkpoint
    cfg2 = _config(tmp_path, ["num_gpus_per_node=1", "total_training_steps=3", "save_steps=-1", "checkpoint_format=both"])
    drv2 = train_agent(cfg2, backend="inline", keep_alive=True)
    try:
        a2 = drv2.sampler_wg.workers[0].role_objects["actor"]
        assert drv2.global_steps == 4 and a2.engine.sched_step == sched + 1 and a2.engine.opt_step >= 3
        assert abs(a2.params_checksum() - sum_after) < 1.0 and a2.params_checksum() != sum_after
    finally:
        drv2.shutdown()
    assert [r["step"] for r in _logged_steps(tmp_path)][-1] == 3


@pytest.mark.timeout(900)
@pytest.mark.parametrize("mode", ["async", "oneoff"])
def test_disaggregated_modes_push_weights(tmp_path, mode):
    extra = ["num_gpus_per_node=2", "hybrid_engine=false", "total_training_steps=2", "save_steps=-1"]
    if mode == "oneoff":
        extra += ["enable_one_off_pipeline=true", "driver_mode=sync"]
    drv = train_agent(_config(tmp_path, extra), backend="process", keep_alive=True)
    try:
        assert drv.global_steps == 3
        a, s = drv.actor_wg.params_checksum()[0], drv.sampler_wg.params_checksum()[0]
        assert a == s                                   # the last push made the sampler's weights bit-identical
    finally:
        drv.shutdown()
    logs = _logged_steps(tmp_path)
    assert [r["step"] for r in logs] == [1, 2]
    assert "timing_s/sync_weights" in logs[0]["data"] and "actor/loss" in logs[1]["data"]
    if mode == "async":
        assert "async/staleness_steps" in logs[0]["data"]


@pytest.mark.timeout(900)
@pytest.mark.parametrize("model", ["dense", "moe", "dense-4", "moe-tp-ep-trainer", "dense-tp-trainer", "dense-pp-trainer", "dense-pp-sampler"])
def test_disaggregated_with_a_tensor_parallel_sampler_group(tmp_path, model):
    """1 trainer + a sampler group of 2 ranks that shard the model: the weight push re-slices every tensor for the
    group's ranks, the group generates in lockstep behind its first rank, and what it samples has the log-probs the
    trainer computes for the same tokens."""
    extra = ["num_gpus_per_node=3", "sampler_trainer_gpu_ratio=2", "hybrid_engine=false", "total_training_steps=2", "save_steps=-1",
             "sampler.tensor_model_parallel_size=2"]
    if model == "dense-4":      # a group of 4 for a model with 2 key / value heads: the push sends each head to the two ranks that hold it
        extra = ["num_gpus_per_node=5", "sampler_trainer_gpu_ratio=4", "hybrid_engine=false", "total_training_steps=2", "save_steps=-1",
                 "sampler.tensor_model_parallel_size=4"]
    if model == "moe-tp-ep-trainer":    # two trainer ranks as one tensor + expert parallel group push to one whole-model sampler
        extra = ["num_gpus_per_node=3", "sampler_trainer_gpu_ratio=0.5", "hybrid_engine=false", "total_training_steps=2", "save_steps=-1",
                 "actor.megatron.tensor_model_parallel_size=2", "actor.megatron.expert_model_parallel_size=2"]
    if model == "dense-pp-sampler":     # the sampler group is cut into two pipeline stages: each receives its own layers
        extra = [e for e in extra if not e.startswith("sampler.tensor_model_parallel_size")] + ["sampler.pipeline_model_parallel_size=2"]
    if model in ("dense-tp-trainer", "dense-pp-trainer"):
        # two trainer ranks as one tensor-parallel group / as two pipeline stages feed one whole-model sampler; the asynchronous
        # driver hands the SAME rows to the ranks of such a group and each stage pushes its own layers
        dim = "tensor_model_parallel_size" if model == "dense-tp-trainer" else "pipeline_model_parallel_size"
        extra = ["num_gpus_per_node=3", "sampler_trainer_gpu_ratio=0.5", "hybrid_engine=false", "total_training_steps=2", "save_steps=-1",
                 "strategy=megatron", f"actor.megatron.{dim}=2"]
    if model == "moe":          # asked for as an expert-parallel size alone: the same group of two
        extra = [e for e in extra if not e.startswith("sampler.tensor_model_parallel_size")] + ["sampler.expert_parallel_size=2"]
    if model.startswith("moe"):  # the group also divides the experts; the routed experts it records are replayed by the trainer
        extra += ["model_path=tiny-moe", "strategy=megatron", "moe_replay=true"]
    drv = train_agent(_config(tmp_path, extra), backend="process", keep_alive=True)
    try:
        assert drv.global_steps == 3
        assert len(drv.server_addresses) == 1           # the group is reached through its first rank
    finally:
        drv.shutdown()
    logs = _logged_steps(tmp_path)
    assert [r["step"] for r in logs] == [1, 2]
    for r in logs:
        assert abs(r["data"]["batch/sampler_logprobs_diff_max"]) < 0.02 and abs(r["data"]["batch/sampler_logprobs_diff_min"]) < 0.02, r["data"]


@pytest.mark.timeout(900)
@pytest.mark.parametrize("model,shards", [("tiny-gemma3", True), ("tiny-qwen3", True), ("tiny-qwen3", False)])
def test_colocated_run_on_two_worker_processes(tmp_path, model, shards):
    """Two colocated ranks, each a worker process that holds the trainer and the sampler role. With parameter shards (a
    family model cut layer by layer / the dense model cut by rows) each sampler holds a whole replica that is refreshed
    from the gathered tensors before every rollout; without, it reads the trainer's buffer. Either way what it samples
    has the trainer's log-probs."""
    extra = ["num_gpus_per_node=2", "total_training_steps=2", "save_steps=-1", f"model_path={model}",
             f"actor.fsdp.param_sharding={'true' if shards else 'false'}"]
    drv = train_agent(_config(tmp_path, extra), backend="process", keep_alive=True)
    try:
        assert drv.global_steps == 3
    finally:
        drv.shutdown()
    logs = _logged_steps(tmp_path)
    assert [r["step"] for r in logs] == [1, 2]
    for r in logs:
        assert abs(r["data"]["batch/sampler_logprobs_diff_max"]) < 0.02 and abs(r["data"]["batch/sampler_logprobs_diff_min"]) < 0.02, r["data"]


@pytest.mark.timeout(900)
@pytest.mark.parametrize("model", ["dense", "moe", "dense-critic"])
def test_colocated_tensor_parallel_trainer_and_sampler_share_their_shards(tmp_path, model):
    """Two colocated ranks form ONE tensor-parallel group for both roles (sparse model: it also divides the experts):
    the sampler group reads the trainer's shards in place, generates in lockstep behind its first rank, and what it
    samples has the trainer's log-probs - also after the optimizer step."""
    extra = ["num_gpus_per_node=2", "total_training_steps=2", "save_steps=-1", "strategy=megatron",
             "actor.megatron.tensor_model_parallel_size=2", "sampler.tensor_model_parallel_size=2"]
    if model == "moe":
        extra += ["model_path=tiny-moe", "actor.megatron.expert_model_parallel_size=2", "moe_replay=true"]
    if model == "dense-critic":         # PPO with a value model that is tensor-parallel too
        extra += ["critic.enable=true", "advantage=gae", "critic.megatron.tensor_model_parallel_size=2"]
    drv = train_agent(_config(tmp_path, extra), backend="process", keep_alive=True)
    try:
        assert drv.global_steps == 3
        assert len(drv.server_addresses) == 1
    finally:
        drv.shutdown()
    logs = _logged_steps(tmp_path)
    assert [r["step"] for r in logs] == [1, 2]
    for r in logs:
        assert abs(r["data"]["batch/sampler_logprobs_diff_max"]) < 0.02 and abs(r["data"]["batch/sampler_logprobs_diff_min"]) < 0.02, r["data"]
        assert model != "dense-critic" or "critic/vf_loss" in r["data"] or any(k.startswith("critic/") for k in r["data"]), sorted(r["data"])[:40]


@pytest.mark.timeout(900)
@pytest.mark.parametrize("layout", ["pp2-sampler-dp", "tp2-sampler-dp", "pp2-sampler-tp2", "pp2xtp2ep2-sampler-tp2", "dp2-sampler-pp2"])
def test_colocated_sampler_next_to_a_trainer_with_another_layout(tmp_path, layout):
    """The trainer's shards are not what the sampler reads (pipeline stages; tensor-parallel shards next to whole-model
    sampler replicas; a sparse pipeline x tensor x expert trainer next to tensor-parallel sampler groups): every sampler
    keeps weights of its own, refreshed before each rollout from the tensors the trainer's model-parallel group gathers,
    and what it samples has the trainer's log-probs."""
    extra = ["total_training_steps=2", "save_steps=-1", "strategy=megatron", "model_path=tiny-qwen3-untied"]
    if layout == "pp2-sampler-dp":
        extra += ["num_gpus_per_node=2", "actor.megatron.pipeline_model_parallel_size=2"]
    elif layout == "tp2-sampler-dp":
        extra += ["num_gpus_per_node=2", "actor.megatron.tensor_model_parallel_size=2"]
    elif layout == "dp2-sampler-pp2":           # a data-parallel trainer next to a sampler group cut into two pipeline stages
        extra = [e for e in extra if e != "strategy=megatron"] + ["num_gpus_per_node=2", "sampler.pipeline_model_parallel_size=2"]
    elif layout == "pp2-sampler-tp2":
        extra += ["num_gpus_per_node=2", "actor.megatron.pipeline_model_parallel_size=2", "sampler.tensor_model_parallel_size=2"]
    else:
        extra = [e for e in extra if not e.startswith("model_path")]
        extra += ["num_gpus_per_node=4", "model_path=tiny-moe", "moe_replay=true", "actor.megatron.pipeline_model_parallel_size=2",
                  "actor.megatron.tensor_model_parallel_size=2", "actor.megatron.expert_model_parallel_size=2",
                  "sampler.tensor_model_parallel_size=2"]
    drv = train_agent(_config(tmp_path, extra), backend="process", keep_alive=True)
    try:
        assert drv.global_steps == 3
    finally:
        drv.shutdown()
    logs = _logged_steps(tmp_path)
    assert [r["step"] for r in logs] == [1, 2]
    for r in logs:
        assert abs(r["data"]["batch/sampler_logprobs_diff_max"]) < 0.02 and abs(r["data"]["batch/sampler_logprobs_diff_min"]) < 0.02, r["data"]
