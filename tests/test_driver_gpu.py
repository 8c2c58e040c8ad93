"""The full driver on real GPUs: ``train_agent`` -> SyncPPO -> worker groups -> Engine -> prefix tree ->
ReactProgram -> sampler engine -> trainer, with the tiny head-dim-128 model. One GPU: colocated synchronous mode
with checkpoint and resume. Two GPUs: disaggregated mode, where the trainer -> sampler weight push has to go
through the peer-store plan kernel (CUDA IPC mapping of the sampler's live weights), not through messages."""
import json
import os

import pytest
import torch

from axon_b200.utils.config import compose_config


def _n_gpus():
    try:
        return torch.cuda.device_count()
    except Exception:  # noqa: BLE001
        return 0


def _config(tmp_path, extra):
    rows = [{"question": f"What is {i}+{i}?", "ground_truth": str(2 * i), "data_source": "toy", "reward_fn": "bernoulli"}
            for i in range(8)]
    data = tmp_path / "train.jsonl"
    with open(data, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    ov = [f"train_files={data}", "model_path=tiny-gpu", "train_batch_size=2", "decoding.n=2",
          "mini_batch_size=2", "max_seq_length=512", "max_prompt_length=256", f"output_dir={tmp_path}/out",
          "advantage=grpo", "validation.before_train=false", "+sampler.num_kv_pages=64", "sampler.max_num_seqs=8",
          "max_tokens_per_step=24", "drop_zero_advantage_samples=false", "actor.max_token_len_per_gpu=1024",
          "save_programs_flag=false", "logger=[file]", "resume_from_checkpoint=true"] + extra
    os.environ["AXON_FILE_LOGGER_ROOT"] = str(tmp_path)
    return compose_config(ov)


def _logged_steps(tmp_path):
    return [json.loads(line) for line in open(tmp_path / "axon-agent_ppo.jsonl")]


@pytest.mark.gpu
@pytest.mark.timeout(900)
def test_sync_colocated_driver_on_gpu_with_resume(tmp_path):
    from axon_b200.driver.train_agent_ppo import train_agent
    from axon_b200.ops import _common as C
    from axon_b200.utils.state import find_latest_ckpt_path, is_valid_checkpoint
    launches0 = C.LAUNCH_COUNT
    cfg = _config(tmp_path, ["num_gpus_per_node=1", "total_training_steps=2", "save_steps=1", "checkpoint_format=both"])
    drv = train_agent(cfg, backend="inline", keep_alive=True)
    try:
        assert drv.global_steps == 3
        a_worker = drv.sampler_wg.workers[0].role_objects["actor"]
        s_worker = drv.sampler_wg.workers[0].role_objects["sampler"]
        assert a_worker.device.type == "cuda" and s_worker.shares_trainer_weights
        # the small KV pool fits beside the optimizer state, so the mode switch leaves that state on the device
        assert a_worker.rollout_kept_optimizer is True and a_worker.engine.master is not None
        checksum, sched = a_worker.params_checksum(), a_worker.engine.sched_step
    finally:
        drv.shutdown()
    assert C.LAUNCH_COUNT > launches0, "the driver ran without launching a native kernel"
    logs = _logged_steps(tmp_path)
    assert [r["step"] for r in logs][:2] == [1, 2]
    first = logs[0]["data"]
    for key in ("actor/loss", "actor/grad_norm", "batch/sampler_logprobs_diff_mean", "timing_s/gen", "timing_s/forward_backward"):
        assert key in first, key
    assert first["batch/sampler_logprobs_diff_mean"] < 5e-3           # bf16 sampler and trainer kernels agree on log-probs
    latest = find_latest_ckpt_path(str(tmp_path / "out" / "axon" / "agent_ppo" / "checkpoints"))
    assert latest.endswith("step_2") and is_valid_checkpoint(latest)
    cfg2 = _config(tmp_path, ["num_gpus_per_node=1", "total_training_steps=3", "save_steps=-1", "checkpoint_format=both"])
    drv2 = train_agent(cfg2, backend="inline", keep_alive=True)
    try:
        a2 = drv2.sampler_wg.workers[0].role_objects["actor"]
        assert drv2.global_steps == 4 and a2.engine.sched_step == sched + 1
        assert abs(a2.params_checksum() - checksum) < 5.0 and a2.params_checksum() != checksum
    finally:
        drv2.shutdown()
    C.check_status()


@pytest.mark.gpu
@pytest.mark.timeout(900)
@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_disaggregated_driver_pushes_weights_with_the_peer_store_kernel(tmp_path):
    from axon_b200.driver.train_agent_ppo import train_agent
    extra = ["num_gpus_per_node=2", "hybrid_engine=false", "total_training_steps=2", "save_steps=-1",
             "enable_one_off_pipeline=true", "driver_mode=sync"]
    drv = train_agent(_config(tmp_path, extra), backend="process", keep_alive=True)
    try:
        assert drv.global_steps == 3
        a, s = drv.actor_wg.params_checksum()[0], drv.sampler_wg.params_checksum()[0]
        assert a == s                                   # the last push made the sampler's weights bit-identical
        sync = drv.last_weight_sync
        assert all(r["transport"] == "peer-store kernel" and r["bytes"] > 0 for r in sync), sync
    finally:
        drv.shutdown()
    logs = _logged_steps(tmp_path)
    assert [r["step"] for r in logs] == [1, 2]
    assert logs[0]["data"]["sync/peer_store_kernel"] == 1.0 and "timing_s/sync_weights" in logs[0]["data"]


@pytest.mark.gpu
@pytest.mark.timeout(900)
@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_colocated_driver_on_two_gpus_as_worker_processes(tmp_path):
    """Two worker processes, each holding the trainer AND the sampler role of its GPU: the optimizer state is sharded over
    the two ranks, every sampler reads its trainer's parameter buffer in place, and the replicas stay equal."""
    from axon_b200.driver.train_agent_ppo import train_agent
    extra = ["num_gpus_per_node=2", "total_training_steps=2", "save_steps=-1"]
    drv = train_agent(_config(tmp_path, extra), backend="process", keep_alive=True)
    try:
        assert drv.global_steps == 3
        sums = drv.actor_wg.params_checksum()
        assert len(sums) == 2 and sums[0] == sums[1], sums
        assert len(drv.server_addresses) == 2
    finally:
        drv.shutdown()
    logs = _logged_steps(tmp_path)
    assert [r["step"] for r in logs] == [1, 2]
    assert logs[0]["data"]["batch/sampler_logprobs_diff_mean"] < 5e-3 and "actor/grad_norm" in logs[1]["data"]
