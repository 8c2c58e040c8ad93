"""Config composition / interpolation / validation and the CLI + run registry."""
import json
import os
import time

import pytest
from click.testing import CliRunner

from axon_b200.cli import _runs, build_overrides, main
from axon_b200.config.validate_config import (needs_critic, needs_reference_policy, validate_axon_config)
from axon_b200.utils.config import Config, ConfigError, compose_config, flatten_yaml_to_overrides, omega_conf_to_dataclass


def test_compose_grafts_templates_and_resolves():
    cfg = compose_config()
    for role in ("actor", "ref", "critic", "reward_model"):
        assert cfg[role].optimizer_args.weight_decay == 0.1
    assert cfg.critic.optimizer_args.lr == 1e-5 and cfg.actor.optimizer_args.lr == 1e-6
    assert cfg.sampler.max_model_len == cfg.max_seq_length == 8192
    assert cfg.critic.forward_max_token_len_per_gpu == 32768          # ${.max_token_len_per_gpu}
    assert cfg.ref.forward_only is True and cfg.ref.strategy == "fsdp"
    assert cfg.actor.forward_max_token_len_per_gpu == 16384           # oc.select with an existing key
    validate_axon_config(cfg)


def test_overrides_and_errors():
    cfg = compose_config(["max_seq_length=4096", "+program.env_name=math", "++actor.fsdp.new_knob=3", "~kl_reward",
                          "loss_args.clip_ratio_high=0.28", "logger=[console,file]"])
    assert cfg.max_seq_length == 4096 and cfg.sampler.max_model_len == 4096 and cfg.program.env_name == "math"
    assert cfg.actor.fsdp.new_knob == 3 and "kl_reward" not in cfg and cfg.logger == ["console", "file"]
    with pytest.raises(ConfigError):
        compose_config(["no_such_key=1"])
    with pytest.raises(ConfigError):
        compose_config(["+max_seq_length=1"])
    c = Config({"a": {"b": 1}, "c": "${a.b}", "d": "x-${a.b}"})
    from axon_b200.utils.config import resolve
    resolve(c)
    assert c.c == 1 and c.d == "x-1" and c.select("a.b") == 1 and c.select("a.z", 7) == 7
    assert flatten_yaml_to_overrides({"a": {"b": [1, 2]}, "c": None}) == ["++a.b=[1, 2]", "++c=null"]


def test_dataclass_conversion():
    from axon_b200.trainer.policy import OptimConfig
    oc = omega_conf_to_dataclass(Config({"lr": 3e-4, "grad_clip": 0.5}), OptimConfig)
    assert oc.lr == 3e-4 and oc.grad_clip == 0.5 and oc.beta2 == 0.95
    with pytest.raises(ConfigError):
        omega_conf_to_dataclass({"bogus": 1}, OptimConfig)


@pytest.mark.parametrize("ov,msg", [
    (["advantage=nope"], "adv_estimator"), (["loss_args.token_reduce=median"], "token_reduce"),
    (["max_prompt_length=9000"], "max_prompt_length"), (["moe_replay=true"], "moe_replay"),
    (["moe_replay=true", "strategy=megatron", "sampler.enable_prefix_caching=true"], "prefix_caching"),
    (["loss_args.sampler_rs=token"], "sampler_rs_threshold"), (["driver_mode=async"], "hybrid_engine"),
    (["actor.use_dynamic_bsz=false"], "micro_batch_size"), (["actor.max_token_len_per_gpu=1024"], "max_token_len_per_gpu"),
    (["mini_batch_size=128"], "mini_batch_size"), (["strategy=deepspeed"], "strategy"),
    (["strategy=megatron", "actor.megatron.tensor_model_parallel_size=3"], "tp*pp*cp"),
    (["hybrid_engine=false", "driver_mode=async", "advantage=gae"], "critic"),
    (["sampler.tensor_model_parallel_size=2", "sampler.pipeline_model_parallel_size=2"], "not both"),
    (["sampler.tensor_model_parallel_size=2", "sampler.expert_parallel_size=4"], "expert_parallel_size"),
    (["moe_replay=true", "strategy=megatron", "sampler.pipeline_model_parallel_size=2"], "pipelined group"),
])
def test_validation_rejects(ov, msg):
    with pytest.raises(ValueError, match=msg.replace("*", r"\*")):
        validate_axon_config(compose_config(ov))


def test_role_requirements():
    assert not needs_reference_policy(compose_config()) and not needs_critic(compose_config())
    assert needs_reference_policy(compose_config(["loss_args.kl_coef=0.01"]))
    assert needs_reference_policy(compose_config(["kl_reward=low_var_kl"]))
    assert needs_critic(compose_config(["advantage=gae"])) and not needs_critic(compose_config(["advantage=gae", "critic.enable=false"]))


def test_cli_dry_run_and_registry(tmp_path, monkeypatch):
    monkeypatch.setenv("AXON_RUNS_DIR", str(tmp_path / "runs"))
    r = CliRunner()
    y = tmp_path / "exp.yaml"
    y.write_text("train_batch_size: 128\nloss_args:\n  clip_ratio: 0.3\n")
    out = r.invoke(main, ["train", "-c", str(y), "--model", "tiny-qwen3", "--gpus", "2", "--dry-run", "--", "mini_batch_size=32"])
    assert out.exit_code == 0, out.output
    assert "train_batch_size: 128" in out.output and "model_path: tiny-qwen3" in out.output and "mini_batch_size: 32" in out.output
    bad = r.invoke(main, ["train", "--dry-run", "--", "advantage=nope"])
    assert bad.exit_code != 0 and "invalid configuration" in bad.output
    assert build_overrides(None, {"gpus": 4, "resume": False}, ("a=1",)) == ["++num_gpus_per_node=4", "++resume_from_checkpoint=False", "a=1"]
    assert "no runs" in r.invoke(main, ["status"]).output
    m1 = _runs.create_run("config", "exp-a")
    m2 = _runs.create_run("config", "exp-b", pid=2 ** 22 + 12345)       # a pid that does not exist
    assert len(m1["run_id"]) == 8 and _runs.read_meta(m1["run_id"])["status"] == "running"
    assert _runs.read_meta(m2["run_id"])["status"] == "crashed"        # lazily flipped
    assert _runs.resolve_run_id(m1["run_id"][:5]) == m1["run_id"]
    with pytest.raises(KeyError):
        _runs.resolve_run_id("zzzz")
    with _runs.tee_to_file(m1["log_path"]):
        print("hello from the run")
    lst = r.invoke(main, ["status"]).output
    assert m1["run_id"] in lst and "crashed" in lst
    assert "hello from the run" in r.invoke(main, ["logs", m1["run_id"][:4], "-n", "5"]).output
    assert "exp-a" in r.invoke(main, ["status", m1["run_id"]]).output
    assert "nothing to cancel" in r.invoke(main, ["cancel", m2["run_id"]]).output
