"""Training entry point: configuration -> worker classes -> resource pools -> driver
(reference: axon/driver/train_agent_ppo.py:41-357).

Worker classes are synthesised at run time from a base worker plus the mixins the deployment needs
(``type(name, (*mixins, base), {})``): colocated mode switching for the hybrid engine, P2P weight push
for disaggregated pools, and the asynchronous data path for ``AsyncPPO``. Worker processes are local
children of this process (one per GPU), launched by the controller with the NCCL / CUDA environment
below; there is no cluster scheduler in the loop.

Runs as ``python -m axon_b200.driver.train_agent_ppo --run-id <id>`` (the CLI's detached launch) or
through ``run_ppo_agent(config)``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from ..core.resource_pool import split_trainer_sampler_pools
from ..core.role import Role
from ..utils.config import Config
from .driver_utils import RoleWorkerConfig

# Environment of every worker process. One hardware queue per process keeps kernel order equal to
# launch order (needed by the overlap logic); NVLS stays on (in-switch reduction); the NCCL CTA
# budget is left to NCCL because our own fused kernels carry the bandwidth-critical paths.
_ENV_VARS = {
    "CUDA_DEVICE_MAX_CONNECTIONS": "1",
    "TOKENIZERS_PARALLELISM": "false",
    "NCCL_P2P_LEVEL": "NVL",
    "NCCL_RAS_ENABLE": "0",
    "TORCH_NCCL_AVOID_RECORD_STREAMS": "1",
    "TORCH_NCCL_ASYNC_ERROR_HANDLING": "1",
    "PYTHONUNBUFFERED": "1",
}


def _get_dynamic_env_vars(config) -> dict[str, str]:
    env = {"AXON_MOE_REPLAY": str(int(bool(config.get("moe_replay", False)))),
           "AXON_ENABLE_MTP": os.environ.get("AXON_ENABLE_MTP", "0"),
           "LD_LIBRARY_PATH": os.environ.get("LD_LIBRARY_PATH", "")}
    if torch.cuda.is_available():
        env["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    return env


def _preprocess_role_configs(config: Config) -> None:
    """Copy the shared fields into every role's sub-config so a worker needs only its own sub-tree."""
    for role in ("actor", "ref", "critic", "reward_model", "sampler"):
        sub = config.get(role)
        if sub is None:
            continue
        if role in ("actor", "ref", "sampler") or not sub.get("model_path"):
            sub["model_path"] = config.get("model_path")
        sub["trust_remote_code"] = config.get("trust_remote_code", False)
        sub["external_lib"] = config.get("external_lib", None)
        sub["global_profiler"] = config.get("global_profiler", None)
        sub["seed"] = config.get("seed", 42)
        if config.get("force_cpu", False):
            sub["force_cpu"] = True
    config["sampler"]["lora_rank"] = (config["actor"].get("lora", {}) or {}).get("rank", 0)
    config["sampler"]["max_model_len"] = config["sampler"].get("max_model_len") or config.get("max_seq_length")


def _build_resource_pools(config, disaggregated: bool):
    pools = split_trainer_sampler_pools(int(config.get("num_nodes", 1)), int(config.get("num_gpus_per_node", 1)),
                                        config.get("sampler_trainer_gpu_ratio", 1), hybrid=not disaggregated)
    if not disaggregated:
        return pools["global"], pools["global"]
    return pools["trainer"], pools["sampler"]


def _synthesize(name: str, base, mixins: list):
    from ..controller.worker_group import synthesize_class
    return synthesize_class(name, base, tuple(mixins))


def build_role_worker_mapping(config, is_async: bool):
    """Role -> (worker class, pool, kwargs) for the chosen strategy and deployment."""
    from ..sampler.sampler import SamplerWorker
    strategy = str(config.get("strategy", "fsdp"))
    hybrid = bool(config.get("hybrid_engine", True))
    disagg = not hybrid
    if strategy in ("fsdp", "fsdp2"):
        from ..trainer.fsdp_trainer import RewardModel, TrainerWorker, ValueModel
    elif strategy == "megatron":
        from ..trainer.megatron_trainer import RewardModel, TrainerWorker, ValueModel
    else:
        raise ValueError(f"unknown strategy '{strategy}' (expected fsdp or megatron)")
    t_mixins, s_mixins = [], []
    if hybrid:
        from ..sampler.mixins.sync_mixin import SyncSamplerMixin
        from ..trainer.mixins.sync_mixin import SyncTrainerMixin
        t_mixins.append(SyncTrainerMixin)
        s_mixins.append(SyncSamplerMixin)
    if disagg or is_async:
        from ..sampler.mixins.p2p_mixin import SamplerP2PMixin
        from ..trainer.mixins.p2p_mixin import TrainerP2PMixin
        t_mixins.append(TrainerP2PMixin)
        s_mixins.append(SamplerP2PMixin)
    if is_async:
        from ..sampler.mixins.async_mixin import AsyncSamplerMixin
        from ..trainer.mixins.async_mixin import AsyncTrainerMixin
        t_mixins.append(AsyncTrainerMixin)
        s_mixins.append(AsyncSamplerMixin)
    actor_cls = _synthesize("ActorWorker", TrainerWorker, t_mixins)
    sampler_cls = _synthesize("SamplerRoleWorker", SamplerWorker, s_mixins)
    actor_pool, sampler_pool = _build_resource_pools(config, disagg)
    sampler_cfg = config if is_async else {**{k: config.get(k) for k in ("model_path", "seed", "force_cpu", "global_profiler", "max_seq_length", "moe_replay")},
                                            "sampler": config["sampler"]}
    mapping = {
        Role.Actor: RoleWorkerConfig(actor_cls, actor_pool, {"config": config["actor"], "name": "actor"}),
        Role.Sampler: RoleWorkerConfig(sampler_cls, sampler_pool, {"config": sampler_cfg, "name": "sampler"}),
    }
    critic_on = config.get("critic", {}).get("enable")
    if critic_on is None:
        critic_on = str(config.get("advantage", "")) in ("gae", "chunked_gae")
    if critic_on:
        mapping[Role.Critic] = RoleWorkerConfig(TrainerWorker, actor_pool, {"config": config["critic"], "model": ValueModel, "name": "critic"})
    loss_args = config.get("loss_args", {}) or {}
    if float(loss_args.get("kl_coef", 0) or 0) > 0 or config.get("kl_reward"):
        mapping[Role.RefPolicy] = RoleWorkerConfig(TrainerWorker, actor_pool, {"config": config["ref"], "name": "ref"})
    if (config.get("reward_model", {}) or {}).get("enable", False):
        mapping[Role.RewardModel] = RoleWorkerConfig(TrainerWorker, actor_pool, {"config": config["reward_model"], "model": RewardModel,
                                                                                  "name": "reward_model"})
    return mapping


def train_agent(config: Config, backend: str | None = None, keep_alive: bool = False):
    """Build everything and run. Returns the driver after ``train_rl`` finished; with ``keep_alive`` the
    workers stay up (the caller shuts the driver down)."""
    from ..utils.tokenizer import hf_tokenizer
    from .async_ppo import AsyncPPO
    from .sync_ppo import SyncPPO
    _preprocess_role_configs(config)
    tokenizer = hf_tokenizer(config.get("model_path"), trust_remote_code=bool(config.get("trust_remote_code", False)))
    mode = config.get("driver_mode")
    if mode is None:
        mode = "sync" if config.get("hybrid_engine", True) or config.get("enable_one_off_pipeline", False) else "async"
    is_async = mode == "async"
    if is_async and config.get("hybrid_engine", True):
        raise ValueError("the asynchronous driver needs disaggregated pools (hybrid_engine=false)")
    if not config.get("hybrid_engine", True):
        config["sampler"]["serve_http"] = True if (backend or "process") == "process" else config["sampler"].get("serve_http", False)
    mapping = build_role_worker_mapping(config, is_async)
    backend = backend or str(config.get("worker_backend", "process"))
    if backend == "process":
        os.environ.update({k: v for k, v in {**_ENV_VARS, **_get_dynamic_env_vars(config)}.items() if k not in os.environ})
        if config.get("hybrid_engine", True):
            config["sampler"]["serve_http"] = True
    driver_cls = AsyncPPO if is_async else SyncPPO
    driver = driver_cls(config, tokenizer, mapping, processor=None, backend=backend)
    try:
        driver.init_workers()
        driver.train_rl()
    except BaseException:
        driver.shutdown()
        raise
    if not keep_alive:
        driver.shutdown()
    return driver


def eval_agent(config: Config, backend: str | None = None):
    config["mode"] = "eval"
    return train_agent(config, backend)


def run_ppo_agent(config: Config, backend: str | None = None):
    from ..config.validate_config import validate_axon_config
    validate_axon_config(config)
    if config.get("mode", "train") == "eval":
        return eval_agent(config, backend)
    return train_agent(config, backend)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="axon_b200.driver.train_agent_ppo")
    ap.add_argument("--run-id", default=None, help="run registered by the CLI; its stored config is used")
    ap.add_argument("--config-json", default=None, help="path of a resolved configuration (JSON)")
    ap.add_argument("overrides", nargs="*")
    args = ap.parse_args(argv)
    from ..utils.config import compose_config
    if args.config_json:
        cfg = Config(json.load(open(args.config_json)))
    else:
        cfg = compose_config(args.overrides)
    if args.run_id:
        from ..cli import _runs
        _runs.set_status(args.run_id, "running")
    status = "failed"
    try:
        run_ppo_agent(cfg)
        status = "finished"
        return 0
    finally:
        if args.run_id:
            from ..cli import _runs
            _runs.set_status(args.run_id, status)


if __name__ == "__main__":
    sys.exit(main())
