"""Fail-fast validation of a composed run configuration (reference: axon/config/validate_config.py:423-502).

``validate_axon_config(cfg)`` runs the section validators (data, algorithm, loss, actor, ref, critic,
reward model, sampler) and the cross-section rules, raising ``ValueError`` with the offending key.
``needs_reference_policy`` / ``needs_critic`` tell the driver which roles to start.
"""
from __future__ import annotations

from typing import Any

VALID_ADV_ESTIMATORS = {"gae", "grpo", "rloo", "loop", "reinforce_plus_plus", "reinforce_plus_plus_baseline", "remax",
                        "opo", "grpo_passk", "gpg", "chunked_gae", "identity", "kimi_k1_5"}
VALID_LOSSES = {"ppo", "gspo", "gpg", "clip_cov", "kl_cov", "geo_mean", "cispo", "reinforce", "value"}
VALID_KL_PENALTIES = {"kl", "k1", "abs", "mse", "k2", "low_var_kl", "k3", "full", "k1+", "k3+"}
VALID_KL_TYPES = {"fixed", "adaptive"}
VALID_SAMPLER_IS = {None, "token", "sequence"}
VALID_SAMPLER_RS = {None, "token", "sequence", "geometric"}
VALID_TOKEN_REDUCE = {"sum", "mean", "mean-norm", "mean-program"}
VALID_BATCH_REDUCE = {"token-mean", "step-mean", "program-mean"}
VALID_PAUSE = {"drain", "hold", "continue", "reset"}
VALID_QUANT = {None, "fp8", "fp8_fast", "int4", "mxfp8"}


def _get(cfg, path: str, default: Any = None) -> Any:
    node = cfg
    for k in path.split("."):
        if isinstance(node, dict) and k in node:
            node = node[k]
        else:
            return default
    return node


def get_effective_strategy(cfg) -> str:
    s = _get(cfg, "actor.strategy") or _get(cfg, "strategy", "fsdp")
    if s not in ("fsdp", "megatron"):
        raise ValueError(f"Invalid strategy: {s}. Must be 'fsdp' or 'megatron'.")
    return s


def is_megatron_strategy(cfg) -> bool:
    return get_effective_strategy(cfg) == "megatron"


def is_fsdp_strategy(cfg) -> bool:
    return get_effective_strategy(cfg) == "fsdp"


def needs_reference_policy(cfg) -> bool:
    """A frozen reference model is needed when a KL term is active in the reward or in the loss."""
    return bool(_get(cfg, "kl_reward")) or float(_get(cfg, "loss_args.kl_coef", 0.0) or 0.0) > 0.0


def needs_critic(cfg) -> bool:
    explicit = _get(cfg, "critic.enable")
    if explicit is not None:
        return bool(explicit)
    return _get(cfg, "advantage") in ("gae", "chunked_gae")


def n_trainer_gpus(cfg) -> int:
    total = int(_get(cfg, "num_nodes", 1)) * int(_get(cfg, "num_gpus_per_node", 8))
    if _get(cfg, "hybrid_engine", True):
        return total
    return max(1, int(total // (float(_get(cfg, "sampler_trainer_gpu_ratio", 1)) + 1)))


def validate_data_config(cfg) -> None:
    mp, ms = _get(cfg, "max_prompt_length", 0), _get(cfg, "max_seq_length", 0)
    if mp is None or mp <= 0:
        raise ValueError("max_prompt_length must be positive.")
    if ms is None or ms <= 0:
        raise ValueError("max_seq_length must be positive.")
    if mp >= ms:
        raise ValueError(f"max_prompt_length ({mp}) must be smaller than max_seq_length ({ms}).")
    if _get(cfg, "prompt_truncation") not in (None, "left", "right"):
        raise ValueError(f"Invalid prompt_truncation: {_get(cfg, 'prompt_truncation')}. Use null, 'left' or 'right'.")
    if _get(cfg, "train_batch_size", 1) <= 0:
        raise ValueError("train_batch_size must be positive.")
    if _get(cfg, "decoding.n", 1) < 1:
        raise ValueError("decoding.n must be >= 1.")


def validate_algorithm_config(cfg) -> None:
    adv = _get(cfg, "advantage")
    if adv not in VALID_ADV_ESTIMATORS:
        raise ValueError(f"Invalid adv_estimator: {adv}. Must be one of {sorted(VALID_ADV_ESTIMATORS)}")
    klr = _get(cfg, "kl_reward")
    if klr is not None and klr not in VALID_KL_PENALTIES:
        raise ValueError(f"Invalid kl_reward: {klr}. Must be null or one of {sorted(VALID_KL_PENALTIES)}")
    if klr is not None:
        t = _get(cfg, "kl_reward_args.type", "fixed")
        if t not in VALID_KL_TYPES:
            raise ValueError(f"Invalid kl_reward_args.type: {t}. Must be one of {sorted(VALID_KL_TYPES)}")
    if adv == "grpo_passk" and _get(cfg, "decoding.n", 1) < 2:
        raise ValueError("advantage=grpo_passk needs decoding.n >= 2.")
    if _get(cfg, "stepwise_advantage_mode", "broadcast") not in ("broadcast", "per_step"):
        raise ValueError(f"Invalid stepwise_advantage_mode: {_get(cfg, 'stepwise_advantage_mode')}")


def validate_loss_config(cfg) -> None:
    if _get(cfg, "loss") not in VALID_LOSSES:
        raise ValueError(f"Invalid loss: {_get(cfg, 'loss')}. Must be one of {sorted(VALID_LOSSES)}")
    a = _get(cfg, "loss_args", {}) or {}
    if a.get("token_reduce", "sum") not in VALID_TOKEN_REDUCE:
        raise ValueError(f"Invalid token_reduce: {a.get('token_reduce')}")
    if a.get("batch_reduce", "token-mean") not in VALID_BATCH_REDUCE:
        raise ValueError(f"Invalid batch_reduce: {a.get('batch_reduce')}")
    if a.get("sampler_is") not in VALID_SAMPLER_IS:
        raise ValueError(f"Invalid loss_args.sampler_is: {a.get('sampler_is')}. Must be one of {VALID_SAMPLER_IS}")
    if a.get("sampler_rs") not in VALID_SAMPLER_RS:
        raise ValueError(f"Invalid loss_args.sampler_rs: {a.get('sampler_rs')}. Must be one of {VALID_SAMPLER_RS}")
    if a.get("sampler_rs") is not None and a.get("sampler_rs_threshold") is None:
        raise ValueError("loss_args.sampler_rs_threshold must be set when loss_args.sampler_rs is enabled.")
    if float(a.get("clip_ratio_c", 3.0)) <= 1.0:
        raise ValueError("loss_args.clip_ratio_c must be > 1.0.")
    if a.get("kl_type", "low_var_kl") not in VALID_KL_PENALTIES:
        raise ValueError(f"Invalid loss_args.kl_type: {a.get('kl_type')}")


def _validate_trainer_section(cfg, section: str, n_gpus: int, trains: bool) -> None:
    sec = _get(cfg, section, {}) or {}
    strategy = sec.get("strategy") or _get(cfg, "strategy", "fsdp")
    if not sec.get("use_dynamic_bsz", True):
        mbs, per = sec.get("micro_batch_size"), sec.get("micro_batch_size_per_gpu")
        if mbs is None and per is None:
            raise ValueError(f"[{section}] Please set at least one of '{section}.micro_batch_size' or "
                             f"'{section}.micro_batch_size_per_gpu'.")
        if mbs is not None and per is not None:
            raise ValueError(f"[{section}] '{section}.micro_batch_size' and '{section}.micro_batch_size_per_gpu' "
                             "are mutually exclusive.")
    elif (sec.get("max_token_len_per_gpu") or 0) < _get(cfg, "max_seq_length", 0):
        raise ValueError(f"[{section}] max_token_len_per_gpu ({sec.get('max_token_len_per_gpu')}) must be >= "
                         f"max_seq_length ({_get(cfg, 'max_seq_length')}).")
    if trains:
        tb, mb = _get(cfg, "train_batch_size", 1), _get(cfg, "mini_batch_size", 1)
        if tb < mb:
            raise ValueError(f"train_batch_size ({tb}) must be >= mini_batch_size ({mb})")
    if strategy == "fsdp":
        sp = int(_get(sec, "fsdp.ulysses_sequence_parallel_size", 1) or 1)
        if sp > 1 and not _get(sec, "fsdp.use_remove_padding", True):
            raise ValueError(f"[{section}] sequence parallelism requires fsdp.use_remove_padding.")
        if n_gpus % sp != 0:
            raise ValueError(f"[{section}] ulysses_sequence_parallel_size ({sp}) must divide the trainer GPUs ({n_gpus}).")
        fs = int(_get(sec, "fsdp.fsdp_size", -1) or -1)
        if fs > 0 and n_gpus % fs != 0:
            raise ValueError(f"[{section}] fsdp_size ({fs}) must divide the trainer GPUs ({n_gpus}).")
    else:
        m = sec.get("megatron", {}) or {}
        tp, pp, cp = int(m.get("tensor_model_parallel_size", 1)), int(m.get("pipeline_model_parallel_size", 1)), \
            int(m.get("context_parallel_size", 1))
        if n_gpus % (tp * pp * cp) != 0:
            raise ValueError(f"[{section}] tp*pp*cp ({tp * pp * cp}) must divide the trainer GPUs ({n_gpus}).")
        ep = int(m.get("expert_model_parallel_size", 1))
        if (n_gpus // pp) % ep != 0:
            raise ValueError(f"[{section}] expert_model_parallel_size ({ep}) must divide GPUs per pipeline stage.")
    if int(_get(sec, "lora.rank", 0) or 0) > 512:
        raise ValueError("LoRA rank must be less than or equal to 512")


def validate_actor_config(cfg, n_gpus: int) -> None:
    _validate_trainer_section(cfg, "actor", n_gpus, trains=True)


def validate_ref_config(cfg, n_gpus: int) -> None:
    if needs_reference_policy(cfg):
        _validate_trainer_section(cfg, "ref", n_gpus, trains=False)


def validate_critic_config(cfg, n_gpus: int) -> None:
    if needs_critic(cfg):
        _validate_trainer_section(cfg, "critic", n_gpus, trains=True)


def validate_reward_model_config(cfg) -> None:
    if _get(cfg, "reward_model.enable", False) and not _get(cfg, "reward_model.model_path"):
        raise ValueError("reward_model.enable is set but reward_model.model_path is empty.")


def validate_sampler_config(cfg) -> None:
    s = _get(cfg, "sampler", {}) or {}
    if s.get("quantization") not in VALID_QUANT:
        raise ValueError(f"Invalid sampler.quantization: {s.get('quantization')}. Must be one of {VALID_QUANT}")
    if not 0.0 < float(s.get("gpu_memory_utilization", 0.85)) <= 1.0:
        raise ValueError("sampler.gpu_memory_utilization must be in (0, 1].")
    if _get(cfg, "moe_replay", False) and s.get("enable_prefix_caching", False):
        raise ValueError("moe_replay requires sampler.enable_prefix_caching=false: cached prefixes carry no routing record.")
    if _get(cfg, "sampler_pausing_strategy", "continue") not in VALID_PAUSE:
        raise ValueError(f"Invalid sampler_pausing_strategy: {_get(cfg, 'sampler_pausing_strategy')}")
    if _get(cfg, "sampler_channel", "nccl") not in ("nccl", "ray"):
        raise ValueError(f"Invalid sampler_channel: {_get(cfg, 'sampler_channel')}")
    if (s.get("max_model_len") or 0) and s["max_model_len"] < _get(cfg, "max_seq_length", 0):
        raise ValueError("sampler.max_model_len must be >= max_seq_length.")
    tp, pp, ep = (int(s.get(k, 1) or 1) for k in ("tensor_model_parallel_size", "pipeline_model_parallel_size", "expert_parallel_size"))
    if tp > 1 and pp > 1:
        raise ValueError("a sampler group is tensor-parallel or cut into pipeline stages, not both "
                         f"(sampler.tensor_model_parallel_size={tp}, sampler.pipeline_model_parallel_size={pp}).")
    if ep > 1 and tp > 1 and ep != tp:
        raise ValueError(f"sampler.expert_parallel_size ({ep}) must equal sampler.tensor_model_parallel_size ({tp}): a group divides "
                         "its experts over its own ranks.")
    if pp > 1 and _get(cfg, "moe_replay", False):
        raise ValueError("moe_replay needs a tensor-parallel sampler group or whole replicas: routed experts are not gathered over "
                         "the stages of a pipelined group.")


def _validate_cross_section_consistency(cfg) -> None:
    mode = _get(cfg, "driver_mode")
    if mode not in (None, "sync", "async"):
        raise ValueError(f"Invalid driver_mode: {mode}. Must be null, 'sync' or 'async'.")
    hybrid = _get(cfg, "hybrid_engine", True)
    if mode == "async" and hybrid:
        raise ValueError("driver_mode=async needs hybrid_engine=false (disaggregated trainer and sampler pools).")
    if mode == "async" or (mode is None and not hybrid and not _get(cfg, "enable_one_off_pipeline", False)):
        if needs_critic(cfg) or needs_reference_policy(cfg):
            raise ValueError("the async driver supports neither a critic nor a reference policy / KL reward.")
    if _get(cfg, "enable_one_off_pipeline", False) and hybrid:
        raise ValueError("enable_one_off_pipeline needs hybrid_engine=false.")
    if _get(cfg, "moe_replay", False):
        if not is_megatron_strategy(cfg):
            raise ValueError("moe_replay requires strategy=megatron.")
        if _get(cfg, "actor.megatron.virtual_pipeline_model_parallel_size"):
            raise ValueError("moe_replay does not support virtual pipeline parallelism.")
    if not hybrid and int(_get(cfg, "num_nodes", 1)) * int(_get(cfg, "num_gpus_per_node", 8)) < 2:
        raise ValueError("disaggregated mode needs at least 2 GPUs.")
    if _get(cfg, "checkpoint_format", "hf") not in ("sharded", "hf", "both"):
        raise ValueError(f"Invalid checkpoint_format: {_get(cfg, 'checkpoint_format')}")
    if _get(cfg, "mode", "train") not in ("train", "eval"):
        raise ValueError(f"Invalid mode: {_get(cfg, 'mode')}")


def validate_axon_config(cfg) -> None:
    get_effective_strategy(cfg)
    n = n_trainer_gpus(cfg)
    validate_data_config(cfg)
    validate_sampler_config(cfg)
    validate_algorithm_config(cfg)
    validate_loss_config(cfg)
    validate_actor_config(cfg, n)
    validate_ref_config(cfg, n)
    validate_critic_config(cfg, n)
    validate_reward_model_config(cfg)
    _validate_cross_section_consistency(cfg)


def print_config_summary(cfg) -> str:
    lines = ["Run configuration:",
             f"  model          {_get(cfg, 'model_path')}",
             f"  strategy       {get_effective_strategy(cfg)}  hybrid={_get(cfg, 'hybrid_engine')}  "
             f"gpus={_get(cfg, 'num_nodes')}x{_get(cfg, 'num_gpus_per_node')} (trainer {n_trainer_gpus(cfg)})",
             f"  algorithm      loss={_get(cfg, 'loss')} advantage={_get(cfg, 'advantage')} n={_get(cfg, 'decoding.n')}",
             f"  batch          train={_get(cfg, 'train_batch_size')} mini={_get(cfg, 'mini_batch_size')} "
             f"seq={_get(cfg, 'max_seq_length')} prompt={_get(cfg, 'max_prompt_length')}",
             f"  roles          ref={needs_reference_policy(cfg)} critic={needs_critic(cfg)} rm={_get(cfg, 'reward_model.enable', False)}"]
    text = "\n".join(lines)
    print(text)
    return text
