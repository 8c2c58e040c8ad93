"""Policy/value loss registry. ``compute_loss_fn(data, name, args)`` first applies the sampler
importance-sampling / rejection / veto correction when any of ``sampler_is``, ``sampler_rs`` or
``sampler_token_veto_threshold`` is configured and ``sampler_log_probs`` is in the batch, then calls
the registered ``fn(data, config) -> (loss, metrics)`` (reference: axon/trainer/algos/loss/registry.py)."""
from __future__ import annotations

from enum import Enum

from ....utils.registry import FunctionRegistry, FunctionRegistryEntry

LossRegistryEntry = FunctionRegistryEntry


class LossFn(str, Enum):
    PPO = "ppo"
    GSPO = "gspo"
    GPG = "gpg"
    CLIP_COV = "clip_cov"
    KL_COV = "kl_cov"
    GEO_MEAN = "geo_mean"
    CISPO = "cispo"
    REINFORCE = "reinforce"
    VALUE = "value"


_loss_registry: FunctionRegistry = FunctionRegistry(name="policy loss")


def register_loss(name_or_enum):
    return _loss_registry.register(name_or_enum)


def get_loss_entry(name_or_enum) -> LossRegistryEntry:
    return _loss_registry.get_entry(name_or_enum)


def get_loss_fn(name_or_enum):
    return _loss_registry.get_fn(name_or_enum)


def compute_loss_fn(data, loss_fn: str, loss_fn_args: dict | None = None):
    args = loss_fn_args if loss_fn_args is not None else {}
    fn = _loss_registry.get_fn(loss_fn)
    extra = {}
    wants_correction = any(args.get(k) is not None for k in ("sampler_is", "sampler_rs", "sampler_token_veto_threshold"))
    if wants_correction and "sampler_log_probs" in data.batch:
        from ....utils.rl.sampler import compute_sampler_correction_and_add_to_batch
        data, extra = compute_sampler_correction_and_add_to_batch(data, args)
    loss, metrics = fn(data, args)
    metrics.update(extra)
    return loss, metrics
