"""``compute_advantage(data, config)``: look up ``config.advantage`` in the registry, call it with
``config.advantage_args`` and store ``advantages`` / ``returns`` on the batch
(reference: axon/trainer/algos/advantages/__init__.py)."""
from __future__ import annotations

from enum import Enum

import torch

from . import advantage as _advantage  # noqa: F401  (registers the estimators)
from .registry import (AdvantageFn, AdvantageRegistryEntry, _advantage_registry, get_advantage_entry,
                       get_advantage_fn, register_advantage)


def _cfg_get(cfg, key, default=None):
    if cfg is None:
        return default
    if isinstance(cfg, dict):
        return cfg.get(key, default)
    return getattr(cfg, key, default)


def compute_advantage(data, config=None):
    name = _cfg_get(config, "advantage")
    if name is None:
        raise ValueError("config must name the estimator in its 'advantage' field")
    name = name.value if isinstance(name, Enum) else name
    args = _cfg_get(config, "advantage_args") or {}
    adv, ret = _advantage_registry.compute(name, data, args)
    if args.get("clip_advantages", False):
        adv = torch.clamp(adv, -1, 1)
    data.batch["advantages"] = adv
    data.batch["returns"] = ret
    return data


__all__ = ["AdvantageFn", "AdvantageRegistryEntry", "register_advantage", "get_advantage_entry",
           "get_advantage_fn", "compute_advantage"]
