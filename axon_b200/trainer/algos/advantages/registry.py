"""Advantage-estimator registry (reference: axon/trainer/algos/advantages/registry.py).
Registered functions have the signature ``fn(data: DataProto, config) -> (advantages, returns)``."""
from __future__ import annotations

from enum import Enum

from ....utils.registry import FunctionRegistry, FunctionRegistryEntry

AdvantageRegistryEntry = FunctionRegistryEntry


class AdvantageFn(str, Enum):
    GAE = "gae"
    GRPO = "grpo"
    RLOO = "rloo"
    LOOP = "loop"
    REINFORCE_PLUS_PLUS = "reinforce_plus_plus"
    REINFORCE_PLUS_PLUS_BASELINE = "reinforce_plus_plus_baseline"
    REMAX = "remax"
    OPO = "opo"
    GRPO_PASSK = "grpo_passk"
    GPG = "gpg"
    CHUNKED_GAE = "chunked_gae"
    KIMI_K1_5 = "kimi_k1_5"
    IDENTITY = "identity"


_advantage_registry: FunctionRegistry = FunctionRegistry(name="advantage estimator")


def register_advantage(name_or_enum):
    return _advantage_registry.register(name_or_enum)


def get_advantage_entry(name_or_enum) -> AdvantageRegistryEntry:
    return _advantage_registry.get_entry(name_or_enum)


def get_advantage_fn(name_or_enum):
    return _advantage_registry.get_fn(name_or_enum)
