"""Worker roles of an RL job (reference: axon/core/role.py)."""
from __future__ import annotations

from enum import Enum


class Role(Enum):
    Actor = "actor"
    Sampler = "sampler"
    ActorSampler = "actor_sampler"
    Critic = "critic"
    RefPolicy = "ref"
    RewardModel = "reward_model"
    ActorSamplerRef = "actor_sampler_ref"

    def __str__(self) -> str:
        return self.value

    @classmethod
    def from_string(cls, name: str) -> "Role":
        key = name.lower().replace("-", "_")
        aliases = {"ref_policy": cls.RefPolicy, "rm": cls.RewardModel, "trainer": cls.Actor}
        for r in cls:
            if r.value == key or r.name.lower() == key:
                return r
        if key in aliases:
            return aliases[key]
        raise ValueError(f"unknown role '{name}'. Known: {[r.value for r in cls]}")

    @property
    def is_trainable(self) -> bool:
        return self in (Role.Actor, Role.ActorSampler, Role.ActorSamplerRef, Role.Critic)
