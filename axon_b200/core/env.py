"""Environment base classes (reference: axon/core/env.py): ``BaseEnv`` (reset/step/close/from_dict),
``MultiTurnEnvironment`` (turn budget + ``get_reward_and_next_obs``) and ``SingleTurnEnvironment``
(one prompt, one response, scored by a function from ``REWARD_FN_REGISTRY``)."""
from __future__ import annotations

import warnings
from abc import ABC, abstractmethod
from typing import Any

from ..utils.registry import ClassRegistry

ENV_CLASS_MAPPING: ClassRegistry = ClassRegistry("environment")
register_env = ENV_CLASS_MAPPING.register


class BaseEnv(ABC):
    @property
    def idx(self) -> Any:
        return getattr(self, "_idx", None)

    @idx.setter
    def idx(self, value: Any):
        self._idx = value

    @abstractmethod
    def reset(self) -> tuple[Any, dict]: ...

    @abstractmethod
    def step(self, action: Any) -> tuple[Any, float, bool, dict]: ...

    def close(self) -> None:
        return None

    @staticmethod
    def from_dict(info: dict) -> "BaseEnv":
        raise NotImplementedError("Subclasses must implement 'from_dict'")

    @staticmethod
    def is_multithread_safe() -> bool:
        return True


class MultiTurnEnvironment(BaseEnv, ABC):
    def __init__(self, task: dict | None = None, max_turns: int = 3, **kwargs):
        self.task = task
        self.max_turns = max_turns
        self.current_turn = 0
        self.done = False
        self.history: list = []

    def reset(self):
        self.done, self.current_turn, self.history = False, 0, []
        return self.task, {}

    def step(self, action):
        self.history.append(action)
        reward, next_obs = self.get_reward_and_next_obs(self.task, action)
        self.current_turn += 1
        if self.current_turn >= self.max_turns:
            self.done = True
            return {}, reward, self.done, self.task
        return next_obs, reward, self.done, self.task

    def get_reward_and_next_obs(self, task: dict, action: Any) -> tuple[float, dict]:
        raise NotImplementedError(f"{type(self).__name__} uses the default step() but does not override "
                                  "get_reward_and_next_obs().")

    @staticmethod
    def from_dict(env_args: dict) -> "MultiTurnEnvironment":
        raise NotImplementedError("Subclasses must implement 'from_dict'")


@register_env("single_turn")
class SingleTurnEnvironment(MultiTurnEnvironment):
    def __init__(self, task: dict | None = None, reward_fn=None, **kwargs):
        super().__init__(task=task, max_turns=1, **kwargs)
        from ..utils.rewards import REWARD_FN_REGISTRY, zero_reward_fn
        if isinstance(reward_fn, str):
            if reward_fn not in REWARD_FN_REGISTRY:
                raise KeyError(f"Unknown reward_fn '{reward_fn}'. Available: {list(REWARD_FN_REGISTRY)}")
            reward_fn = REWARD_FN_REGISTRY[reward_fn]
        if reward_fn is None:
            warnings.warn("No reward function provided, using zero reward", stacklevel=2)
        self.reward_fn = reward_fn or zero_reward_fn

    def get_reward_and_next_obs(self, task: dict, action: Any) -> tuple[float, dict]:
        return self.reward_fn(task_info=task, action=action).reward, {}

    @staticmethod
    def from_dict(env_args: dict) -> "SingleTurnEnvironment":
        env_args = dict(env_args)
        reward_fn = env_args.pop("reward_fn", None)
        task = env_args.get("task", env_args)
        return SingleTurnEnvironment(task=task, reward_fn=reward_fn)
