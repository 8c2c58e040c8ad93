"""Single-turn math environment: one question, one answer, scored by the math reward function
(reference: recipes/math/env.py)."""
from __future__ import annotations

from axon_b200.core.env import SingleTurnEnvironment, register_env
from axon_b200.utils.rewards import REWARD_FN_REGISTRY


@register_env("math")
class MathEnvironment(SingleTurnEnvironment):
    @staticmethod
    def from_dict(env_args: dict) -> "SingleTurnEnvironment":
        env_args = dict(env_args)
        reward_fn = env_args.pop("reward_fn", None) or REWARD_FN_REGISTRY["math"]
        return SingleTurnEnvironment(task=env_args, reward_fn=reward_fn)
