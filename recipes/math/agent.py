"""Math agent: asks for step-by-step reasoning with the final answer in ``\\boxed{}``; on a second turn (when the
environment allows one) asks the model to re-check its answer (reference: recipes/math/agent.py)."""
from __future__ import annotations

from typing import Any

from axon_b200.core.agent import Action, BaseAgent, register_agent

INSTRUCTION = "Let's think step by step, and put your final answer within \\boxed{}."
RETRY = "Your previous answer may or may not contain a mistake. Please review it carefully and put your final answer within \\boxed{}."


@register_agent("math")
class MathAgent(BaseAgent):
    def __init__(self, instruction: str = INSTRUCTION):
        self.instruction = instruction
        self.reset()

    def reset(self) -> None:
        self.first = True

    def process_observation(self, observation: Any, reward: float, done: bool, info: dict, **kwargs) -> str:
        if self.first:
            self.first = False
            question = observation["question"] if isinstance(observation, dict) else str(observation)
            return f"{question} {self.instruction}"
        return RETRY

    def process_action(self, action: str) -> Action:
        return Action(action=action)
