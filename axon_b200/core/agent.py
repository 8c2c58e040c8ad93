"""Agent base classes used by ReAct-style programs: prompt construction and response parsing
(reference: axon/core/agent.py)."""
from __future__ import annotations

from abc import ABC
from dataclasses import dataclass
from typing import Any

from ..utils.registry import ClassRegistry

AGENT_CLASS_MAPPING: ClassRegistry = ClassRegistry("agent")
register_agent = AGENT_CLASS_MAPPING.register


@dataclass
class Action:
    """A parsed model response: the reasoning trace and the action handed to the environment."""
    thought: str = ""
    action: Any = None


class BaseAgent(ABC):
    @property
    def system_prompt(self) -> str:
        return ""

    def reset(self) -> None:
        return None

    def process_observation(self, observation: Any, reward: float, done: bool, info: dict, **kwargs) -> Any:
        raise NotImplementedError("BaseAgent.process_observation must be implemented")

    def process_action(self, action: str) -> Action:
        raise NotImplementedError("BaseAgent.process_action must be implemented")


def split_thought(text: str) -> tuple[str, str]:
    """(thought, rest) around a ``</think>`` marker; no marker means no thought."""
    if "</think>" in text:
        head, _, tail = text.partition("</think>")
        return head.replace("<think>", "").strip(), tail.strip()
    return "", text.strip()


@register_agent("default")
class DefaultAgent(BaseAgent):
    """Pass-through: the observation text is the user message, the raw response is the action."""

    def process_observation(self, observation, reward, done, info, **kwargs):
        if isinstance(observation, dict):
            for key in ("question", "prompt", "observation", "content"):
                if key in observation:
                    return observation[key]
            return str(observation)
        return observation

    def process_action(self, action: str) -> Action:
        thought, rest = split_thought(action)
        return Action(thought=thought, action=rest)
