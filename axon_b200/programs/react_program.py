"""``ReactProgram``: agent -> action -> environment -> observation, repeated until the environment
reports done or the engine stops the program (truncation, step limit). The data row selects the
environment and agent classes by registered name; an unknown ``env_name`` is treated as the name of a
reward function for a single-turn environment (reference: axon/programs/react_program.py:37-262)."""
from __future__ import annotations

from copy import deepcopy
from typing import Any

from ..core.agent import AGENT_CLASS_MAPPING, Action, DefaultAgent
from ..core.env import ENV_CLASS_MAPPING, SingleTurnEnvironment
from ..utils.module_loader import load_class
from .base_program import BaseProgram, ProgramResult, register_program


def _as_list(v, n):
    if isinstance(v, list):
        assert len(v) == n, f"expected {n} entries, got {len(v)}"
        return [dict(x or {}) for x in v]
    return [dict(v or {}) for _ in range(n)]


def _resolve(mapping, name):
    """Registered name, or 'path/file.py:Class' / 'pkg.module:Class' loaded and registered on the fly."""
    if name in mapping:
        return mapping[name]
    if ":" in name:
        cls = load_class(name)
        mapping.register(name, cls, override=True)
        return cls
    return mapping[name]


@register_program("react")
class ReactProgram(BaseProgram):
    def __init__(self, agent_name: str | list = "default", env_name: str | list = "single_turn",
                 agent_args: dict | list | None = None, env_args: dict | list | None = None,
                 accumulate_thinking: bool = True, accumulate_history: bool = True, group_id: str = "",
                 sample_params: dict | None = None, endpoint_url: str = "", retry_limit: int = 1,
                 program_timeout: int = 10800):
        super().__init__(group_id=group_id, sample_params=sample_params, endpoint_url=endpoint_url,
                         retry_limit=retry_limit, program_timeout=program_timeout)
        self.accumulate_thinking, self.accumulate_history = accumulate_thinking, accumulate_history
        envs = [env_name] if isinstance(env_name, str) else list(env_name)
        agents = [agent_name] if isinstance(agent_name, str) else list(agent_name)
        assert len(envs) == len(agents), f"env_name/agent_name length mismatch: {len(envs)} vs {len(agents)}"
        self._env_defaults, self._agent_defaults = {}, {}
        for en, an, ea, aa in zip(envs, agents, _as_list(env_args, len(envs)), _as_list(agent_args, len(envs))):
            self._env_defaults[_resolve(ENV_CLASS_MAPPING, en)] = ea
            self._agent_defaults[_resolve(AGENT_CLASS_MAPPING, an)] = aa
        self.env_class, self.agent_class = _resolve(ENV_CLASS_MAPPING, envs[0]), _resolve(AGENT_CLASS_MAPPING, agents[0])
        self.env_name = envs[0] if len(envs) == 1 else envs
        self.agent_name = agents[0] if len(agents) == 1 else agents
        self.env_args = env_args if isinstance(env_args, dict) else {}
        self.messages: list = []

    def init_env_and_agent(self):
        args = dict(self.env_args)
        env_name, agent_name = args.pop("env_name", None), args.pop("agent_name", None)
        env_cls = self.env_class if env_name is None and self.env_class is not None else None
        if env_name:
            if env_name in ENV_CLASS_MAPPING:
                env_cls = ENV_CLASS_MAPPING[env_name]
            else:
                env_cls = SingleTurnEnvironment
                args.setdefault("reward_fn", env_name)
        if env_cls is None:
            env_cls = SingleTurnEnvironment
        agent_cls = None
        for name in (agent_name, env_name):
            if name is not None and name in AGENT_CLASS_MAPPING:
                agent_cls = AGENT_CLASS_MAPPING[name]
                break
        if agent_cls is None:
            agent_cls = self.agent_class if agent_name is None and env_name is None else DefaultAgent
        self.env = env_cls.from_dict({**self._env_defaults.get(env_cls, {}), **args})
        self.agent = agent_cls(**self._agent_defaults.get(agent_cls, {}))
        return self.env, self.agent

    def format_messages(self, messages: list[dict]) -> list[dict]:
        messages = deepcopy(messages)
        if not self.accumulate_thinking:
            for m in messages:
                if m["role"] == "assistant" and isinstance(m.get("content"), str):
                    _, sep, after = m["content"].partition("</think>")
                    if sep:
                        m["content"] = after
        if not self.accumulate_history and len(messages) > 1:
            return [messages[0], messages[-1]]
        return messages

    def add_observation_to_messages(self, observation: Any) -> None:
        if isinstance(observation, list) and all(isinstance(x, dict) for x in observation):
            self.messages.extend(observation)
        else:
            self.messages.append({"role": "user", "content": observation})

    def add_action_to_messages(self, action: Any) -> None:
        self.messages.append({"role": "assistant", "content": action})

    async def run(self) -> ProgramResult:
        self.init_env_and_agent()
        self.agent.reset()
        obs, info = self.env.reset()
        first = self.agent.process_observation(observation=obs, reward=0.0, done=False, info=info)
        sys_prompt = self.agent.system_prompt
        self.messages = [{"role": "system", "content": sys_prompt}] if sys_prompt else []
        self.add_observation_to_messages(first)
        steps, reward, done = 0, 0.0, False
        while not done:
            text, stop_program, _ = await self.generate(messages=self.format_messages(self.messages),
                                                        sample_params=self.sample_params)
            self.add_action_to_messages(text)
            action: Action = self.agent.process_action(text)
            obs, reward, done, info = self.env.step(action.action)
            done = done or stop_program
            steps += 1
            self.add_observation_to_messages(self.agent.process_observation(observation=obs, reward=reward, done=done, info=info))
        if hasattr(self.env, "post_compute_reward"):
            reward = self.env.post_compute_reward()
        self.env.close()
        return ProgramResult(reward=reward, done=done, metadata={"steps": steps})
