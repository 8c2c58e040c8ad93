"""``BaseProgram``: the rollout abstraction. A program decides when to call the model, what to do with
each response and when to stop; the engine records every token it generates. Subclass, implement the
async ``run()`` returning a ``ProgramResult``, and register with ``@register_program("name")``.

``run_program()`` wraps ``run()`` with session handling, a wall-clock timeout and retries; a program
that fails every attempt ends its session with reward -1e99 so the batch builder drops it
(reference: axon/programs/base_program.py:28-270). The engine is reached in-process or over HTTP.
"""
from __future__ import annotations

import asyncio
import traceback
from dataclasses import dataclass, field

from ..utils.registry import ClassRegistry

PROGRAM_CLASS_MAPPING: ClassRegistry = ClassRegistry("program")
register_program = PROGRAM_CLASS_MAPPING.register

FAILED_PROGRAM_REWARD = -1e99


@dataclass
class ProgramResult:
    reward: float
    done: bool
    metadata: dict = field(default_factory=dict)
    step_rewards: dict = field(default_factory=dict)


class BaseProgram:
    def __init__(self, group_id: str = "", sample_params: dict | None = None, endpoint_url: str = "",
                 retry_limit: int = 1, program_timeout: int = 10800):
        self.group_id = group_id
        self.sample_params = sample_params or {}
        self.endpoint_url = endpoint_url
        self.retry_limit = retry_limit
        self.program_timeout = program_timeout
        self.session_id = None
        self.engine = None
        self._http_client = None

    def set_sample_params(self, sample_params: dict) -> None:
        self.sample_params.update(sample_params)

    def set_engine(self, engine) -> None:
        self.engine = engine

    def set_endpoint_url(self, endpoint_url: str) -> None:
        self.endpoint_url = endpoint_url

    def set_group_id(self, group_id: str) -> None:
        self.group_id = group_id

    @property
    def api_base_url(self) -> str:
        return self.endpoint_url

    def _get_http_client(self):
        if self._http_client is None:
            import httpx
            self._http_client = httpx.AsyncClient(timeout=httpx.Timeout(3600.0, connect=5.0),
                                                  limits=httpx.Limits(max_connections=100, max_keepalive_connections=20))
        return self._http_client

    async def _close_http_client(self) -> None:
        if self._http_client is not None:
            await self._http_client.aclose()
            self._http_client = None

    async def _post(self, route: str, payload: dict) -> dict:
        r = await self._get_http_client().post(f"{self.api_base_url}{route}", json=payload)
        r.raise_for_status()
        return r.json()

    async def init_session(self, group_id: str | None = None, sample_params: dict | None = None):
        if self.session_id is not None:
            return self.session_id
        if self.engine:
            self.session_id = await self.engine.run_in_engine_loop_async(self.engine.init_session(group_id, sample_params))
        else:
            self.session_id = (await self._post("/init_session", {"group_id": group_id, "sample_params": sample_params}))["session_id"]
        return self.session_id

    async def generate(self, messages: list[dict], sample_params: dict | None = None, parser_kwargs: dict | None = None):
        """Returns (response_text, stop_program, step_idx)."""
        sample_params = sample_params or {}
        if self.engine:
            return await self.engine.run_in_engine_loop_async(
                self.engine.generate(messages, session_id=self.session_id, sample_params=sample_params,
                                     parser_kwargs=parser_kwargs))
        assert not parser_kwargs, f"parser_kwargs not supported in API server mode yet: {parser_kwargs}"
        d = await self._post("/generate", {"messages": messages, "session_id": self.session_id, "sample_params": sample_params})
        return d["response"], d["stop_program"], d.get("step_idx", -1)

    async def end_session(self, reward: float, step_rewards: dict | None = None):
        if self.engine:
            return await self.engine.run_in_engine_loop_async(
                self.engine.end_session(self.session_id, reward=reward, step_rewards=step_rewards))
        payload = {"session_id": self.session_id, "reward": reward}
        if step_rewards:
            payload["step_rewards"] = {str(k): v for k, v in step_rewards.items()}
        return await self._post("/end_session", payload)

    async def run_program(self):
        """Run with retries and timeout; after the last failed attempt the session is closed with the
        failure reward and the last exception is re-raised."""
        self._http_client = None
        last_exc: BaseException | None = None
        try:
            for attempt in range(max(1, self.retry_limit)):
                if attempt > 0:
                    if self.session_id is not None:      # close the abandoned attempt so its group can complete
                        await self.end_session(reward=FAILED_PROGRAM_REWARD)
                    self.session_id = None
                try:
                    return await asyncio.wait_for(self._run_program_inner(self.sample_params), timeout=self.program_timeout)
                except asyncio.TimeoutError:
                    last_exc = asyncio.TimeoutError(f"Program timed out after {self.program_timeout} seconds")
                except Exception as e:  # noqa: BLE001
                    traceback.print_exc()
                    last_exc = e
            if self.session_id is not None:
                await self.end_session(reward=FAILED_PROGRAM_REWARD)
            raise last_exc
        finally:
            await self._close_http_client()

    async def _run_program_inner(self, sample_params):
        await self.init_session(group_id=self.group_id, sample_params=sample_params)
        result = await self.run()
        await self.end_session(reward=result.reward, step_rewards=result.step_rewards or None)
        return result

    async def run(self) -> ProgramResult:
        raise NotImplementedError("Subclasses must implement this method")
