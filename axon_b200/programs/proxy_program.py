"""``ProxyProgram``: the rollout logic lives in an external service. The program starts a job there
(POST ``proxy_url`` with the engine's callback ``server_url`` and the session id), the service drives
the conversation through the engine's HTTP routes (``/generate``, ``/end_session``), and the program
polls the engine until the session is marked done (reference: axon/programs/proxy_program.py:25-260)."""
from __future__ import annotations

import asyncio
from typing import Any

from .base_program import BaseProgram, ProgramResult, register_program


@register_program("proxy")
class ProxyProgram(BaseProgram):
    def __init__(self, proxy_url: str, proxy_token: str = "", server_url: str = "", env_args: dict | None = None,
                 poll_interval: float = 1.0, start_retries: int = 3, **kw):
        super().__init__(**kw)
        self.proxy_url, self.proxy_token, self.server_url = proxy_url, proxy_token, server_url
        self.env_args = env_args or {}
        self.poll_interval, self.start_retries = poll_interval, start_retries
        self.external_session_id: str | None = None

    def _prepare_reset_payload(self) -> dict[str, Any]:
        return {**self.env_args, "session_id": self.session_id, "server_url": self.server_url or self.endpoint_url,
                "sample_params": self.sample_params, "group_id": self.group_id}

    async def _start_program_with_retry(self, payload: dict) -> dict:
        headers = {"Authorization": f"Bearer {self.proxy_token}"} if self.proxy_token else {}
        last = None
        for attempt in range(self.start_retries):
            try:
                r = await self._get_http_client().post(self.proxy_url, json=payload, headers=headers)
                r.raise_for_status()
                return r.json()
            except Exception as e:  # noqa: BLE001
                last = e
                await asyncio.sleep(min(2 ** attempt, 10))
        raise last

    @staticmethod
    def _extract_session_id(data: dict) -> str:
        for k in ("sessionId", "session_id", "id"):
            if data.get(k):
                return str(data[k])
        raise RuntimeError(f"no session id in the service response: {data}")

    async def _session_done(self) -> bool:
        if self.engine is not None:
            st = self.engine.session_state_map.get(self.session_id)
            return st is None or st.done
        d = await self._post("/session_status", {"session_id": self.session_id})
        return bool(d.get("done", False))

    async def run(self) -> ProgramResult:
        data = await self._start_program_with_retry(self._prepare_reset_payload())
        self.external_session_id = self._extract_session_id(data)
        while not await self._session_done():
            await asyncio.sleep(self.poll_interval)
        return ProgramResult(reward=0, done=True, metadata={"external_session_id": self.external_session_id})

    async def _run_program_inner(self, sample_params):
        # the external service ends the session itself (with the real reward); do not overwrite it
        await self.init_session(group_id=self.group_id, sample_params=sample_params)
        return await self.run()
