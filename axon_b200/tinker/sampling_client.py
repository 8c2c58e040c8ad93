"""``SamplingClient``: the rollout side's handle on one or more sampler replicas.

Routes each request to the least-used replica, keeping a session on the replica it first used
(prefix locality), bounds in-flight requests per replica with a semaphore, retries aborted
requests, and fans ``pause_all`` / ``continue_all`` / ``sleep`` / ``wake_up`` out to every replica.
A replica is either an in-process ``SamplerServer`` or the URL of an OpenAI-compatible server
(reference: axon/tinker/sampling_client.py:121-433). ``sample`` returns the reference's dict:
``token_ids, logprobs, token_strs, finish_reasons, stop_reasons, moe_routermap``.
"""
from __future__ import annotations

import asyncio
from typing import Any

from ..sampler.server import decode_routed_experts


class SamplingClient:
    def __init__(self, addresses: list, tokenizer=None, max_concurrency_per_address: int = 1024,
                 max_retries: int = 3, request_timeout: float = 3600.0):
        assert addresses, "at least one sampler address is required"
        self.addresses = list(addresses)
        self.tokenizer = tokenizer
        self.max_retries = max_retries
        self.request_timeout = request_timeout
        self._inflight = [0] * len(self.addresses)
        self._session_addr: dict[str, int] = {}
        self._max_conc = max_concurrency_per_address
        self._sems: dict[int, asyncio.Semaphore] = {}
        self._http = None
        self._paused = False

    # ------------------------------------------------------------------ routing
    def _pick(self, session_id: str | None) -> int:
        if session_id is not None and session_id in self._session_addr:
            return self._session_addr[session_id]
        idx = min(range(len(self.addresses)), key=lambda i: (self._inflight[i], i))
        if session_id is not None:
            self._session_addr[session_id] = idx
        return idx

    def release_session(self, session_id: str) -> None:
        self._session_addr.pop(session_id, None)

    def _sem(self, idx: int) -> asyncio.Semaphore:
        # one semaphore per (address, running loop) so the client works from any event loop
        key = (idx, id(asyncio.get_running_loop()))
        if key not in self._sems:
            self._sems[key] = asyncio.Semaphore(self._max_conc)
        return self._sems[key]

    def _client(self):
        # one HTTP client per running event loop (connections are bound to the loop that opened them)
        import httpx
        if self._http is None:
            self._http = {}
        key = id(asyncio.get_running_loop())
        if key not in self._http:
            self._http[key] = httpx.AsyncClient(timeout=httpx.Timeout(self.request_timeout, connect=5.0))
        return self._http[key]

    # ------------------------------------------------------------------ sampling
    async def _one(self, addr, prompt_ids, params: dict, image_data=None) -> dict:
        if isinstance(addr, str):
            body = {"prompt": list(prompt_ids), "logprobs": 1, "return_token_ids": True, **params}
            if image_data:
                from ..utils.openai_client import serialize_images_for_http
                body["image_data"] = ({k: (v.tolist() if hasattr(v, "tolist") else v) for k, v in image_data.items()}
                                      if isinstance(image_data, dict) else serialize_images_for_http(image_data))
            r = await self._client().post(addr.rstrip("/") + "/v1/completions", json=body)
            r.raise_for_status()
            ch = r.json()["choices"][0]
            return {"token_ids": ch["token_ids"], "logprobs": ch["logprobs"]["token_logprobs"],
                    "token_strs": ch["logprobs"].get("tokens") or [], "finish_reason": ch.get("finish_reason"),
                    "stop_reason": ch.get("stop_reason"), "moe_routermap": decode_routed_experts(ch.get("routed_experts")),
                    "spec_decode_metrics": ch.get("spec_decode_metrics")}
        out = await (addr.generate(prompt_ids, params, image_data) if image_data else addr.generate(prompt_ids, params))
        strs = []
        tok = self.tokenizer or getattr(addr, "tokenizer", None)
        if tok is not None:
            strs = tok.token_strs(out.token_ids) if hasattr(tok, "token_strs") else [tok.decode([t]) for t in out.token_ids]
        return {"token_ids": out.token_ids, "logprobs": out.logprobs, "token_strs": strs,
                "finish_reason": out.finish_reason, "stop_reason": out.stop_reason, "moe_routermap": out.moe_routermap,
                "spec_decode_metrics": out.spec_decode_metrics.to_dict() if getattr(out, "spec_decode_metrics", None) is not None else None}

    async def sample(self, prompt_token_ids, sampling_params: dict | None = None, session_id: str | None = None,
                     image_data=None) -> dict:
        """One completion per call (``n`` > 1 returns lists with n entries)."""
        params = dict(sampling_params or {})
        n = int(params.pop("n", 1))
        idx = self._pick(session_id)
        addr = self.addresses[idx]

        async def run_one():
            acc = {"token_ids": [], "logprobs": [], "token_strs": [], "moe_routermap": None, "spec_decode_metrics": None}
            prompt, p = list(prompt_token_ids), dict(params)
            for _ in range(self.max_retries + 1):
                async with self._sem(idx):
                    self._inflight[idx] += 1
                    try:
                        r = await self._one(addr, prompt, p, image_data)
                    finally:
                        self._inflight[idx] -= 1
                acc["token_ids"] += r["token_ids"]
                acc["logprobs"] += r["logprobs"]
                acc["token_strs"] += r["token_strs"]
                if r["moe_routermap"] is not None:
                    acc["moe_routermap"] = r["moe_routermap"] if acc["moe_routermap"] is None else \
                        __import__("numpy").concatenate([acc["moe_routermap"], r["moe_routermap"]], 0)
                if r.get("spec_decode_metrics"):
                    acc["spec_decode_metrics"] = {k: (acc["spec_decode_metrics"] or {}).get(k, 0) + int(v) for k, v in r["spec_decode_metrics"].items()}
                if r["finish_reason"] != "abort":
                    return {**acc, "finish_reason": r["finish_reason"], "stop_reason": r["stop_reason"]}
                # aborted by a pause(reset): continue from what was generated, with the remaining budget
                prompt = list(prompt_token_ids) + acc["token_ids"]
                if "max_tokens" in p:
                    p["max_tokens"] = max(1, int(params.get("max_tokens", 0)) - len(acc["token_ids"]))
                while self._paused:
                    await asyncio.sleep(0.01)
            return {**acc, "finish_reason": "abort", "stop_reason": None}

        outs = await asyncio.gather(*(run_one() for _ in range(n)))
        return {"token_ids": [o["token_ids"] for o in outs], "logprobs": [o["logprobs"] for o in outs],
                "token_strs": [o["token_strs"] for o in outs], "finish_reasons": [o["finish_reason"] for o in outs],
                "stop_reasons": [o["stop_reason"] for o in outs], "moe_routermap": [o["moe_routermap"] for o in outs],
                "spec_decode_metrics": [o.get("spec_decode_metrics") for o in outs]}

    # ------------------------------------------------------------------ fleet control
    async def _fanout(self, local_call: str, http_path: str, payload: dict | None = None, **kw) -> None:
        async def one(addr):
            if isinstance(addr, str):
                r = await self._client().post(addr.rstrip("/") + http_path, json=payload or {})
                r.raise_for_status()
            else:
                await asyncio.get_running_loop().run_in_executor(None, lambda: getattr(addr, local_call)(**kw))
        await asyncio.gather(*(one(a) for a in self.addresses))

    async def pause_all(self, strategy: str = "drain") -> None:
        self._paused = True
        await self._fanout("pause_generation", "/pause_generation", {"strategy": strategy}, strategy=strategy)

    async def continue_all(self) -> None:
        await self._fanout("continue_generation", "/continue_generation")
        self._paused = False

    async def sleep(self) -> None:
        await self._fanout("sleep", "/sleep")

    async def wake_up(self) -> None:
        await self._fanout("wake_up", "/wake_up")

    def load_statistics(self) -> dict[str, Any]:
        return {"inflight": list(self._inflight), "sessions": len(self._session_addr)}

    async def close(self) -> None:
        if self._http:
            mine = self._http.pop(id(asyncio.get_running_loop()), None)
            if mine is not None:
                await mine.aclose()
            self._http = None
