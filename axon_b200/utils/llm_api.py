"""Calls to external judge / reward LLMs over OpenAI-compatible chat endpoints
(reference: axon/utils/llm_api.py:29-177). Endpoints and keys come from the environment
(``OPENAI_BASE_URL`` / ``OPENAI_API_KEY``); nothing is contacted at import time."""
from __future__ import annotations

import os
import time


def call_oai_rm_llm(prompt: str, system_prompt: str = "", n: int = 1, temperature: float = 1.0, model_id: str = "gpt-4o-mini",
                    retry_count: int = 5, base_url: str | None = None, api_key: str | None = None, timeout: float = 120.0) -> list[str]:
    """``n`` chat completions for (system, user); returns their texts ([] after exhausting the retries)."""
    import httpx
    base = (base_url or os.environ.get("OPENAI_BASE_URL", "https://api.openai.com/v1")).rstrip("/")
    key = api_key or os.environ.get("OPENAI_API_KEY", "")
    body = {"model": model_id, "n": n, "temperature": temperature,
            "messages": ([{"role": "system", "content": system_prompt}] if system_prompt else []) + [{"role": "user", "content": prompt}]}
    delay = 1.0
    for _ in range(retry_count):
        try:
            r = httpx.post(base + "/chat/completions", json=body, headers={"Authorization": f"Bearer {key}"}, timeout=timeout)
            if r.status_code == 429:
                time.sleep(delay)
                delay = min(delay * 2, 60.0)
                continue
            r.raise_for_status()
            return [c["message"]["content"] for c in r.json()["choices"]]
        except Exception:                             # noqa: BLE001
            time.sleep(delay)
            delay = min(delay * 2, 60.0)
    return []


def call_gemini_llm(prompt: str, system_prompt: str = "", n: int = 1, temperature: float = 1.0, model_id: str = "gemini-1.5-pro",
                    retry_count: int = 5, **kw) -> list[str]:
    """Gemini through its OpenAI-compatible endpoint (``GEMINI_API_KEY``)."""
    return call_oai_rm_llm(prompt, system_prompt, n, temperature, model_id, retry_count,
                           base_url=os.environ.get("GEMINI_BASE_URL", "https://generativelanguage.googleapis.com/v1beta/openai"),
                           api_key=os.environ.get("GEMINI_API_KEY", ""), **kw)
