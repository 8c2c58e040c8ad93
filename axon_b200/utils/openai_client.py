"""Async client helpers for OpenAI-compatible ``/v1/completions`` servers
(reference: axon/utils/openai_client.py:26-228).

``poll_completions_openai`` posts one request with exponential back-off; a response whose finish
reason says the request was aborted (server paused for a weight update) is retried without using up
an attempt. ``fetch_responses_from_addresses`` fans a control call out to several servers.
"""
from __future__ import annotations

import asyncio
import base64
import io
from typing import Any


def pil_to_b64_png(img) -> str:
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    return base64.b64encode(buf.getvalue()).decode("ascii")


def serialize_images_for_http(images: list[Any]) -> list[dict]:
    out = []
    for im in images or []:
        if isinstance(im, dict):
            out.append(im)
        elif isinstance(im, str):
            out.append({"type": "image_url", "image_url": {"url": im}})
        else:
            out.append({"type": "image_url", "image_url": {"url": "data:image/png;base64," + pil_to_b64_png(im)}})
    return out


def load_images(items: list[Any]) -> list[Any]:
    """The inverse of ``serialize_images_for_http``: PIL images from PIL images, ``data:`` URLs, file paths / ``file://``
    URLs and OpenAI ``image_url`` items (remote URLs are refused: a sampler does not fetch from the network)."""
    import base64
    import io
    from PIL import Image
    out = []
    for it in items or []:
        if isinstance(it, dict):
            it = (it.get("image_url") or {}).get("url") if it.get("type") == "image_url" else it.get("url") or it.get("image")
        if isinstance(it, str):
            if it.startswith("data:"):
                out.append(Image.open(io.BytesIO(base64.b64decode(it.split(",", 1)[1]))).convert("RGB"))
            elif it.startswith(("http://", "https://")):
                raise ValueError("remote image URLs are not fetched by the sampler; send a data: URL")
            else:
                out.append(Image.open(it[len("file://"):] if it.startswith("file://") else it).convert("RGB"))
        else:
            out.append(it)
    return out


def _url(address: str, path: str) -> str:
    base = address if address.startswith("http") else f"http://{address}"
    return base.rstrip("/") + path


async def poll_completions_openai(address: str, timeout: int = 2700, max_retries: int = 3, **request) -> dict:
    import httpx
    for k in ("meta_info", "extra_headers"):
        request.pop(k, None)
    if request.get("image_data"):
        request["image_data"] = serialize_images_for_http(request["image_data"])
    delay, attempt, last = 1.0, 0, None
    while attempt < max_retries:
        try:
            async with httpx.AsyncClient(timeout=httpx.Timeout(timeout)) as client:
                r = await client.post(_url(address, "/v1/completions"), json=request)
            if r.status_code != 200:
                raise RuntimeError(f"completions request failed with status {r.status_code}: {r.text[:500]}")
            result = r.json()
            if any("abort" in (c.get("finish_reason") or "").lower() for c in result.get("choices", [])):
                await asyncio.sleep(delay)            # paused server: wait, do not count the attempt
                delay = min(delay * 2, 30.0)
                continue
            return result
        except Exception as e:                        # noqa: BLE001
            last = e
            attempt += 1
            if attempt < max_retries:
                await asyncio.sleep(delay)
                delay = min(delay * 2, 30.0)
    raise RuntimeError(f"all {max_retries} attempts failed: {last}") from last


async def _call_api(address: str, endpoint: str, payload: dict | None = None, timeout: int = 300, max_retries: int = 3):
    import httpx
    delay, last = 1.0, None
    for attempt in range(max_retries):
        try:
            async with httpx.AsyncClient(timeout=httpx.Timeout(timeout)) as client:
                r = await client.post(_url(address, endpoint), json=payload or {})
            r.raise_for_status()
            return r.json() if r.content else {}
        except Exception as e:                        # noqa: BLE001
            last = e
            if attempt < max_retries - 1:
                await asyncio.sleep(delay)
                delay *= 2
    raise RuntimeError(f"{endpoint} on {address} failed: {last}") from last


async def fetch_responses_from_addresses(addresses: list[str], endpoint: str, payload: dict | None = None, timeout: int = 300,
                                         max_retries: int = 3) -> list:
    return list(await asyncio.gather(*(_call_api(a, endpoint, payload, timeout, max_retries) for a in addresses)))
