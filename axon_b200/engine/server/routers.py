"""HTTP front of the engine: the native session routes and an OpenAI-compatible chat route.

  POST /init_session {group_id, sample_params} -> {session_id}
  POST /generate {messages, session_id, sample_params} -> {response, stop_program, step_idx}
  POST /end_session {session_id, reward, step_rewards} ; POST /session_status ; GET /health
  POST /v1/chat/completions  (the session rides in ``user = "axon:<session_id>"``) ; GET /v1/models ;
  POST /tokenize

JSON has no infinity: rewards of +-inf travel as +-1e98 (reference: axon/engine/server/engine_router.py,
oai_router.py)."""
from __future__ import annotations

import math
import time
import uuid

INF_SENTINEL = 1e98


def encode_reward(r: float) -> float:
    if isinstance(r, float) and math.isinf(r):
        return INF_SENTINEL if r > 0 else -INF_SENTINEL
    return r


def decode_reward(r: float) -> float:
    if r >= INF_SENTINEL:
        return float("inf")
    if r <= -INF_SENTINEL:
        return float("-inf")
    return r


def build_engine_app(engine, model_name: str = "axon-policy"):
    from fastapi import FastAPI, HTTPException
    app = FastAPI(title="axon_b200 engine")

    async def on_engine(coro):
        return await engine.run_in_engine_loop_async(coro)

    @app.get("/health")
    async def health():
        return {"status": "ok", "diagnostics": await on_engine(engine.get_session_diagnostics())}

    @app.post("/init_session")
    async def init_session(body: dict | None = None):
        body = body or {}
        return {"session_id": await on_engine(engine.init_session(body.get("group_id"), body.get("sample_params")))}

    @app.post("/generate")
    async def generate(body: dict):
        sid = body.get("session_id")
        if sid not in engine.session_state_map:
            raise HTTPException(404, f"unknown session_id {sid}")
        text, stop, idx = await on_engine(engine.generate(body["messages"], session_id=sid,
                                                          sample_params=body.get("sample_params") or {},
                                                          tools_json=body.get("tools")))
        return {"response": text, "stop_program": stop, "step_idx": idx}

    @app.post("/end_session")
    async def end_session(body: dict):
        sr = body.get("step_rewards")
        sr = {int(k): decode_reward(float(v)) for k, v in sr.items()} if sr else None
        return await on_engine(engine.end_session(body["session_id"], reward=decode_reward(float(body.get("reward", 0.0))),
                                                  step_rewards=sr)) or {"status": "ok"}

    @app.post("/session_status")
    async def session_status(body: dict):
        st = engine.session_state_map.get(body.get("session_id"))
        return {"done": st is None or st.done, "num_steps": 0 if st is None else st.num_steps}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "axon"}]}

    @app.post("/tokenize")
    async def tokenize(body: dict):
        text = body.get("prompt")
        if text is None and body.get("messages") is not None:
            text = engine.chat_parser.parse(body["messages"], add_generation_prompt=body.get("add_generation_prompt", True))
        out = await on_engine(engine.chat_parser.tokenize(text or ""))
        return {"tokens": out.token_ids, "count": len(out.token_ids)}

    @app.post("/v1/chat/completions")
    async def chat_completions(body: dict):
        user = body.get("user") or ""
        sid = user.split("axon:", 1)[1] if user.startswith("axon:") else None
        implicit = sid is None
        if implicit:
            sid = await on_engine(engine.init_session(None, None))
        elif sid not in engine.session_state_map:
            raise HTTPException(404, f"unknown session {sid}")
        params = {k: body[k] for k in ("temperature", "top_p", "top_k", "max_tokens", "repetition_penalty") if k in body}
        text, stop, idx = await on_engine(engine.generate(body["messages"], session_id=sid, sample_params=params,
                                                          tools_json=body.get("tools")))
        if implicit:
            await on_engine(engine.end_session(sid, reward=0.0))
        return {"id": "chatcmpl-" + uuid.uuid4().hex[:24], "object": "chat.completion", "created": int(time.time()),
                "model": body.get("model", model_name), "axon": {"session_id": sid, "step_idx": idx, "stop_program": stop},
                "choices": [{"index": 0, "message": {"role": "assistant", "content": text},
                             "finish_reason": "length" if stop else "stop"}]}

    return app
