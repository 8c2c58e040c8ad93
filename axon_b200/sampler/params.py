"""Sampling parameters (the ``decoding`` block of the reference config:
axon/config/config.yaml:212-231) and per-request outputs (``TokenOutput``:
axon/sampler/base/server.py:35-181)."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_k: int = 0            # <= 0: off
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    max_tokens: int = 256
    n: int = 1
    logprobs: int = 1
    stop_token_ids: tuple = ()
    ignore_eos: bool = False
    seed: int | None = None


@dataclass
class TokenOutput:
    token_ids: list[int] = field(default_factory=list)
    logprobs: list[float] = field(default_factory=list)
    finish_reason: str | None = None      # "stop" | "length" | "abort"
    stop_reason: int | None = None
    moe_routermap: object | None = None   # int16 [n_tokens, n_moe_layers, top_k] or None
    prompt_len: int = 0
