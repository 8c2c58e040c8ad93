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
class SpecDecodeMetrics:
    """Speculative decoding of ONE request (reference: ``SpecDecodeMetrics``, axon/sampler/base/server.py:35-57)."""
    num_draft_tokens: int = 0         # tokens proposed by the drafter
    num_accepted_tokens: int = 0      # of those, kept after the model verified them
    num_completions: int = 0          # verification rounds (each yields at least one token)

    @property
    def accept_rate(self) -> float:
        return self.num_accepted_tokens / self.num_draft_tokens if self.num_draft_tokens > 0 else 0.0

    @property
    def accept_length(self) -> float:
        """Average tokens per verification round (1.0 = no gain)."""
        return (self.num_accepted_tokens + self.num_completions) / self.num_completions if self.num_completions > 0 else 0.0

    def to_dict(self) -> dict:
        return {"num_draft_tokens": self.num_draft_tokens, "num_accepted_tokens": self.num_accepted_tokens,
                "num_completions": self.num_completions}


@dataclass
class TokenOutput:
    token_ids: list[int] = field(default_factory=list)
    logprobs: list[float] = field(default_factory=list)
    finish_reason: str | None = None      # "stop" | "length" | "abort"
    stop_reason: int | None = None
    moe_routermap: object | None = None   # int16 [n_tokens, n_moe_layers, top_k] or None
    prompt_len: int = 0
    spec_decode_metrics: SpecDecodeMetrics | None = None      # set when the request went through speculative rounds
