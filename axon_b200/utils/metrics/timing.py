"""Wall-clock section timers and per-token timing metrics
(reference: axon/utils/metrics/timing.py:60-204)."""
from __future__ import annotations

import time
from contextlib import contextmanager
from typing import Any

_TOKEN_SECTIONS_ALL = ("ref", "values", "adv", "update_critic", "forward_backward")


class Timer:
    def __init__(self, name: str = ""):
        self.name, self.last = name, 0.0

    def __enter__(self):
        self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        self.last = time.perf_counter() - self._t0
        return False


@contextmanager
def marked_timer(name: str, timing_raw: dict[str, float], color: str | None = None, domain: str | None = None,
                 category: str | None = None):
    """Accumulates the section's seconds into ``timing_raw[name]`` and brackets it with an NVTX range
    when CUDA is in use, so one call site serves both the metrics and an external profiler."""
    pushed = False
    try:
        import torch
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            torch.cuda.nvtx.range_push(name)
            pushed = True
    except Exception:
        pushed = False
    t0 = time.perf_counter()
    try:
        yield
    finally:
        timing_raw[name] = timing_raw.get(name, 0.0) + time.perf_counter() - t0
        if pushed:
            import torch
            torch.cuda.nvtx.range_pop()


def _token_counts(batch):
    rm, am = batch.batch["response_mask"].bool(), batch.batch["attention_mask"].bool()
    return float((am & ~rm).sum()), float(rm.sum())


def compute_timing_metrics(batch, timing_raw: dict[str, float], include_detail: bool = False) -> dict[str, Any]:
    """``timing_s/<section>`` plus ``timing_per_token_ms/<section>``: generation is normalised by
    response tokens, the training-side sections by all tokens."""
    n_prompt, n_resp = _token_counts(batch)
    per = {"gen": n_resp, **{k: n_prompt + n_resp for k in _TOKEN_SECTIONS_ALL}}
    m = {f"timing_s/{k}": v for k, v in timing_raw.items()}
    m.update({f"timing_per_token_ms/{k}": timing_raw[k] * 1000 / max(1, per[k]) for k in per if k in timing_raw})
    if include_detail:
        m.update({"_num_prompt_tokens": n_prompt, "_num_response_tokens": n_resp, "_num_overall_tokens": n_prompt + n_resp})
    return m


def reduce_timing_metrics(metrics_list: list[dict]) -> dict[str, Any]:
    if not metrics_list:
        return {}
    keys = {k for m in metrics_list for k in m if k.startswith("timing_s/")}
    out = {k: metrics_list[0].get(k, 0) for k in keys}       # sections are shared wall-clock, not additive
    n_resp = sum(m.get("_num_response_tokens", 0) for m in metrics_list)
    n_all = sum(m.get("_num_overall_tokens", 0) for m in metrics_list)
    per = {"gen": n_resp, **{k: n_all for k in _TOKEN_SECTIONS_ALL}}
    for k in keys:
        s = k[len("timing_s/"):]
        if per.get(s, 0) > 0:
            out[f"timing_per_token_ms/{s}"] = out[k] * 1000 / per[s]
    return out
