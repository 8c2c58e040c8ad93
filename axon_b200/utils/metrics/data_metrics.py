"""Per-step statistics of a training batch: scores, rewards, advantages, returns, values, lengths
(reference: axon/utils/metrics/data_metrics.py:29-371). Programs are counted once (last step,
non-padding rows); token statistics use the trained tokens of those rows."""
from __future__ import annotations

from typing import Any

import numpy as np
import torch

_SEQ_STATS = (("critic/score", "score"), ("critic/rewards", "reward"))
_TOK_STATS = (("critic/advantages", "adv"), ("critic/returns", "returns"))


def compute_response_mask(data) -> torch.Tensor:
    """The trailing ``responses``-wide slice of the attention mask (prompt-then-response layouts)."""
    n = data.batch["responses"].size(1)
    return data.batch["attention_mask"][:, -n:]


def _lengths(batch):
    rm, am = batch.batch["response_mask"].bool(), batch.batch["attention_mask"].bool()
    return (am & ~rm).sum(-1).float(), rm.sum(-1).float()


def _mmm(prefix: str, t: torch.Tensor) -> dict:
    return {f"{prefix}/mean": t.mean().item(), f"{prefix}/max": t.max().item(), f"{prefix}/min": t.min().item()}


def compute_data_metrics(batch, use_critic: bool = True, include_detail: bool = False) -> dict[str, Any]:
    nt = batch.non_tensor_batch
    if "is_last_step" in nt:
        batch = batch.select_idxs(np.nonzero(np.asarray(nt["is_last_step"], dtype=bool))[0])
    if "is_padding" in batch.non_tensor_batch:
        batch = batch.select_idxs(np.nonzero(~np.asarray(batch.non_tensor_batch["is_padding"], dtype=bool))[0])
    if len(batch) == 0:
        return {}
    b = batch.batch
    T = b["input_ids"].shape[-1]
    rmask = b["response_mask"].bool()
    prompt_len, resp_len = _lengths(batch)
    alive = resp_len > 0
    if not alive.any():
        raise ValueError("every sample has an empty response; cannot compute data metrics")
    seq = {"score": b["token_level_scores"].sum(-1)[alive], "reward": b["token_level_rewards"].sum(-1)[alive]}
    tok = {"adv": b["advantages"][rmask], "returns": b["returns"][rmask]}
    m: dict[str, Any] = {}
    for prefix, key in _SEQ_STATS:
        m.update(_mmm(prefix, seq[key]))
    for prefix, key in _TOK_STATS:
        m.update(_mmm(prefix, tok[key]))
    if use_critic:
        vals = b["values"][rmask]
        m.update(_mmm("critic/values", vals))
        m["critic/vf_explained_var"] = (1.0 - torch.var(tok["returns"] - vals) / (torch.var(tok["returns"]) + 1e-5)).item()
    live_len = resp_len[alive]
    m.update(_mmm("response_length", resp_len))
    m["response_length/clip_ratio"] = (resp_len == T).float().mean().item()
    m.update(_mmm("response_length_non_aborted", live_len))
    m["response_length_non_aborted/clip_ratio"] = (live_len == T).float().mean().item()
    m["response/aborted_ratio"] = (~alive).float().mean().item()
    m.update(_mmm("prompt_length", prompt_len))
    m["prompt_length/clip_ratio"] = (prompt_len == T).float().mean().item()
    if include_detail:
        m.update({"_count_non_aborted": int(alive.sum()), "_count_valid_tokens": int(tok["adv"].numel()), "_count_all": len(batch),
                  "_count_aborted": int((~alive).sum()), "_count_non_aborted_response": int(alive.sum()),
                  "_sum_score": seq["score"].sum().item(), "_sum_reward": seq["reward"].sum().item(),
                  "_sum_adv": tok["adv"].sum().item(), "_sum_returns": tok["returns"].sum().item(),
                  "_sum_response_length": resp_len.sum().item(), "_sum_non_aborted_response_length": live_len.sum().item(),
                  "_sum_prompt_length": prompt_len.sum().item(), "_count_clipped_response": int((resp_len == T).sum()),
                  "_count_non_aborted_clipped": int((live_len == T).sum()), "_count_clipped_prompt": int((prompt_len == T).sum())})
        if use_critic:
            m.update({"_sum_values": vals.sum().item(), "_sum_returns_squared": (tok["returns"] ** 2).sum().item(),
                      "_sum_values_squared": (vals ** 2).sum().item(), "_sum_returns_times_values": (tok["returns"] * vals).sum().item()})
    return m


def reduce_data_metrics(metrics_list: list[dict]) -> dict[str, Any]:
    ms = [m for m in (metrics_list or []) if m]
    if not ms:
        return {}
    tot = lambda k: sum(m.get(k, 0) for m in ms)                     # noqa: E731
    n_all, n_alive, n_tok, n_live = tot("_count_all"), tot("_count_non_aborted"), tot("_count_valid_tokens"), tot("_count_non_aborted_response")
    if n_all == 0:
        return {}
    out: dict[str, Any] = {}
    for p in ("critic/score", "critic/rewards", "critic/advantages", "critic/returns", "response_length",
              "response_length_non_aborted", "prompt_length"):
        out[f"{p}/max"] = max(m.get(f"{p}/max", float("-inf")) for m in ms)
        out[f"{p}/min"] = min(m.get(f"{p}/min", float("inf")) for m in ms)
    if n_alive:
        out["critic/score/mean"], out["critic/rewards/mean"] = tot("_sum_score") / n_alive, tot("_sum_reward") / n_alive
    if n_tok:
        out["critic/advantages/mean"], out["critic/returns/mean"] = tot("_sum_adv") / n_tok, tot("_sum_returns") / n_tok
    out["response_length/mean"] = tot("_sum_response_length") / n_all
    out["response_length/clip_ratio"] = tot("_count_clipped_response") / n_all
    out["response/aborted_ratio"] = tot("_count_aborted") / n_all
    if n_live:
        out["response_length_non_aborted/mean"] = tot("_sum_non_aborted_response_length") / n_live
        out["response_length_non_aborted/clip_ratio"] = tot("_count_non_aborted_clipped") / n_live
    out["prompt_length/mean"] = tot("_sum_prompt_length") / n_all
    out["prompt_length/clip_ratio"] = tot("_count_clipped_prompt") / n_all
    if any("_sum_values" in m for m in ms) and n_tok:
        out["critic/values/max"] = max(m.get("critic/values/max", float("-inf")) for m in ms)
        out["critic/values/min"] = min(m.get("critic/values/min", float("inf")) for m in ms)
        out["critic/values/mean"] = tot("_sum_values") / n_tok
        r2, v2, rv = tot("_sum_returns_squared") / n_tok, tot("_sum_values_squared") / n_tok, tot("_sum_returns_times_values") / n_tok
        r_mean = out["critic/returns/mean"]
        out["critic/vf_explained_var"] = 1.0 - (r2 - 2 * rv + v2) / (r2 - r_mean ** 2 + 1e-5)
    for name in ("num_turns", "tool_call_counts"):
        if any(f"_sum_{name}" in m for m in ms):
            out[f"{name}/min"] = min(m.get(f"{name}/min", float("inf")) for m in ms)
            out[f"{name}/max"] = max(m.get(f"{name}/max", float("-inf")) for m in ms)
            out[f"{name}/mean"] = tot(f"_sum_{name}") / n_all
    return out
