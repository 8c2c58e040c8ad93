"""Loss aggregation. ``agg_loss`` reduces a ``[B, T]`` per-token loss in two stages
(reference: axon/trainer/algos/loss/utils.py:120-251):

  token_reduce  [B,T] -> [B]   sum | mean (per-row token count) | mean-norm (/T) |
                               mean-program (/ tokens of the whole program)
  batch_reduce  [B] -> scalar  token-mean (/ valid tokens) | step-mean (/ valid rows) |
                               program-mean (rows first divided by their program's step count,
                               then / valid programs)

The ``valid_*`` denominators are mini-batch-global counts supplied by the driver so that every
data-parallel rank divides by the same number; without them local counts are used.
"""
from __future__ import annotations

import torch

TOKEN_REDUCE = ("sum", "mean", "mean-norm", "mean-program")
BATCH_REDUCE = ("token-mean", "step-mean", "program-mean")


def masked_mean(values: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    return (values * mask).sum() / mask.sum().clamp_min(1.0)


def clip_by_value(t: torch.Tensor, lo, hi) -> torch.Tensor:
    if isinstance(lo, torch.Tensor) or isinstance(hi, torch.Tensor):
        return torch.maximum(torch.minimum(t, torch.as_tensor(hi, dtype=t.dtype, device=t.device)),
                             torch.as_tensor(lo, dtype=t.dtype, device=t.device))
    return torch.clamp(t, min=lo, max=hi)


def entropy_from_logits(logits: torch.Tensor) -> torch.Tensor:
    lp = torch.log_softmax(logits, -1)
    return -(lp.exp() * lp).sum(-1)


def _denominator(val, like: torch.Tensor) -> torch.Tensor:
    t = torch.as_tensor(val, dtype=like.dtype, device=like.device)
    if t.dim() > 0:
        t = t.reshape(-1)[0]
    return t.clamp(min=1)


def agg_loss(loss_mat, loss_mask, *, token_reduce="sum", batch_reduce="token-mean", num_program_tokens=None,
             num_program_steps=None, valid_token_count=None, valid_batch_size=None, valid_program_count=None,
             per_row_token_count=None) -> torch.Tensor:
    if token_reduce not in TOKEN_REDUCE:
        raise ValueError(f"Invalid token_reduce: {token_reduce!r}. Choose from: {sorted(TOKEN_REDUCE)}")
    if batch_reduce not in BATCH_REDUCE:
        raise ValueError(f"Invalid batch_reduce: {batch_reduce!r}. Choose from: {sorted(BATCH_REDUCE)}")
    rows = (loss_mat * loss_mask).sum(-1)
    if token_reduce == "mean":
        per_row = per_row_token_count if per_row_token_count is not None else loss_mask.sum(-1)
        rows = rows / per_row.clamp(min=1)
    elif token_reduce == "mean-norm":
        rows = rows / loss_mask.shape[-1]
    elif token_reduce == "mean-program":
        assert num_program_tokens is not None, "num_program_tokens required for token_reduce='mean-program'"
        rows = rows / num_program_tokens.clamp(min=1)
    if batch_reduce == "program-mean":
        assert num_program_steps is not None, "num_program_steps required for batch_reduce='program-mean'"
        assert valid_program_count is not None, "valid_program_count required for batch_reduce='program-mean'"
        return (rows / num_program_steps.clamp(min=1)).sum() / _denominator(valid_program_count, rows)
    total = rows.sum()
    if batch_reduce == "token-mean":
        if valid_token_count is not None:
            return total / _denominator(valid_token_count, total)
        return total / loss_mask.sum().clamp_min(1.0)
    if valid_batch_size is not None:           # step-mean
        return total / _denominator(valid_batch_size, total)
    return total / (loss_mask.sum(-1) > 0).float().sum().clamp(min=1)
