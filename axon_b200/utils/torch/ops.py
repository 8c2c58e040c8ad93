"""Tensor helpers for the logits path and masked statistics (reference: axon/utils/torch/ops.py:39-360).

The hot path never materialises ``[T, V]`` logits (the fused vocabulary head in ``ops/lm_head`` gives
log-probs and entropy directly); these functions serve the non-fused path, tests and utilities.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F


def logprobs_from_logits(logits: torch.Tensor, labels: torch.Tensor, inplace_backward: bool = True) -> torch.Tensor:
    """log softmax(logits)[labels] computed row-wise in fp32 without keeping the full log-softmax."""
    shape = labels.shape
    lg = logits.reshape(-1, logits.shape[-1])
    lb = labels.reshape(-1)
    out = lg.float().gather(-1, lb.unsqueeze(-1)).squeeze(-1) - torch.logsumexp(lg.float(), dim=-1)
    return out.view(shape)


def logprobs_from_logits_v2(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Memory-lean variant: per-row loop for low-precision inputs (log_softmax in the input dtype)."""
    if logits.dtype in (torch.float32, torch.float64):
        picked = torch.gather(logits, -1, labels.unsqueeze(-1)).squeeze(-1)
        return picked - torch.stack([torch.logsumexp(row, dim=-1) for row in logits])
    return torch.stack([F.log_softmax(row, dim=-1).gather(-1, lab.unsqueeze(-1)).squeeze(-1)
                        for row, lab in zip(logits, labels)])


def entropy_from_logits(logits: torch.Tensor) -> torch.Tensor:
    pd = F.softmax(logits, dim=-1)
    return torch.logsumexp(logits, dim=-1) - (pd * logits).sum(-1)


def entropy_from_logits_with_chunking(logits: torch.Tensor, chunk_size: int = 2048) -> torch.Tensor:
    out = torch.zeros(logits.shape[0], device=logits.device)
    for s in range(0, logits.shape[0], chunk_size):
        out[s:s + chunk_size] = entropy_from_logits(logits[s:s + chunk_size].float())
    return out


def masked_sum(values, mask, axis=None):
    valid = ~torch.isnan(values)
    return (torch.where(valid, values, torch.zeros_like(values)) * mask).sum(axis=axis)


def masked_mean(values, mask, axis=None):
    return masked_sum(values, mask, axis) / (mask.sum(axis=axis) + 1e-8)


def distributed_masked_mean(local_tensor, local_mask, group=None):
    s = torch.stack([(local_tensor * local_mask).sum(), local_mask.sum().to(local_tensor.dtype)])
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(s, group=group)
    return s[0] / s[1].clamp_min(1e-8)


def masked_var(values, mask, unbiased: bool = True):
    mean = masked_mean(values, mask)
    var = masked_mean((values - mean) ** 2, mask)
    if unbiased:
        n = mask.sum()
        if n == 0:
            raise ValueError("the mask has no valid element")
        if n == 1:
            raise ValueError("unbiased variance needs at least two valid elements")
        var = var * n / (n - 1)
    return var


def masked_whiten(values, mask, shift_mean: bool = True):
    mean, var = masked_mean(values, mask), masked_var(values, mask)
    out = (values - mean) * torch.rsqrt(var + 1e-8)
    return out if shift_mean else out + mean


def get_response_mask(response_id: torch.Tensor, eos_token=2, dtype=torch.int64) -> torch.Tensor:
    """1 up to and including the first EOS of every row, 0 after it."""
    eos = torch.tensor([eos_token] if isinstance(eos_token, int) else list(eos_token), device=response_id.device)
    hit = torch.isin(response_id, eos).long()
    return (torch.cumsum(hit, dim=1) - hit).eq(0).to(dtype)


def broadcast_dict_tensor(tensors: dict, src: int, group=None) -> None:
    for k in sorted(tensors.keys()):
        dist.broadcast(tensors[k], src=src, group=group)


def allgather_dict_tensors(tensors: dict, size: int, group=None, dim: int = 0) -> dict:
    out = {}
    for k in sorted(tensors.keys()):
        parts = [torch.empty_like(tensors[k]) for _ in range(size)]
        dist.all_gather(parts, tensors[k].contiguous(), group=group)
        out[k] = torch.cat(parts, dim=dim)
    return out


def pad_from_left(input_id_list: list[list[int]], pad_token_id: int) -> list[list[int]]:
    n = max(len(x) for x in input_id_list)
    return [[pad_token_id] * (n - len(x)) + list(x) for x in input_id_list]


def pad_sequence_to_length(t: torch.Tensor, max_seq_len: int, pad_token_id, left_pad: bool = False) -> torch.Tensor:
    if t.shape[-1] >= max_seq_len:
        return t
    pad = (max_seq_len - t.shape[-1], 0) if left_pad else (0, max_seq_len - t.shape[-1])
    return F.pad(t, pad, value=pad_token_id)


def log_probs_from_logits_response(input_ids, logits, response_length: int):
    """Log-probs of the last ``response_length`` tokens of every row (logits[t] predicts token t+1)."""
    resp_logits = logits[:, -response_length - 1:-1]
    return logprobs_from_logits(resp_logits, input_ids[:, -response_length:])


def get_unpad_data(attention_mask: torch.Tensor):
    """(flat indices of real tokens, cu_seqlens int32, longest row)."""
    lens = attention_mask.sum(-1, dtype=torch.int32)
    idx = torch.nonzero(attention_mask.flatten(), as_tuple=False).flatten()
    cu = F.pad(torch.cumsum(lens, 0, dtype=torch.int32), (1, 0))
    return idx, cu, int(lens.max().item()) if lens.numel() else 0


def log_probs_from_logits_response_rmpad(input_ids, attention_mask, logits_rmpad, response_length: int):
    """Same as ``log_probs_from_logits_response`` for padding-free logits ``[total_tokens, V]``."""
    B, T = input_ids.shape
    idx, _, _ = get_unpad_data(attention_mask)
    flat_ids = input_ids.flatten()[idx]
    rolled = torch.roll(flat_ids, shifts=-1, dims=0)
    lp = logprobs_from_logits(logits_rmpad, rolled)
    full = torch.zeros(B * T, dtype=lp.dtype, device=lp.device)
    full[idx] = lp
    return full.view(B, T)[:, -response_length - 1:-1]
