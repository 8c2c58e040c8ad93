"""Padding helpers for packed (varlen) attention (reference: axon/utils/torch/attention.py, which forwards to
flash-attn's ``bert_padding``). Plain PyTorch: the packed layout they produce is the one the attention
kernels of ``ops/attention.py`` take."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def index_first_axis(x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """Rows ``indices`` of ``x`` flattened over its first axis' remaining dims (differentiable)."""
    return x.reshape(x.shape[0], -1)[indices.long()].reshape(indices.numel(), *x.shape[1:])


def get_unpad_data(attention_mask: torch.Tensor):
    """(indices of real tokens in the flattened batch, cu_seqlens int32 [B+1], longest sequence)."""
    seqlens = attention_mask.sum(-1, dtype=torch.int32)
    indices = torch.nonzero(attention_mask.flatten(), as_tuple=False).flatten()
    cu = F.pad(torch.cumsum(seqlens, 0, dtype=torch.int32), (1, 0))
    return indices, cu, int(seqlens.max()) if seqlens.numel() else 0


def unpad_input(hidden_states: torch.Tensor, attention_mask: torch.Tensor):
    """[B, S, ...] + mask [B, S] -> (packed [T, ...], indices, cu_seqlens, max_seqlen, tokens per sequence)."""
    indices, cu, longest = get_unpad_data(attention_mask)
    flat = hidden_states.reshape(-1, *hidden_states.shape[2:])
    return index_first_axis(flat, indices), indices, cu, longest, attention_mask.sum(-1, dtype=torch.int32)


def pad_input(hidden_states: torch.Tensor, indices: torch.Tensor, batch: int, seqlen: int) -> torch.Tensor:
    """Inverse of ``unpad_input``: packed [T, ...] -> [B, S, ...] with zeros at the padding."""
    out = torch.zeros(batch * seqlen, *hidden_states.shape[1:], dtype=hidden_states.dtype, device=hidden_states.device)
    out = out.index_put((indices.long(),), hidden_states)
    return out.view(batch, seqlen, *hidden_states.shape[1:])


def rearrange(x, pattern: str, **axes):
    from einops import rearrange as _rearrange
    return _rearrange(x, pattern, **axes)
