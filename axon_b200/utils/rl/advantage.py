"""Group statistics and masked whitening shared by the advantage estimators
(reference: axon/utils/rl/advantage.py)."""
from __future__ import annotations

from typing import Any

import numpy as np
import torch


def as_torch_index(index: Any, device=None) -> torch.Tensor:
    """Map arbitrary hashable group ids (strings, ints, arrays) to dense int64 ids 0..G-1 in order
    of first appearance."""
    if isinstance(index, torch.Tensor) and index.dtype in (torch.int32, torch.int64):
        vals = index.detach().cpu().tolist()
    else:
        vals = list(np.asarray(index, dtype=object).ravel())
    table: dict = {}
    dense = [table.setdefault(v if not isinstance(v, np.generic) else v.item(), len(table)) for v in vals]
    return torch.tensor(dense, dtype=torch.long, device=device)


@torch.no_grad()
def group_mean_std(scores: torch.Tensor, gidx: torch.Tensor, eps: float = 1e-6, device=None):
    """Per-group mean, Bessel-corrected std (variance floored at eps) and count. Singleton groups
    get mean 0 and std 1 so callers can zero them out by count."""
    dev = device or scores.device
    scores = scores.to(dev, torch.float32)
    gidx = gidx.to(dev)
    G = int(gidx.max().item()) + 1 if gidx.numel() else 0
    if G == 0:
        e = torch.empty(0, device=dev)
        return e, e.clone(), e.clone()
    cnt = torch.zeros(G, device=dev).index_add_(0, gidx, torch.ones_like(scores))
    s1 = torch.zeros(G, device=dev).index_add_(0, gidx, scores)
    s2 = torch.zeros(G, device=dev).index_add_(0, gidx, scores * scores)
    n = cnt.clamp_min(1.0)
    mean = s1 / n
    var = (s2 - s1 * s1 / n) / (cnt - 1.0).clamp_min(1.0)
    std = var.clamp(min=eps).sqrt()
    lone = cnt <= 1.0
    mean = torch.where(lone, torch.zeros_like(mean), mean)
    std = torch.where(lone, torch.ones_like(std), std)
    return mean, std, cnt


@torch.no_grad()
def masked_mean(values: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    m = mask.to(values.dtype)
    return (values * m).sum() / m.sum().clamp_min(1.0)


@torch.no_grad()
def masked_var(values: torch.Tensor, mask: torch.Tensor, bessel_correction: bool = True) -> torch.Tensor:
    m = mask.to(values.dtype)
    n = m.sum()
    mu = (values * m).sum() / n.clamp_min(1.0)
    var = ((values - mu) ** 2 * m).sum() / n.clamp_min(1.0)
    if bessel_correction and n > 1:
        var = var * n / (n - 1)
    return var


@torch.no_grad()
def masked_whiten(values: torch.Tensor, mask: torch.Tensor, shift_mean: bool = True) -> torch.Tensor:
    mu, var = masked_mean(values, mask), masked_var(values, mask)
    out = (values - mu) * torch.rsqrt(var + 1e-8)
    return out if shift_mean else out + mu
