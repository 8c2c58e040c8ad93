"""Advantage estimators. Every estimator is ``fn(data, config) -> (advantages, returns)`` with
``[B, T]`` outputs masked by ``response_mask``; group-based ones key on ``non_tensor_batch['uid']``
and use the per-row scalar score ``token_level_rewards.sum(-1)``.

Same estimators and conventions as the reference (axon/trainer/algos/advantages/advantage.py:40-645):
Bessel-corrected group std, singleton groups produce zero advantage (or an un-baselined score
where the reference does so), GAE whitening over the response mask.
"""
from __future__ import annotations

import torch

from ....utils.rl.advantage import as_torch_index, group_mean_std, masked_whiten
from .registry import AdvantageFn, register_advantage


class _Groups:
    """Scores and per-row group statistics for one batch."""

    def __init__(self, data):
        self.rewards = data.batch["token_level_rewards"]
        self.mask = data.batch["response_mask"]
        self.scores = self.rewards.sum(-1)
        self.g = as_torch_index(data.non_tensor_batch["uid"], device=self.scores.device)
        n_groups = int(self.g.max().item()) + 1 if self.g.numel() else 0
        self.n_groups = n_groups
        self.count = torch.bincount(self.g, minlength=n_groups)[self.g].to(self.scores.dtype)

    def gsum(self, values: torch.Tensor) -> torch.Tensor:
        """Sum of ``values`` over each row's group, broadcast back to rows."""
        return torch.bincount(self.g, weights=values.double(), minlength=self.n_groups)[self.g].to(values.dtype)

    def spread(self, scalars: torch.Tensor):
        adv = scalars.unsqueeze(-1) * self.mask
        return adv, adv


def _gae_scan(rewards, values, mask, gamma, lam):
    B, T = rewards.shape
    adv = torch.zeros_like(rewards)
    next_v = torch.zeros(B, dtype=rewards.dtype, device=rewards.device)
    run = torch.zeros_like(next_v)
    for t in range(T - 1, -1, -1):
        m = mask[:, t]
        delta = rewards[:, t] + gamma * next_v - values[:, t]
        cand = delta + gamma * lam * run
        next_v = values[:, t] * m + (1 - m) * next_v   # masked positions are skipped over
        run = cand * m + (1 - m) * run
        adv[:, t] = run
    return adv


@register_advantage(AdvantageFn.GAE)
@torch.no_grad()
def gae_advantage_fn(data, config):
    r, v, m = data.batch["token_level_rewards"], data.batch["values"], data.batch["response_mask"]
    adv = _gae_scan(r, v, m.to(r.dtype), config.get("gamma", 0.99), config.get("lam", 0.95))
    returns = adv + v
    return masked_whiten(adv, m), returns


@register_advantage(AdvantageFn.GRPO)
@torch.no_grad()
def grpo_advantage_fn(data, config):
    eps = config.get("epsilon", 1e-6)
    G = _Groups(data)
    mean, std, cnt = group_mean_std(G.scores, G.g, eps=eps)
    centred = G.scores - mean[G.g]
    if config.get("norm_adv_by_std", True):
        centred = centred / (std[G.g] + eps)
    return G.spread(centred * (cnt[G.g] > 1))


@register_advantage(AdvantageFn.RLOO)
@register_advantage(AdvantageFn.LOOP)
@torch.no_grad()
def rloo_advantage_fn(data, config):
    """Leave-one-out baseline: a_i = (n s_i - S_g) / (n - 1); zero for singleton groups."""
    G = _Groups(data)
    n = G.count
    adv = (n * G.scores - G.gsum(G.scores)) / (n - 1).clamp_min(1) * (n > 1)
    return G.spread(adv)


@register_advantage(AdvantageFn.REINFORCE_PLUS_PLUS)
@torch.no_grad()
def reinforce_plus_plus_advantage_fn(data, config):
    r, m = data.batch["token_level_rewards"], data.batch["response_mask"]
    gamma = config.get("gamma", 1.0)
    returns = torch.zeros_like(r)
    run = torch.zeros(r.shape[0], dtype=r.dtype, device=r.device)
    for t in range(r.shape[1] - 1, -1, -1):
        run = r[:, t] + gamma * run
        returns[:, t] = run
        run = run * m[:, t]
    return masked_whiten(returns, m) * m, returns


@register_advantage(AdvantageFn.REINFORCE_PLUS_PLUS_BASELINE)
@torch.no_grad()
def reinforce_plus_plus_baseline_advantage_fn(data, config):
    """Group-mean baseline (none for singletons), then batch-wide whitening."""
    G = _Groups(data)
    base = torch.where(G.count > 1, G.gsum(G.scores) / G.count.clamp_min(1), torch.zeros_like(G.scores))
    spread = (G.scores - base).unsqueeze(-1).expand_as(G.mask) * G.mask
    out = masked_whiten(spread, G.mask) * G.mask
    return out, out


@register_advantage(AdvantageFn.REMAX)
@torch.no_grad()
def remax_advantage_fn(data, config):
    r, m = data.batch["token_level_rewards"], data.batch["response_mask"]
    returns = (r * m).flip(-1).cumsum(-1).flip(-1)
    return returns - data.batch["reward_baselines"].unsqueeze(-1) * m, returns


@register_advantage(AdvantageFn.OPO)
@torch.no_grad()
def opo_advantage_fn(data, config):
    """Length-weighted group baseline sum(len_i s_i) / sum(len_i); singleton groups keep their score."""
    G = _Groups(data)
    lens = G.mask.sum(-1).to(G.scores.dtype)
    base = torch.where(G.count > 1, G.gsum(lens * G.scores) / G.gsum(lens).clamp_min(1), torch.zeros_like(G.scores))
    return G.spread(G.scores - base)


@register_advantage(AdvantageFn.GRPO_PASSK)
@torch.no_grad()
def grpo_passk_advantage_fn(data, config):
    """Only the best row of each group gets (r_max - r_second) [/ std]; needs >= 2 rows per group."""
    eps = config.get("epsilon", 1e-6)
    G = _Groups(data)
    adv = torch.zeros_like(G.scores)
    for gid in range(G.n_groups):
        rows = torch.nonzero(G.g == gid).flatten()
        if rows.numel() < 2:
            raise ValueError(f"Pass@k requires at least 2 samples per group, got {rows.numel()}")
        vals = G.scores[rows]
        top, idx = torch.topk(vals, 2)
        a = top[0] - top[1]
        if config.get("norm_adv_by_std", True):
            a = a / (vals.std() + eps)
        adv[rows[idx[0]]] = a
    return G.spread(adv)


@register_advantage(AdvantageFn.GPG)
@torch.no_grad()
def gpg_advantage_fn(data, config):
    """alpha (s - group mean) / f_norm with alpha = B / #nonzero scores."""
    G = _Groups(data)
    alpha = G.scores.shape[0] / torch.count_nonzero(G.scores).clamp(min=1).to(G.scores.dtype)
    mean = torch.where(G.count > 1, G.gsum(G.scores) / G.count, torch.zeros_like(G.scores))
    return G.spread(alpha * (G.scores - mean) / config.get("f_norm", 1.0))


def _chunked_gae_core(rewards, values, gamma, lam, chunk_size=128):
    """GAE as a blocked scan: inside a chunk of the time-reversed TD errors the discounted suffix sums
    are one matmul with a lower-triangular power matrix; chunks are chained through one carry per row.
    V beyond the last position is zero."""
    B, T = rewards.shape
    w = gamma * lam
    nxt = torch.cat([values[:, 1:], values.new_zeros(B, 1)], 1)
    d = (rewards + gamma * nxt - values).flip(1)
    pad = (-T) % chunk_size
    if pad:
        d = torch.nn.functional.pad(d, (0, pad))
    C = d.shape[1] // chunk_size
    k = torch.arange(chunk_size, device=d.device)
    lag = k[None, :] - k[:, None]                       # column j collects rows i <= j with weight w^(j-i)
    tri = torch.where(lag >= 0, torch.tensor(float(w), dtype=d.dtype, device=d.device) ** lag.clamp(min=0).to(d.dtype),
                      torch.zeros((), dtype=d.dtype, device=d.device))
    carry_w = torch.tensor(float(w), dtype=d.dtype, device=d.device) ** (k + 1).to(d.dtype)
    local = (d.view(B * C, chunk_size) @ tri).view(B, C, chunk_size)
    out = torch.empty_like(local)
    carry = d.new_zeros(B)
    valid_last = chunk_size - pad if pad else chunk_size
    for c in range(C):
        out[:, c] = local[:, c] + carry[:, None] * carry_w
        last = valid_last - 1 if c == C - 1 else chunk_size - 1
        carry = out[:, c, last]
    adv = out.view(B, -1)[:, :T].flip(1)
    return adv, adv + values


@register_advantage(AdvantageFn.CHUNKED_GAE)
@torch.no_grad()
def chunked_gae_advantage_fn(data, config):
    """GAE over the response tokens only (arbitrary masks are compacted first), blocked scan."""
    r, v, m = data.batch["token_level_rewards"], data.batch["values"], data.batch["response_mask"]
    B, T = r.shape
    n = m.sum(1).long()
    width = int(n.max().item()) if B else 0
    if width == 0:
        z = torch.zeros_like(r)
        return z, z
    order = torch.argsort((m <= 0).to(torch.int8), dim=1, stable=True)[:, :width]   # response positions first
    keep = torch.arange(width, device=r.device)[None, :] < n[:, None]
    cr = torch.where(keep, r.gather(1, order), torch.zeros((), dtype=r.dtype, device=r.device))
    cv = torch.where(keep, v.gather(1, order), torch.zeros((), dtype=v.dtype, device=v.device))
    a, ret = _chunked_gae_core(cr, cv, config.get("gamma", 0.99), config.get("lam", 0.95),
                               config.get("chunk_size", 128))
    adv, returns = torch.zeros_like(r), torch.zeros_like(r)
    rows = torch.arange(B, device=r.device)[:, None].expand_as(order)
    adv[rows[keep], order[keep]] = a[keep]
    returns[rows[keep], order[keep]] = ret[keep]
    return masked_whiten(adv, m), returns


@register_advantage(AdvantageFn.KIMI_K1_5)
@torch.no_grad()
def kimi_k1_5_advantage_fn(data, config):
    """GRPO on length-shaped scores: lam_i = coef (0.5 - (len_i - min)/(max - min)) is added to correct
    rollouts, min(0, lam_i) to incorrect ones; no shaping when all lengths in the group are equal.
    The coefficient follows a warm-up / linear-ramp schedule on ``meta_info['global_steps']``."""
    eps = config.get("epsilon", 1e-6)
    target = float(config.get("length_coef", 0.0))
    warm, ramp = int(config.get("length_coef_warmup_steps", 0)), int(config.get("length_coef_ramp_steps", 0))
    step = int((getattr(data, "meta_info", None) or {}).get("global_steps", 0) or 0)
    if step < warm:
        coef = 0.0
    elif ramp > 0 and step < warm + ramp:
        coef = target * (step - warm) / ramp
    else:
        coef = target
    G = _Groups(data)
    scores = G.scores
    if coef > 0.0 and G.g.numel():
        lens = G.mask.sum(-1).to(scores.dtype)
        lo = torch.full((G.n_groups,), float("inf"), dtype=scores.dtype, device=scores.device)
        hi = torch.full((G.n_groups,), float("-inf"), dtype=scores.dtype, device=scores.device)
        lo.scatter_reduce_(0, G.g, lens, reduce="amin", include_self=False)
        hi.scatter_reduce_(0, G.g, lens, reduce="amax", include_self=False)
        span = (hi - lo)[G.g]
        lam = coef * (0.5 - (lens - lo[G.g]) / span.clamp_min(1.0))
        correct = scores >= float(config.get("correct_threshold", 1.0))
        bonus = torch.where(correct, lam, lam.clamp(max=0.0)) * (span > 0)
        scores = scores + bonus
    mean, std, cnt = group_mean_std(scores, G.g, eps=eps)
    centred = scores - mean[G.g]
    if config.get("norm_adv_by_std", True):
        centred = centred / (std[G.g] + eps)
    return G.spread(centred * (cnt[G.g] > 1))


@register_advantage(AdvantageFn.IDENTITY)
@torch.no_grad()
def identity_advantage_fn(data, config):
    adv = data.batch["token_level_rewards"] * data.batch["response_mask"]
    return adv, adv
