"""Policy and value losses. Uniform signature ``fn(data: DataProto, config) -> (loss, metrics)``
where ``config`` is the ``loss_args`` mapping. Each loss reads ``old_log_probs``, ``log_probs``,
``advantages`` and ``response_mask`` (all ``[B, T]``) plus the optional ``sampler_is_weights`` and
program-count tensors from ``data.batch``.

Objectives and defaults follow the reference (axon/trainer/algos/loss/loss.py:47-590): PPO with
asymmetric and dual clipping, GSPO, GPG/REINFORCE, Clip-Cov, KL-Cov, GMPO (``geo_mean``), CISPO and
the clipped value loss. Log-ratios are clamped to [-20, 20] before exponentiation.
"""
from __future__ import annotations

import torch

from .registry import LossFn, register_loss
from .utils import agg_loss, clip_by_value, masked_mean


class _Inputs:
    """The tensors every policy loss needs, plus the aggregation call bound to this batch."""

    def __init__(self, data, config, default_token_reduce="sum"):
        b = data.batch
        self.old, self.new = b["old_log_probs"], b["log_probs"]
        self.adv, self.mask = b["advantages"], b["response_mask"]
        self.is_w = b.get("sampler_is_weights", None)
        self.config = config
        self._agg = dict(
            token_reduce=config.get("token_reduce", default_token_reduce),
            batch_reduce=config.get("batch_reduce", "token-mean"),
            num_program_tokens=b.get("num_program_tokens", None),
            num_program_steps=b.get("num_program_steps", None),
            valid_token_count=b.get("valid_token_count", None),
            valid_batch_size=b.get("valid_batch_size", None),
            valid_program_count=b.get("valid_program_count", None),
            per_row_token_count=b.get("per_row_token_count", None),
        )
        self.log_ratio = self.new - self.old

    def clip_range(self, low_default=None):
        c = self.config
        base = c.get("clip_ratio", 0.2)
        lo, hi = c.get("clip_ratio_low", None), c.get("clip_ratio_high", None)
        lo = lo if lo is not None else (base if low_default is None else low_default)
        hi = hi if hi is not None else base
        return lo, hi

    def ratio(self):
        return torch.exp(self.log_ratio.clamp(-20.0, 20.0))

    def weighted(self, per_token):
        return per_token if self.is_w is None else per_token * self.is_w

    def aggregate(self, per_token):
        return agg_loss(loss_mat=per_token, loss_mask=self.mask, **self._agg)

    def kl(self):
        return masked_mean(-self.log_ratio.clamp(-20.0, 20.0), self.mask).detach().item()

    def frac(self, cond):
        return masked_mean(cond.float(), self.mask).detach().item()


@register_loss(LossFn.PPO)
def ppo_loss_fn(data, config):
    x = _Inputs(data, config)
    lo, hi = x.clip_range()
    dual = config.get("clip_ratio_c", 3.0)
    assert dual > 1.0, f"clip_ratio_c must be > 1.0, got {dual}"
    r = x.ratio()
    unclipped = -x.adv * r
    clipped = -x.adv * r.clamp(1 - lo, 1 + hi)
    pess = torch.maximum(unclipped, clipped)
    cap = -x.adv * dual                      # dual clip: bounds the loss of negative-advantage tokens
    neg = x.adv < 0
    per_token = torch.where(neg, torch.minimum(cap, pess), pess)
    loss = x.aggregate(x.weighted(per_token))
    return loss, {"pg_clipfrac": x.frac(clipped > unclipped), "ppo_kl": x.kl(),
                  "pg_clipfrac_lower": x.frac((pess > cap) & neg)}


@register_loss(LossFn.GSPO)
def gspo_loss_fn(data, config):
    """Sequence-level importance ratio (length-normalised), token-level gradient path."""
    x = _Inputs(data, config, default_token_reduce="mean")
    lo, hi = x.clip_range()
    n = x.mask.sum(-1).clamp(min=1)
    seq_log_ratio = (x.log_ratio * x.mask).sum(-1) / n
    s = torch.exp((x.new - x.new.detach() + seq_log_ratio.detach().unsqueeze(-1)).clamp(-20.0, 20.0))
    unclipped = -x.adv * s
    clipped = -x.adv * s.clamp(1 - lo, 1 + hi)
    loss = x.aggregate(x.weighted(torch.maximum(unclipped, clipped)))
    return loss, {"pg_clipfrac": x.frac(clipped > unclipped),
                  "ppo_kl": masked_mean(-x.log_ratio, x.mask).detach().item(), "pg_clipfrac_lower": 0.0}


@register_loss(LossFn.REINFORCE)
def reinforce_loss_fn(data, config):
    x = _Inputs(data, config)
    loss = x.aggregate(x.weighted(-x.adv * x.new))
    return loss, {"ppo_kl": masked_mean(-x.log_ratio, x.mask).detach().item()}


@register_loss(LossFn.GPG)
def gpg_loss_fn(data, config):
    """-log pi * A, the REINFORCE objective; pairs with the ``gpg`` advantage estimator."""
    return reinforce_loss_fn(data, config)


@register_loss(LossFn.CLIP_COV)
def clip_cov_loss_fn(data, config):
    """PPO clip plus: a random subset (``clip_cov_ratio`` of the tokens) of not-already-clipped tokens
    whose advantage/log-prob covariance lies in (lb, ub) gets zero gradient."""
    x = _Inputs(data, config, default_token_reduce="mean")
    lo, hi = x.clip_range()
    frac = config.get("clip_cov_ratio", 0.0002)
    lb, ub = config.get("clip_cov_lb", 1.0), config.get("clip_cov_ub", 5.0)
    assert frac > 0, "clip_cov_ratio must be > 0"
    r = x.ratio()
    unclipped = -x.adv * r
    clipped = -x.adv * r.clamp(1 - lo, 1 + hi)
    live = x.mask > 0
    already = (clipped > unclipped) & live
    lp = x.new.detach()
    cov = (x.adv - masked_mean(x.adv, x.mask)) * (lp - masked_mean(lp, x.mask))
    cov = cov.masked_fill(~live | already, float("-inf"))
    cand = torch.nonzero((cov < ub) & (cov > lb) & live)
    budget = max(int(frac * x.mask.sum().item()), 1)
    keep = torch.ones_like(x.adv)
    if len(cand):
        pick = cand[torch.randperm(len(cand), device=cand.device)[: min(budget, len(cand))]]
        keep[pick[:, 0], pick[:, 1]] = 0
    loss = x.aggregate(x.weighted(torch.maximum(unclipped, clipped) * keep))
    return loss, {"pg_clipfrac": x.frac(keep == 0), "ppo_kl": x.kl()}


@register_loss(LossFn.KL_COV)
def kl_cov_loss_fn(data, config):
    """Unclipped surrogate; the top ``kl_cov_ratio`` fraction of tokens by advantage/log-prob covariance
    additionally pay ``ppo_kl_coef * |log ratio|``."""
    x = _Inputs(data, config)
    frac = config.get("kl_cov_ratio", 0.0002)
    coef = config.get("ppo_kl_coef", 1.0)
    assert frac > 0, "kl_cov_ratio must be > 0"
    lr = x.log_ratio.clamp(-20.0, 20.0)
    r = torch.exp(lr)
    base = -x.adv * r
    live = x.mask > 0
    flat_idx = torch.nonzero(live.reshape(-1)).flatten()
    per_token = base
    if flat_idx.numel():
        a = x.adv[live].detach().float()
        lp = x.new[live].detach().float()
        cov = (a - a.mean()) * (lp - lp.mean())
        k = max(1, int(cov.numel() * frac))
        chosen = flat_idx[torch.topk(cov, k).indices]
        pen = torch.zeros_like(base).reshape(-1)
        pen[chosen] = 1.0
        per_token = base + pen.view_as(base) * coef * lr.abs()
    loss = x.aggregate(x.weighted(per_token))
    return loss, {"ppo_kl": masked_mean(lr.abs(), x.mask).detach().item()}


@register_loss(LossFn.GEO_MEAN)
def geo_mean_loss_fn(data, config):
    """GMPO: sequence ratio = geometric mean of token ratios whose log is clipped to
    [-low, high] on the pessimistic side; one loss term per sequence."""
    x = _Inputs(data, config)
    lo, hi = x.clip_range()
    sgn = torch.sign(x.adv)
    clamped = x.log_ratio.clamp(-lo, hi)
    chosen = sgn * torch.minimum(sgn * x.log_ratio, sgn * clamped)
    n = x.mask.sum(-1)
    seq_ratio = torch.exp((chosen * x.mask).sum(-1) / (n + 1e-8))
    seq_adv = (x.adv * x.mask).sum(-1) / (n + 1e-8)
    per_seq = -seq_adv * seq_ratio
    if x.is_w is not None:
        per_seq = per_seq * torch.exp((torch.log(x.is_w + 1e-10) * x.mask).sum(-1) / (n + 1e-8))
    has = n > 0
    loss = per_seq[has].mean() if has.any() else per_seq.mean()
    hit = clamped != x.log_ratio
    return loss, {"pg_clipfrac": x.frac(hit & (x.adv > 0)),
                  "ppo_kl": masked_mean(-x.log_ratio, x.mask).detach().item(),
                  "pg_clipfrac_lower": x.frac(hit & (x.adv < 0))}


@register_loss(LossFn.CISPO)
def cispo_loss_fn(data, config):
    """Clipped importance weight applied with stop-gradient to -A log pi; every token keeps a gradient
    unless ``token_level_mask`` drops those already outside the trust region in the advantage direction.
    The lower clip is off unless ``clip_ratio_low`` is given."""
    x = _Inputs(data, config)
    lo, hi = x.clip_range(low_default=1e10)
    r = x.ratio()
    w = r.clamp(1 - lo, 1 + hi).detach()
    per_token = -w * x.adv * x.new
    if config.get("token_level_mask", False):
        drop = ((x.adv > 0) & (r > 1 + hi)) | ((x.adv < 0) & (r < 1 - lo))
        per_token = per_token * (~drop).to(per_token.dtype)
    loss = x.aggregate(per_token)
    return loss, {"pg_clipfrac": x.frac((r > 1 + hi) | (r < 1 - lo)), "ppo_kl": x.kl()}


@register_loss(LossFn.VALUE)
def value_loss_fn(data, config):
    b = data.batch
    vpreds, values, returns, mask = b["vpreds"], b["values"], b["returns"], b["response_mask"]
    rng = config.get("cliprange_value", 0.5)
    clipped = clip_by_value(vpreds, values - rng, values + rng)
    l1, l2 = (vpreds - returns) ** 2, (clipped - returns) ** 2
    loss = 0.5 * agg_loss(loss_mat=torch.maximum(l1, l2), loss_mask=mask,
                          token_reduce=config.get("token_reduce", "sum"),
                          batch_reduce=config.get("batch_reduce", "token-mean"),
                          num_program_tokens=b.get("num_program_tokens", None),
                          num_program_steps=b.get("num_program_steps", None),
                          valid_token_count=b.get("valid_token_count", None),
                          valid_batch_size=b.get("valid_batch_size", None),
                          valid_program_count=b.get("valid_program_count", None),
                          per_row_token_count=b.get("per_row_token_count", None))
    return loss, {"vf_loss": loss.detach().item(), "vf_clipfrac": masked_mean((l2 > l1).float(), mask).detach().item(),
                  "vpred_mean": masked_mean(vpreds, mask).detach().item()}
