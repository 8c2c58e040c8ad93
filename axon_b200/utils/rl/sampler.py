"""Sampler/trainer mismatch correction: truncated importance-sampling weights, rejection masks
(token / sequence / geometric), catastrophic-token veto, and off-policy diagnostics. All inputs are
``[B, T]`` log-probs and masks; ``log_ratio = log pi_train - log pi_sampler``.

Behaviour and metric names follow the reference (axon/utils/rl/sampler.py:35-597); metrics are
returned under the ``sampler_corr/`` prefix.
"""
from __future__ import annotations

import math
from typing import Any

import torch

SAFETY_BOUND = 20.0


def _msum(x, m, axis=None):
    return (x * m).sum() if axis is None else (x * m).sum(axis)


def _mmean(x, m, axis=None):
    if axis is None:
        return (x * m).sum() / m.sum().clamp_min(1e-8)
    return (x * m).sum(axis) / m.sum(axis).clamp_min(1e-8)


def _level_weights(log_ratio, mask, level):
    """IS weights at the requested aggregation level, broadcast to [B,T]; also the log ratio they came from."""
    if level == "token":
        basis = log_ratio
    elif level == "sequence":
        basis = _msum(log_ratio, mask, -1).unsqueeze(-1)
    elif level == "geometric":
        basis = _mmean(log_ratio, mask, -1).unsqueeze(-1)
    else:
        raise ValueError(f"unsupported aggregation level: {level}")
    return torch.exp(basis.clamp(-SAFETY_BOUND, SAFETY_BOUND)).expand_as(log_ratio), basis


def _weight_stats(w, basis, mask, prefix, upper, lower=None):
    m = mask.to(w.dtype)
    seq_level = basis.shape[-1] == 1 and w.shape[-1] != 1
    vals = w[:, 0] if seq_level else w
    vm = torch.ones_like(vals) if seq_level else m
    mean = _mmean(vals, vm)
    out = {f"{prefix}_mean": mean.item(),
           f"{prefix}_max": vals.masked_fill(vm == 0, float("-inf")).max().item(),
           f"{prefix}_min": vals.masked_fill(vm == 0, float("inf")).min().item(),
           f"{prefix}_std": (_mmean((vals - mean) ** 2, vm)).sqrt().item(),
           f"{prefix}_ratio_fraction_high": _mmean((vals > upper).float(), vm).item()}
    if lower is not None:
        out[f"{prefix}_ratio_fraction_low"] = _mmean((vals < lower).float(), vm).item()
    ess_num = _msum(vals, vm) ** 2
    out[f"{prefix}_eff_sample_size"] = (ess_num / (_msum(vals ** 2, vm) * vm.sum()).clamp_min(1e-8)).item()
    return out


def compute_sampler_rejection_mask(log_ratio, response_mask, sampler_rs="token", sampler_rs_threshold=None,
                                   sampler_rs_threshold_lower=None):
    """Zero the mask where the IS weight (at the chosen level) leaves [lower, upper]; lower defaults to 1/upper."""
    if sampler_rs not in ("token", "sequence", "geometric"):
        raise ValueError(f"Invalid sampler_rs: {sampler_rs}. Must be one of token, sequence, geometric.")
    if sampler_rs_threshold is None:
        raise ValueError("sampler_rs_threshold must be provided for rejection sampling.")
    upper = sampler_rs_threshold
    lower = sampler_rs_threshold_lower if sampler_rs_threshold_lower is not None else 1.0 / upper
    w, basis = _level_weights(log_ratio, response_mask, sampler_rs)
    keep = ((w >= lower) & (w <= upper)).float()
    metrics = _weight_stats(w, basis, response_mask, "sampler_rs", upper, lower)
    metrics["sampler_rs_masked_fraction"] = _mmean(1 - keep, response_mask).item()
    if sampler_rs == "token":
        metrics["sampler_rs_seq_masked_fraction"] = (_msum(1 - keep, response_mask, -1) > 0).float().mean().item()
    else:
        metrics["sampler_rs_seq_masked_fraction"] = (1 - keep[:, 0]).mean().item()
    return response_mask * keep, metrics


def compute_sampler_correction_weights(log_ratio, response_mask, sampler_is="token", sampler_is_threshold=2.0,
                                       sampler_is_batch_normalize=False):
    """Truncated (at ``sampler_is_threshold``), detached IS weights; optional normalisation to batch mean 1."""
    if sampler_is not in ("token", "sequence"):
        raise ValueError(f"Invalid sampler_is: {sampler_is}. Must be one of token, sequence.")
    if sampler_is_threshold <= 0:
        raise ValueError(f"sampler_is_threshold must be positive, got {sampler_is_threshold}.")
    w, basis = _level_weights(log_ratio, response_mask, sampler_is)
    w = w * response_mask
    metrics = _weight_stats(w, basis, response_mask, "sampler_is", sampler_is_threshold)
    w = w.clamp(max=sampler_is_threshold).detach()
    if sampler_is_batch_normalize:
        if sampler_is == "token":
            num, den = _msum(w, response_mask), response_mask.sum().to(w.dtype)
        else:
            seq_w = _mmean(w, response_mask, -1)
            seq_m = (response_mask.sum(-1) > 0).to(w.dtype)
            num, den = (seq_w * seq_m).sum(), seq_m.sum()
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            pair = torch.stack([num, den]).to(w.device)
            torch.distributed.all_reduce(pair)
            num, den = pair[0], pair[1]
        mean = num / den.clamp_min(1e-8)
        if mean > 1e-8:
            w = w / mean
            metrics["sampler_is_batch_norm_factor"] = mean.item()
        else:
            metrics["sampler_is_batch_norm_factor"] = 1.0
    return w, metrics


def compute_sampler_correction_and_rejection_mask(old_log_prob, sampler_log_prob, response_mask, sampler_is=None,
                                                  sampler_is_threshold=2.0, sampler_rs=None,
                                                  sampler_rs_threshold=None, sampler_rs_threshold_lower=None,
                                                  sampler_token_veto_threshold=None,
                                                  sampler_is_batch_normalize=False):
    """Returns (weights or None, modified mask, metrics). The veto removes whole sequences containing a
    token whose ratio fell below ``sampler_token_veto_threshold``."""
    if not response_mask.any():
        return None, response_mask, {}
    if old_log_prob.shape != sampler_log_prob.shape or old_log_prob.shape != response_mask.shape:
        raise ValueError(f"shape mismatch: old {tuple(old_log_prob.shape)}, sampler {tuple(sampler_log_prob.shape)}, "
                         f"mask {tuple(response_mask.shape)}")
    log_ratio = old_log_prob - sampler_log_prob
    metrics: dict[str, float] = {}
    weights = None
    if sampler_is is not None and sampler_is_threshold is not None:
        weights, m = compute_sampler_correction_weights(log_ratio, response_mask, sampler_is, sampler_is_threshold,
                                                        sampler_is_batch_normalize)
        metrics.update(m)
    mask = response_mask.clone()
    if sampler_rs is not None:
        if sampler_rs_threshold is None:
            raise ValueError("sampler_rs_threshold must be explicitly provided when sampler_rs is enabled.")
        mask, m = compute_sampler_rejection_mask(log_ratio, response_mask, sampler_rs, sampler_rs_threshold,
                                                 sampler_rs_threshold_lower)
        metrics.update(m)
    if sampler_token_veto_threshold is not None:
        if sampler_token_veto_threshold <= 0:
            raise ValueError(f"sampler_token_veto_threshold must be positive, got {sampler_token_veto_threshold}.")
        bad = (log_ratio < math.log(sampler_token_veto_threshold)) & response_mask.bool()
        seq_bad = bad.any(-1, keepdim=True)
        metrics["sampler_is_veto_fraction"] = seq_bad.float().mean().item()
        metrics["sampler_is_catastrophic_token_fraction"] = _mmean(bad.float(), response_mask).item()
        mask = mask * (~seq_bad).float()
    else:
        metrics["sampler_is_veto_fraction"] = 0.0
        metrics["sampler_is_catastrophic_token_fraction"] = 0.0
    return weights, mask, {f"sampler_corr/{k}": (v.item() if isinstance(v, torch.Tensor) else v)
                           for k, v in metrics.items()}


@torch.no_grad()
def compute_offpolicy_metrics(old_log_prob, sampler_log_prob, response_mask) -> dict[str, Any]:
    """Perplexities, KL estimates (k1 'kl', 'k3_kl') and chi-square divergences between the training
    policy and the sampler on the sampled tokens."""
    out: dict[str, Any] = {}
    mean_lp = _mmean(old_log_prob, response_mask, -1)
    out["training_ppl"] = torch.exp(-mean_lp).mean().item()
    out["training_log_ppl"] = (-mean_lp).mean().item()
    if sampler_log_prob is None:
        return out
    lr = old_log_prob - sampler_log_prob
    out["kl"] = _mmean(sampler_log_prob - old_log_prob, response_mask).item()
    out["k3_kl"] = _mmean(torch.exp(lr) - lr - 1, response_mask).item()
    mean_s = _mmean(sampler_log_prob, response_mask, -1)
    out["sampler_ppl"] = torch.exp(-mean_s).mean().item()
    out["sampler_log_ppl"] = (-mean_s).mean().item()
    d = mean_s - mean_lp
    out.update(log_ppl_diff=d.mean().item(), log_ppl_abs_diff=d.abs().mean().item(), log_ppl_diff_max=d.max().item(),
               log_ppl_diff_min=d.min().item(), ppl_ratio=torch.exp(d).mean().item())
    rho = torch.exp(lr.clamp(-SAFETY_BOUND, SAFETY_BOUND))
    out["chi2_token"] = (_mmean(rho.square(), response_mask) - 1.0).item()
    seq = _msum(lr, response_mask, -1).clamp(-SAFETY_BOUND, SAFETY_BOUND)
    out["chi2_seq"] = (torch.exp(2.0 * seq).mean() - 1.0).item()
    return out


def compute_sampler_correction_and_add_to_batch(batch, config: dict):
    """Apply the configured correction to a DataProto: always rewrites ``response_mask``; adds
    ``sampler_is_weights`` when IS is enabled. Returns (batch, metrics)."""
    with torch.no_grad():
        w, mask, metrics = compute_sampler_correction_and_rejection_mask(
            old_log_prob=batch.batch["old_log_probs"], sampler_log_prob=batch.batch["sampler_log_probs"],
            response_mask=batch.batch["response_mask"], sampler_is=config.get("sampler_is", None),
            sampler_is_threshold=config.get("sampler_is_threshold", 2.0), sampler_rs=config.get("sampler_rs", None),
            sampler_rs_threshold=config.get("sampler_rs_threshold", None),
            sampler_rs_threshold_lower=config.get("sampler_rs_threshold_lower", None),
            sampler_token_veto_threshold=config.get("sampler_token_veto_threshold", None),
            sampler_is_batch_normalize=config.get("sampler_is_batch_normalize", False))
    batch.batch["response_mask"] = mask
    if w is not None:
        batch.batch["sampler_is_weights"] = w
    return batch, metrics


def compute_sampler_corr_metrics_from_logprobs(log_prob, sampler_log_prob, response_mask) -> dict[str, float]:
    return {f"sampler_corr/{k}": v for k, v in
            compute_offpolicy_metrics(log_prob, sampler_log_prob, response_mask).items()}
