"""KL estimators and coefficient controllers (reference: axon/utils/rl/kl.py:53-316).

``kl_penalty(logprob, ref_logprob, kind)`` with kinds k1/``kl``, ``abs``, k2/``mse``, k3/``low_var_kl``;
a trailing ``+`` keeps the estimator's value but routes the gradient through the k2 form
(straight-through), which is unbiased for the KL gradient."""
from __future__ import annotations

import math

import torch


class FixedKLController:
    def __init__(self, kl_coef: float):
        self.value = kl_coef

    def update(self, current_kl: float, n_steps: int) -> None:
        return None


class AdaptiveKLController:
    """Proportional controller (Ziegler et al. 2019): the coefficient is multiplied by
    ``1 + clip(kl/target - 1, +-0.2) * n_steps / horizon`` after every batch."""

    def __init__(self, init_kl_coef: float, target_kl: float, horizon: int):
        self.value, self.target, self.horizon = init_kl_coef, target_kl, horizon

    def update(self, current_kl: float, n_steps: int) -> None:
        if self.target == 0:
            err = 0.0 if current_kl == 0 else math.copysign(0.2, current_kl)
        else:
            err = min(0.2, max(-0.2, current_kl / self.target - 1))
        self.value *= 1 + err * n_steps / self.horizon


def get_kl_controller(kl_ctrl):
    get = (lambda k, d=None: kl_ctrl.get(k, d)) if isinstance(kl_ctrl, dict) else (lambda k, d=None: getattr(kl_ctrl, k, d))
    kind = get("type")
    if kind == "fixed":
        return FixedKLController(get("kl_coef"))
    if kind == "adaptive":
        assert get("horizon") > 0, f"horizon must be larger than 0. Got {get('horizon')}"
        return AdaptiveKLController(get("kl_coef"), get("target_kl"), get("horizon"))
    raise NotImplementedError(f"Unknown KL controller type: {kind}")


def kl_penalty_forward(logprob: torch.Tensor, ref_logprob: torch.Tensor, kl_penalty_type: str = "low_var_kl"):
    kind = kl_penalty_type.rstrip("+")
    d = logprob - ref_logprob
    if kind in ("kl", "k1"):
        return d
    if kind == "abs":
        return d.abs()
    if kind in ("mse", "k2"):
        return 0.5 * d.square()
    if kind in ("low_var_kl", "k3"):
        x = (-d).clamp(-20, 20)
        return (torch.exp(x) - x - 1).contiguous().clamp(-10, 10)
    if kind == "full":
        raise NotImplementedError("Full KL divergence requires logits, not just log probs")
    raise NotImplementedError(f"Unknown KL penalty type: {kl_penalty_type}")


def kl_penalty(logprob: torch.Tensor, ref_logprob: torch.Tensor, kl_penalty_type: str = "low_var_kl"):
    value = kl_penalty_forward(logprob, ref_logprob, kl_penalty_type)
    if not kl_penalty_type.endswith("+") or kl_penalty_type in ("mse", "k2"):
        return value
    through = 0.5 * (logprob - ref_logprob).square()
    return through - through.detach() + value.detach()


def compute_rewards_with_kl(token_level_scores, old_log_prob, ref_log_prob, kl_coef: float):
    return token_level_scores - (old_log_prob - ref_log_prob) * kl_coef


def apply_kl_penalty(token_level_scores, old_log_probs, ref_log_prob, response_mask, kl_ctrl, kl_penalty_type="kl"):
    """r_t = score_t - beta * KL_t; updates the controller with the mean per-sequence KL."""
    kld = kl_penalty(old_log_probs, ref_log_prob, kl_penalty_type) * response_mask
    beta = kl_ctrl.value
    rewards = token_level_scores - beta * kld
    current = (kld.sum(-1) / response_mask.sum(-1).clamp(min=1)).mean().item()
    kl_ctrl.update(current_kl=current, n_steps=token_level_scores.shape[0])
    return rewards, {"actor/reward_kl_penalty": current, "actor/reward_kl_penalty_coeff": beta}
