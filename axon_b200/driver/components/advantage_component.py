"""Advantage computation over a program batch (reference:
axon/driver/components/advantage_component.py:35-178).

Programs with several steps carry their reward on the last step only: the estimator runs on the
last-step rows and every earlier step of the same program receives that program's scalar advantage
(the mean over the last step's trained tokens) on its own trained tokens. Programs that supplied
per-step rewards are estimated on all rows directly.
"""
from __future__ import annotations

import numpy as np
import torch

from ...protocol import DataProto
from ...trainer.algos.advantages import compute_advantage
from ...utils.rl.utils import compute_pass_metrics, compute_reward_statistics, filter_zero_advantage_samples


def _get(config, key, default=None):
    if isinstance(config, dict):
        return config.get(key, default)
    return getattr(config, key, default)


def stepwise_advantage_broadcast(last_step_batch: DataProto, other_step_batch: DataProto):
    adv, mask = last_step_batch.batch["advantages"], last_step_batch.batch["response_mask"].float()
    scalar = (adv * mask).sum(-1) / mask.sum(-1).clamp_min(1)
    scalar = torch.where(mask.sum(-1) > 0, scalar, torch.zeros_like(scalar))
    by_uid = {str(u): scalar[i] for i, u in enumerate(last_step_batch.non_tensor_batch["program_uids"])}
    tgt_mask = other_step_batch.batch["response_mask"]
    if len(other_step_batch):
        per_row = torch.stack([by_uid[str(u)] for u in other_step_batch.non_tensor_batch["program_uids"]]).to(torch.float32)
        out = per_row[:, None] * tgt_mask
    else:
        out = torch.zeros(tgt_mask.shape, dtype=torch.float32)
    other_step_batch.batch["advantages"] = out
    other_step_batch.batch["returns"] = out.clone()
    return other_step_batch, last_step_batch


def compute_advantage_component(batch: DataProto, config, metrics: dict) -> DataProto:
    pass_metrics, rates = compute_pass_metrics(batch)
    metrics.update(pass_metrics)
    metrics.update(compute_reward_statistics(batch))
    batch.non_tensor_batch["pass_rate"] = np.array([rates.get(str(u), 0.0) for u in batch.non_tensor_batch["uid"]], dtype=np.float64)
    if "token_level_rewards" not in batch.batch:
        batch.batch["token_level_rewards"] = batch.batch["token_level_scores"]
    per_step = "has_step_rewards" in batch.non_tensor_batch and bool(
        np.any(np.asarray(batch.non_tensor_batch["has_step_rewards"], dtype=bool)))
    if per_step or "is_last_step" not in batch.non_tensor_batch:
        batch = compute_advantage(batch, config=config)
    else:
        last = np.asarray(batch.non_tensor_batch["is_last_step"], dtype=bool)
        others = batch.select_idxs(np.nonzero(~last)[0])
        batch = compute_advantage(batch.select_idxs(np.nonzero(last)[0]), config=config)
        if len(others):
            others, batch = stepwise_advantage_broadcast(batch, others)
            batch = DataProto.concat([batch, others])
    if _get(config, "drop_zero_advantage_samples", False):
        before = len(batch)
        batch = filter_zero_advantage_samples(batch)
        metrics["batch/filtered_zero_adv_count"] = before - len(batch)
        metrics["batch/filtered_zero_adv_frac"] = (before - len(batch)) / max(before, 1)
    if "advantages" in batch.batch:
        valid = batch.batch["advantages"][batch.batch["response_mask"].bool()]
        if valid.numel() > 0:
            metrics["batch/advantages_std"] = valid.std().item() if valid.numel() > 1 else 0.0
            metrics["batch/advantages_mean"] = valid.mean().item()
            metrics["batch/advantages_abs_max"] = valid.abs().max().item()
    return batch
