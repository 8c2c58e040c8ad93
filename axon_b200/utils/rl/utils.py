"""Batch-level RL statistics and filters used by the driver (reference: axon/utils/rl/utils.py:23-123)."""
from __future__ import annotations

import numpy as np
import torch

from ...protocol import DataProto

_ZERO_ADV_EPS = 1e-5


def filter_zero_advantage_samples(batch: DataProto) -> DataProto:
    """Drop rows whose advantage is zero everywhere (their gradient is zero). If nothing would be
    left, one whole prompt group is kept so that padding and data-parallel sharding still have rows."""
    adv = batch.batch["advantages"]
    keep = torch.nonzero((adv.abs() > _ZERO_ADV_EPS).any(dim=1)).flatten().tolist()
    if keep:
        return batch.select_idxs(keep) if len(keep) < len(batch) else batch
    uids = batch.non_tensor_batch.get("uid", None)
    if uids is None or len(batch) == 0:
        return batch
    return batch.select_idxs([i for i, u in enumerate(uids) if u == uids[0]])


def _program_rows(batch: DataProto) -> np.ndarray:
    n = len(batch)
    pad = np.asarray(batch.non_tensor_batch.get("is_padding", np.zeros(n, dtype=bool)), dtype=bool)
    last = np.asarray(batch.non_tensor_batch.get("is_last_step", np.ones(n, dtype=bool)), dtype=bool)
    return ~pad & last


def compute_reward_statistics(batch: DataProto) -> dict:
    """Mean / max / min program reward: one value per program (its last step), padding rows excluded."""
    rows = _program_rows(batch)
    if not rows.any():
        return {"batch/reward/mean": 0.0, "batch/reward/max": 0.0, "batch/reward/min": 0.0}
    r = batch.batch["token_level_scores"][torch.from_numpy(rows)].sum(dim=1)
    return {"batch/reward/mean": r.mean().item(), "batch/reward/max": r.max().item(), "batch/reward/min": r.min().item()}


def compute_pass_metrics(batch: DataProto) -> tuple[dict, dict]:
    """Per prompt group (``uid``): pass rate = share of programs with reward >= 1; counts of groups
    where none / all / some programs pass."""
    if "is_last_step" in batch.non_tensor_batch:
        rows = np.nonzero(np.asarray(batch.non_tensor_batch["is_last_step"], dtype=bool))[0]
    else:
        rows = np.arange(len(batch))
    rewards = batch.batch["token_level_scores"][torch.from_numpy(rows)].sum(-1).cpu().numpy()
    uids = np.asarray([str(u) for u in batch.non_tensor_batch["uid"]])[rows]
    rates: dict[str, float] = {}
    none = all_ = 0
    for uid in np.unique(uids):
        r = rewards[uids == uid]
        rates[uid] = float((r >= 1).mean())
        if (r <= 0).all():
            none += 1
        elif (r >= 1).all():
            all_ += 1
    return {"batch/solve/none": none, "batch/solve/all": all_, "batch/solve/partial": len(rates) - none - all_}, rates
