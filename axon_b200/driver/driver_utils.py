"""Driver-side batch plumbing: dataloader rows -> DataProto, padding to the workers' world sizes,
token balancing across data-parallel ranks, mini-batch splitting by program, mini-batch-global loss
denominators, and the PPO update loop (reference: axon/driver/driver_utils.py:50-618).
"""
from __future__ import annotations

import math
import uuid
from dataclasses import dataclass, field
from functools import reduce
from typing import Any

import numpy as np
import torch

from ..protocol import DataProto, pad_dataproto_to_divisor
from ..utils.metrics import append_to_dict, reduce_metrics
from ..utils.seqlen_balancing import calculate_workload, get_seqlen_balanced_partitions, log_seqlen_unbalance

PAD_FILLER_TOKEN_ID = 0


@dataclass
class RoleWorkerConfig:
    """Worker class + resource pool (+ constructor kwargs) of one role."""
    cls: type
    resource_pool: Any
    init_kwargs: dict[str, Any] = field(default_factory=dict)
    max_concurrency: int | None = None


def convert_batch_dict_to_dataproto(batch_dict: dict, global_steps: int, n_samples: int = 1, temperature_scheduler=None,
                                    temperature_config=None, val: bool = False, val_n_samples: int | None = None) -> DataProto:
    """One row per dataset task with a fresh group ``uid``, repeated (interleaved) ``n`` times so the
    n rollouts of a task share that uid."""
    env_args = batch_dict.get("env_args", [])
    n = len(env_args)
    non_tensors = {"uid": np.array([str(uuid.uuid4()) for _ in range(n)], dtype=object)}
    if n:
        arr = np.empty(n, dtype=object)
        arr[:] = list(env_args)
        non_tensors["env_args"] = arr
    if "index" in batch_dict:
        non_tensors["index"] = np.asarray(batch_dict["index"])
    batch = DataProto.from_dict(tensors={}, non_tensors=non_tensors)
    batch.meta_info.update({"sample_params": {}, "global_steps": global_steps})
    enabled = getattr(temperature_config, "enable", False) if temperature_config is not None else False
    if isinstance(temperature_config, dict):
        enabled = temperature_config.get("enable", False)
    if not val and temperature_scheduler is not None and enabled:
        batch.meta_info["sample_params"]["temperature"] = temperature_scheduler.get_temperature(max(global_steps - 1, 0))
    rep = val_n_samples if val else n_samples
    if rep and rep > 1:
        batch = batch.repeat(repeat_times=rep, interleave=True)
    return batch


class ValidationResult:
    """Accumulates validation rewards; ``pass@n`` counts a task solved when its best rollout scores >= 1."""

    def __init__(self, n_samples: int = 1):
        self.n_samples = n_samples
        self.rewards: list[float] = []
        self.uids: list[str] = []
        self.data_sources: list[str] = []

    def add(self, reward: float, uid: str, data_source: str = "unknown") -> None:
        self.rewards.append(float(reward))
        self.uids.append(uid)
        self.data_sources.append(data_source)

    def compute_metrics(self) -> dict:
        if not self.rewards:
            return {}
        r = np.asarray(self.rewards, dtype=np.float64)
        best: dict[str, float] = {}
        for x, u in zip(self.rewards, self.uids):
            best[u] = max(best.get(u, float("-inf")), x)
        out = {"val/reward": float(r.mean()), "val/reward_clip[-1, 1]": float(np.clip(r, -1, 1).mean()),
               "val/reward_clip[0, 1]": float(np.clip(r, 0, 1).mean()),
               f"val/pass@{self.n_samples}": float(np.mean([b >= 1 for b in best.values()]))}
        sources = set(self.data_sources)
        if len(sources) > 1:
            for s in sorted(sources):
                sel = np.asarray([d == s for d in self.data_sources])
                out[f"val/{s}/reward"] = float(r[sel].mean())
        return out


# ------------------------------------------------------------------------------------------ padding
def _mark_padding_rows(batch: DataProto, rows: slice) -> None:
    """Rows that padding copied in become inert: unique ids (never grouped with real programs), no
    trained tokens, flagged ``is_padding``."""
    start = rows.start or 0
    stop = rows.stop if rows.stop is not None else len(batch)
    nt = batch.non_tensor_batch
    for i in range(start, stop):
        gid, pid = str(uuid.uuid4()), str(uuid.uuid4())
        for key, val in (("uid", gid), ("program_group_ids", gid), ("program_uids", pid), ("step_ids", str(uuid.uuid4())),
                         ("program_step_ids", f"{pid}_padding_step0"), ("multi_modal_inputs", {})):
            if key in nt:
                nt[key][i] = val
    for key, val in (("num_program_steps", 1), ("is_last_step", False), ("has_step_rewards", False), ("is_padding", True),
                     ("index", -1)):
        if key in nt:
            nt[key][rows] = val
    if batch.batch is not None:
        if "response_mask" in batch.batch:
            batch.batch["response_mask"][rows] = 0
        for key in ("token_level_scores", "token_level_rewards", "advantages", "returns"):
            if key in batch.batch:
                batch.batch[key][rows] = 0
        if "multi_modal_inputs" in nt and "input_ids" in batch.batch:
            batch.batch["input_ids"][rows] = PAD_FILLER_TOKEN_ID


def pad_dataproto_to_world_size(batch: DataProto, world_sizes: list[int]) -> DataProto:
    """Pad to a multiple of the least common multiple of all worker-group sizes."""
    if not world_sizes:
        return batch
    n0 = len(batch)
    batch, pad = pad_dataproto_to_divisor(batch, reduce(math.lcm, world_sizes))
    if pad > 0:
        _mark_padding_rows(batch, slice(n0, n0 + pad))
    return batch


def _pad_mini_batch(mb: DataProto, world_size: int) -> DataProto:
    if world_size <= 1:
        return mb
    n0 = len(mb)
    mb, pad = pad_dataproto_to_divisor(mb, world_size)
    if pad > 0:
        _mark_padding_rows(mb, slice(n0, n0 + pad))
    return mb


# ---------------------------------------------------------------------------------------- balancing
def _program_groups(program_uids) -> dict[str, list[int]]:
    groups: dict[str, list[int]] = {}
    for i, u in enumerate(program_uids):
        groups.setdefault(str(u), []).append(i)
    return groups


def _balance_by_programs(batch: DataProto, world_size: int, program_uids, is_padding):
    """Longest-processing-time assignment of whole programs to ranks (fewest rows first, then least
    tokens), padding rows handed out last; extra padding rows are appended when the ranks' row counts
    cannot otherwise be made equal."""
    seqlens = batch.batch["attention_mask"].sum(-1).tolist()
    real, pad_rows = [], []
    for uid, idxs in _program_groups(program_uids).items():
        if is_padding is not None and all(bool(is_padding[i]) for i in idxs):
            pad_rows.extend(idxs)
        else:
            real.append((sum(seqlens[i] for i in idxs), idxs))
    real.sort(key=lambda x: -x[0])
    parts: list[list[int]] = [[] for _ in range(world_size)]
    rows, load = [0] * world_size, [0.0] * world_size
    for w, idxs in real:
        p = min(range(world_size), key=lambda r: (rows[r], load[r]))
        parts[p].extend(idxs)
        rows[p] += len(idxs)
        load[p] += w
    target = math.ceil(max(rows) / world_size) * world_size if max(rows) else world_size
    spare = iter(pad_rows)
    for p in range(world_size):
        while rows[p] < target:
            i = next(spare, None)
            if i is None:
                break
            parts[p].append(i)
            rows[p] += 1
    missing = target * world_size - sum(rows)
    if missing > 0:
        n0 = len(batch)
        batch, _ = pad_dataproto_to_divisor(batch, n0 + missing)
        _mark_padding_rows(batch, slice(n0, len(batch)))
        nxt = n0
        for p in range(world_size):
            while rows[p] < target:
                parts[p].append(nxt)
                rows[p] += 1
                nxt += 1
    return batch, parts


def balance_batch(batch: DataProto, world_size: int, metrics: dict, logging_prefix: str = "global_seqlen") -> DataProto:
    """Reorder rows so that chunking into ``world_size`` contiguous shards gives every rank a similar
    token load; with ``program_uids`` present, all steps of a program land on one rank. Within a rank
    rows are arranged short-long-...-long-short so consecutive micro-batches are similar too."""
    nt = batch.non_tensor_batch or {}
    if nt.get("program_uids") is not None:
        batch, parts = _balance_by_programs(batch, world_size, nt["program_uids"], nt.get("is_padding"))
    else:
        lens = batch.batch["attention_mask"].sum(-1)
        parts = get_seqlen_balanced_partitions(calculate_workload(lens).tolist(), k_partitions=world_size, equal_size=True)
    lens = batch.batch["attention_mask"].view(len(batch), -1).sum(-1)
    work = calculate_workload(lens).tolist()
    for k, part in enumerate(parts):
        part = sorted(part, key=lambda i: (work[i], i))
        parts[k] = part[::2] + part[1::2][::-1]
    batch.reorder(torch.tensor([i for part in parts for i in part], dtype=torch.long))
    # after the reorder partition k is the k-th contiguous block
    sizes = [len(p) for p in parts]
    offs = np.concatenate([[0], np.cumsum(sizes)])
    new_parts = [list(range(int(offs[k]), int(offs[k + 1]))) for k in range(len(parts))]
    new_lens = batch.batch["attention_mask"].view(len(batch), -1).sum(-1).tolist()
    metrics.update(log_seqlen_unbalance(seqlen_list=new_lens, partitions=new_parts, prefix=logging_prefix))
    return batch


# ------------------------------------------------------------------------------------- mini-batches
def process_mini_batch(mini_batch: DataProto) -> None:
    """Attach the mini-batch-wide denominators the loss reductions divide by, as per-row constant
    columns so they survive data-parallel chunking: ``valid_batch_size`` (rows with a trained token),
    ``valid_token_count``, ``per_row_token_count`` and ``valid_program_count``."""
    mask = mini_batch.batch.get("response_mask", None) if mini_batch.batch is not None else None
    if mask is None:
        return
    n = len(mini_batch)
    per_row = mask.sum(-1).to(torch.long)
    valid = per_row > 0
    mini_batch.batch["valid_batch_size"] = torch.full((n,), int(valid.sum()), dtype=torch.long)
    mini_batch.batch["valid_token_count"] = torch.full((n,), int(per_row.sum()), dtype=torch.long)
    mini_batch.batch["per_row_token_count"] = per_row
    uids = (mini_batch.non_tensor_batch or {}).get("program_uids")
    if uids is not None:
        count = len({str(uids[i]) for i in torch.nonzero(valid).flatten().tolist()})
        mini_batch.batch["valid_program_count"] = torch.full((n,), count, dtype=torch.long)


def split_mini_batches_by_programs(batch: DataProto, mini_batch_size: int, world_size: int, shuffle: bool = False,
                                   generator: torch.Generator | None = None) -> list[DataProto]:
    """Mini-batches of ``mini_batch_size`` PROGRAMS (all rows of a program together), each padded to a
    multiple of ``world_size`` rows."""
    groups = _program_groups(batch.non_tensor_batch["program_uids"])
    uids = list(groups)
    if mini_batch_size >= len(uids):
        if shuffle:
            batch = batch.select_idxs(torch.randperm(len(batch), generator=generator).tolist())
        return [_pad_mini_batch(batch, world_size)]
    if shuffle:
        uids = [uids[j] for j in torch.randperm(len(uids), generator=generator).tolist()]
    out = []
    for s in range(0, len(uids), mini_batch_size):
        rows = [i for u in uids[s:s + mini_batch_size] for i in groups[u]]
        out.append(_pad_mini_batch(batch.select_idxs(rows), world_size))
    return out


def update_trainer(batch: DataProto, training_client, loss_fn: str, loss_fn_args: dict, epochs: int = 1,
                   mini_batch_size: int | None = None, mini_batch_shuffle: bool = False, mini_batch_seed: int | None = None,
                   world_size: int = 1) -> dict:
    """PPO epochs x mini-batches: each mini-batch gets its global denominators, one
    ``forward_backward`` and one ``optim_step`` (the LR schedule advances on the last one only)."""
    metrics: dict[str, list] = {}
    mini_batch_size = mini_batch_size or len(batch)
    gen = torch.Generator().manual_seed(mini_batch_seed) if mini_batch_seed is not None else None
    for epoch in range(epochs):
        mbs = split_mini_batches_by_programs(batch, mini_batch_size, world_size, shuffle=mini_batch_shuffle, generator=gen)
        for i, mb in enumerate(mbs):
            process_mini_batch(mb)
            out = training_client.forward_backward(mb, loss_fn=loss_fn, loss_fn_args=loss_fn_args)
            append_to_dict(metrics, out.meta_info["metrics"])
            last = epoch == epochs - 1 and i == len(mbs) - 1
            out = training_client.optim_step(step_lr=last)
            append_to_dict(metrics, out.meta_info["metrics"])
    return reduce_metrics(metrics)
