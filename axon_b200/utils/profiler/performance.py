"""Memory logging and cross-rank timing reduction (reference: axon/utils/profiler/performance.py:28-204)."""
from __future__ import annotations

import functools
import logging
from typing import Any

import torch
import torch.distributed as dist


def _mem_info(unit: str = "GB", precision: int = 2) -> tuple[str, str, str, str]:
    div = {"GB": 1 << 30, "MB": 1 << 20, "KB": 1 << 10}[unit]
    if not torch.cuda.is_available():
        return ("0",) * 4
    free, total = torch.cuda.mem_get_info()
    f = lambda x: f"{x / div:.{precision}f}"          # noqa: E731
    return f(torch.cuda.memory_allocated()), f(torch.cuda.memory_reserved()), f(total - free), f(total)


def log_gpu_memory_usage(head: str, logger: logging.Logger | None = None, level=logging.DEBUG, rank: int = 0) -> None:
    if dist.is_initialized() and rank is not None and dist.get_rank() != rank:
        return
    alloc, reserved, used, total = _mem_info()
    msg = f"{head}, memory allocated (GB): {alloc}, reserved (GB): {reserved}, device used/total (GB): {used}/{total}"
    (logger.log(level, msg) if logger is not None else print(msg, flush=True))


class GPUMemoryLogger:
    """Decorator that logs device memory before and after the wrapped method."""

    def __init__(self, role: str, logger: logging.Logger | None = None, level=logging.DEBUG, log_only_rank_0: bool = True):
        self.role, self.logger, self.level, self.rank0 = role, logger, level, log_only_rank_0

    def __call__(self, fn):
        @functools.wraps(fn)
        def wrapped(*a, **k):
            rank = 0 if self.rank0 else None
            log_gpu_memory_usage(f"{self.role} before {fn.__name__}", self.logger, self.level, rank)
            out = fn(*a, **k)
            log_gpu_memory_usage(f"{self.role} after {fn.__name__}", self.logger, self.level, rank)
            return out
        return wrapped


def reduce_timing(timing_raw: dict[str, float], reduce_op=None, group=None) -> dict[str, float]:
    """All-reduce (mean by default) a dict of section times across ranks."""
    if not timing_raw or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return dict(timing_raw)
    keys = sorted(timing_raw)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([timing_raw[k] for k in keys], dtype=torch.float64, device=dev)
    if reduce_op is None:
        dist.all_reduce(t, group=group)
        t /= dist.get_world_size(group)
    else:
        dist.all_reduce(t, op=reduce_op, group=group)
    return dict(zip(keys, t.tolist()))


def topk_reduce_ratio_min_max(timing: float, k: int = 10, group=None) -> tuple[float, float, float]:
    """(mean of the k slowest ranks / mean of all ranks, min, max) of one timing value."""
    vals = gather_timing({"t": timing}, group)["t"]
    top = sorted(vals, reverse=True)[: max(1, min(k, len(vals)))]
    mean = sum(vals) / len(vals)
    return (sum(top) / len(top)) / mean if mean > 0 else 1.0, min(vals), max(vals)


def gather_timing(timing_raw: dict[str, float], group=None) -> dict[str, list[float]]:
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return {k: [v] for k, v in timing_raw.items()}
    out: list[Any] = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, timing_raw, group=group)
    return {k: [d.get(k, 0.0) for d in out] for k in timing_raw}
