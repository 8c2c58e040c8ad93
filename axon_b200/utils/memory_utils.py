"""Device memory housekeeping and snapshots (reference: axon/utils/memory_utils.py:31-292)."""
from __future__ import annotations

import gc
import os
import time

import torch


def aggressive_empty_cache(force_sync: bool = True, max_retries: int = 3) -> None:
    """Collect garbage and return cached blocks to the driver until the reserved size stops shrinking."""
    if not torch.cuda.is_available():
        gc.collect()
        return
    for _ in range(max_retries):
        before = torch.cuda.memory_reserved()
        gc.collect()
        torch.cuda.empty_cache()
        if force_sync:
            torch.cuda.synchronize()
        if before - torch.cuda.memory_reserved() < (1 << 30):
            break


def reset_memory_stats() -> None:
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats()
        torch.cuda.reset_accumulated_memory_stats()


def get_memory_info() -> dict:
    if not torch.cuda.is_available():
        return {"allocated_gb": 0.0, "reserved_gb": 0.0, "max_allocated_gb": 0.0, "free_gb": 0.0, "total_gb": 0.0}
    free, total = torch.cuda.mem_get_info()
    g = 1 << 30
    return {"allocated_gb": torch.cuda.memory_allocated() / g, "reserved_gb": torch.cuda.memory_reserved() / g,
            "max_allocated_gb": torch.cuda.max_memory_allocated() / g, "free_gb": free / g, "total_gb": total / g}


def log_memory_usage(stage: str = "current") -> None:
    m = get_memory_info()
    print(f"[memory] {stage}: allocated {m['allocated_gb']:.2f} GB, reserved {m['reserved_gb']:.2f} GB, "
          f"peak {m['max_allocated_gb']:.2f} GB, free {m['free_gb']:.2f}/{m['total_gb']:.2f} GB", flush=True)


def optimize_memory_for_inference() -> None:
    """Before a rollout: drop caches so the KV pool can take the space."""
    aggressive_empty_cache(force_sync=True)


def optimize_memory_for_training() -> None:
    aggressive_empty_cache(force_sync=False)


def enable_memory_visualize(trace_alloc_max_entries: int = 200_000, stack_depth: int = 32) -> None:
    if torch.cuda.is_available():
        torch.cuda.memory._record_memory_history(max_entries=trace_alloc_max_entries, stacks="python")


class MemorySnapshotSampler:
    """Dumps allocator snapshots (pickle files readable by PyTorch's memory visualiser)."""

    def __init__(self, out_dir: str = "./mem_snapshots", tag: str = "periodic"):
        self.out_dir, self.tag = out_dir, tag

    def dump_memory_snapshot(self, out_dir: str | None = None, tag: str | None = None, sub_dir: str | None = None) -> str | None:
        if not torch.cuda.is_available():
            return None
        d = os.path.join(out_dir or self.out_dir, sub_dir) if sub_dir else (out_dir or self.out_dir)
        os.makedirs(d, exist_ok=True)
        rank = int(os.environ.get("RANK", "0"))
        path = os.path.join(d, f"{tag or self.tag}_rank{rank}_{int(time.time())}.pickle")
        torch.cuda.memory._dump_snapshot(path)
        return path
