"""Process-group bootstrap helpers (reference: axon/utils/torch/distributed.py)."""
from __future__ import annotations

import logging
import os
from datetime import timedelta

import torch
import torch.distributed as dist

from .device import get_nccl_backend

logger = logging.getLogger(__name__)


def set_numa_affinity(local_rank: int | None = None) -> bool:
    """Pin this process to the CPU cores NVML reports as close to its GPU. Reads the affinity mask (a query,
    nothing on the GPU changes) and applies it to the process; returns whether anything was set."""
    try:
        import pynvml
    except ImportError:
        logger.warning("pynvml not available, skipping NUMA affinity setup")
        return False
    started = False
    try:
        pynvml.nvmlInit()
        started = True
        idx = int(os.environ.get("LOCAL_RANK", 0)) if local_rank is None else local_rank
        handle = pynvml.nvmlDeviceGetHandleByIndex(idx)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = {64 * w + b for w, word in enumerate(mask) for b in range(64) if (word >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if cpus:
            os.sched_setaffinity(0, cpus)
            return True
    except Exception as e:      # noqa: BLE001 - no NVML device, container without the permission, ...
        logger.warning("Failed to set NUMA affinity: %s", e)
    finally:
        if started:
            pynvml.nvmlShutdown()
    return False


def initialize_global_process_group(timeout_second: int = 36000):
    """Reads RANK / LOCAL_RANK / WORLD_SIZE (and DIST_INIT_METHOD) and joins the default group."""
    dist.init_process_group(get_nccl_backend(), timeout=timedelta(seconds=timeout_second),
                            init_method=os.environ.get("DIST_INIT_METHOD", None))
    local_rank, rank, world_size = int(os.environ["LOCAL_RANK"]), int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if torch.cuda.is_available():
        torch.cuda.set_device(local_rank)
    return local_rank, rank, world_size


def destroy_global_process_group() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()
