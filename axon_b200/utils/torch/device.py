"""Device helpers (reference: axon/utils/torch/device.py). This framework targets CUDA (B200) with a CPU
fall-back for host-side logic; there is no other accelerator branch."""
from __future__ import annotations

import os
from types import ModuleType

import torch

is_cuda_available: bool = torch.cuda.is_available()


def get_device_name() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


def get_torch_device() -> ModuleType:
    """``torch.cuda`` or ``torch.cpu``: the namespace with ``current_device`` / ``synchronize`` / ``set_device``."""
    return torch.cuda if torch.cuda.is_available() else torch.cpu


def get_device_id() -> int:
    return torch.cuda.current_device() if torch.cuda.is_available() else 0


def get_nccl_backend() -> str:
    """Collective backend for the device: nccl on GPUs, gloo on CPU-only hosts."""
    return "nccl" if torch.cuda.is_available() else "gloo"


def set_expandable_segments(enable: bool) -> None:
    """Switch the caching allocator's expandable segments (less fragmentation when tensor sizes vary)."""
    if torch.cuda.is_available():
        torch.cuda.memory._set_allocator_settings(f"expandable_segments:{bool(enable)}")
    else:
        os.environ["PYTORCH_CUDA_ALLOC_CONF"] = f"expandable_segments:{bool(enable)}"
