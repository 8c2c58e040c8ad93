"""Base of the SPMD state managers (reference: axon/utils/state/state_manager.py:24-97)."""
from __future__ import annotations

import random
from enum import Enum

import numpy as np
import torch


class StateSaveMode(str, Enum):
    SHARDED = "sharded"      # per-rank model + optimizer + extra files (resume)
    HF = "hf"                # per-rank optimizer + extra files, model as HuggingFace weights
    BOTH = "both"


class BaseStateManager:
    def __init__(self, model, optimizer, lr_scheduler=None, processing_class=None, rank: int | None = None,
                 world_size: int | None = None):
        import torch.distributed as dist
        self.model, self.optimizer, self.lr_scheduler = model, optimizer, lr_scheduler
        self.processing_class = processing_class
        live = dist.is_available() and dist.is_initialized()
        self.rank = rank if rank is not None else (dist.get_rank() if live else 0)
        self.world_size = world_size if world_size is not None else (dist.get_world_size() if live else 1)

    def load_state(self, local_path: str, save_mode: str | None = None):
        raise NotImplementedError

    def save_state(self, local_path: str, global_step: int = 0, max_ckpt_to_keep: int | None = None,
                   save_mode: str | None = None, async_save: bool | None = None):
        raise NotImplementedError

    @staticmethod
    def get_rng_state() -> dict:
        state = {"cpu": torch.get_rng_state(), "numpy": np.random.get_state(), "random": random.getstate()}
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            state["cuda"] = torch.cuda.get_rng_state()
        return state

    @staticmethod
    def load_rng_state(state: dict) -> None:
        torch.set_rng_state(state["cpu"])
        np.random.set_state(state["numpy"])
        random.setstate(state["random"])
        if "cuda" in state and torch.cuda.is_available():
            torch.cuda.set_rng_state(state["cuda"])
