"""Checkpoint directory discovery, validation and rotation
(reference: axon/utils/state/utils.py:20-198).

Layout of one checkpoint::

    <root>/global_step_N/            (also accepted: N/, step_N/)
        data.pt                      dataloader + driver state
        actor/                       (critic/ likewise)
            model_world_size_W_rank_R.pt      sharded modes only
            optim_world_size_W_rank_R.pt
            extra_state_world_size_W_rank_R.pt
            fsdp_config.json
            huggingface/             config + tokenizer, and weights in the hf / both modes
"""
from __future__ import annotations

import logging
import os
import re
import shutil

logger = logging.getLogger(__name__)
_DIR_PATTERNS = (re.compile(r"^(\d+)$"), re.compile(r"^step_(\d+)$"), re.compile(r"^global_step_(\d+)$"))


def is_valid_checkpoint(ckpt_path: str) -> bool:
    if not os.path.exists(os.path.join(ckpt_path, "data.pt")):
        logger.warning("checkpoint %s has no data.pt", ckpt_path)
        return False
    actor = os.path.join(ckpt_path, "actor")
    hf = os.path.join(actor, "huggingface")
    if not os.path.isdir(actor) or not os.path.isdir(hf):
        logger.warning("checkpoint %s has no actor/huggingface folder", ckpt_path)
        return False
    files = os.listdir(actor)
    if any(f.endswith(".distcp") for f in files) or "common.pt" in files:      # distributed-checkpoint layout
        return True
    for prefix in ("optim_world_size_", "extra_state_world_size_"):
        if not any(f.startswith(prefix) and f.endswith(".pt") for f in files):
            logger.warning("checkpoint %s has no '%s*.pt' shard", ckpt_path, prefix)
            return False
    shards = any(f.startswith("model_world_size_") and f.endswith(".pt") for f in files)
    hf_weights = any(f.endswith(".safetensors") or f == "pytorch_model.bin" for f in os.listdir(hf))
    if not shards and not hf_weights:
        logger.warning("checkpoint %s has neither model shards nor HF weights", ckpt_path)
        return False
    return True


def get_checkpoint_directories(path: str | None) -> list[tuple[int, str]]:
    if path is None or not os.path.isdir(path):
        return []
    found = []
    for entry in os.listdir(path):
        full = os.path.join(path, entry)
        if not os.path.isdir(full):
            continue
        for pat in _DIR_PATTERNS:
            m = pat.match(entry)
            if m:
                found.append((int(m.group(1)), full))
                break
    return sorted(found)


def delete_oldest_checkpoints(path: str, max_to_keep: int | None) -> list[str]:
    if not max_to_keep or max_to_keep <= 0:
        return []
    ckpts = get_checkpoint_directories(path)
    deleted = []
    for _, p in ckpts[: max(0, len(ckpts) - max_to_keep)]:
        try:
            shutil.rmtree(p)
            deleted.append(p)
        except OSError as e:
            logger.warning("could not delete checkpoint %s: %s", p, e)
    return deleted


def find_latest_ckpt_path(path: str | None) -> str | None:
    for _, cand in reversed(get_checkpoint_directories(path)):
        if is_valid_checkpoint(cand):
            return cand
        logger.warning("checkpoint %s is incomplete, skipping", cand)
    return None


def tensor_digest(t) -> tuple:
    """(fp64 sum, shape, position-weighted fp64 sum) of a tensor: equal tensors give equal digests, and rows that were
    swapped or shifted change the third entry."""
    import torch
    flat = t.detach().double().reshape(-1).cpu()
    w = 1.0 + (torch.arange(flat.numel(), dtype=torch.float64) % 1009) / 1009.0
    return float(flat.sum().item()), tuple(t.shape), float((flat * w).sum().item())
