"""Colocated (hybrid engine) mode switching, trainer side
(reference: axon/trainer/mixins/sync_mixin.py:24-59).

``trainer_mode`` makes the GPU ready for training after a rollout: the optimizer shard returns from
pinned host memory (the sampler has already released its KV pool). ``rollout_mode`` is the inverse,
called before the sampler wakes: gradients are freed, the allocator cache is returned, and the optimizer
state leaves the device ONLY IF the KV pool the sampler is about to create does not fit beside it
(``rollout_optimizer_offload: auto``; ``always`` restores the reference's unconditional move). Twelve bytes of
optimizer state per parameter cross PCIe twice per step otherwise - 21 s of a 73 s step for an 8B model on a
180 GB device, where pool and state fit together."""
from __future__ import annotations

import torch

from ...controller.decorator import Dispatch, register


class SyncTrainerMixin:
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def trainer_mode(self):
        if getattr(self, "_rng_state_training", None) is not None and self.device.type == "cuda":
            torch.cuda.set_rng_state(self._rng_state_training)
        self.engine.load_optimizer()

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def rollout_mode(self, kv_bytes_needed: int | None = None):
        """``kv_bytes_needed``: size of the KV pool the colocated sampler will allocate next (None: unknown)."""
        if self.device.type == "cuda":
            self._rng_state_training = torch.cuda.get_rng_state()
        if not self._forward_only:
            self.model.params.free_grads()
            if self.device.type == "cuda":
                torch.cuda.empty_cache()
            from ..fsdp_trainer import _get
            policy = str(_get(self.config, "rollout_optimizer_offload", "auto"))
            keep = False
            if policy == "auto" and kv_bytes_needed is not None and self.device.type == "cuda":
                free, _ = torch.cuda.mem_get_info(self.device)
                keep = free >= int(kv_bytes_needed) + (4 << 30)        # head-room for the decode graphs' workspaces
            self.rollout_kept_optimizer = keep
            if not keep:
                self.engine.offload_optimizer()
        if self.device.type == "cuda":
            torch.cuda.empty_cache()


FSDPSyncTrainerMixin = SyncTrainerMixin
MegatronSyncTrainerMixin = SyncTrainerMixin
