"""Colocated (hybrid engine) mode switching, trainer side
(reference: axon/trainer/mixins/sync_mixin.py:24-59).

``trainer_mode`` makes the GPU ready for training after a rollout: the optimizer shard returns from
pinned host memory (the sampler has already released its KV pool). ``rollout_mode`` is the inverse,
called before the sampler wakes: optimizer state leaves the device and the allocator cache is
returned so the KV pool can take the space."""
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
    def rollout_mode(self):
        if self.device.type == "cuda":
            self._rng_state_training = torch.cuda.get_rng_state()
        if not self._forward_only:
            self.engine.offload_optimizer()
            self.model.params.free_grads()
        if self.device.type == "cuda":
            torch.cuda.empty_cache()


FSDPSyncTrainerMixin = SyncTrainerMixin
MegatronSyncTrainerMixin = SyncTrainerMixin
