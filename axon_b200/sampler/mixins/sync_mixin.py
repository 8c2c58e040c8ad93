"""Colocated (hybrid engine) weight hand-over, sampler side
(reference: axon/sampler/mixins/sync_mixin.py:86-247).

The reference materialises every parameter out of its sharded trainer (all-gathers), renames it and
loads it into the inference engine. Here the sampler and the trainer of a GPU share one flat
parameter buffer, so ``sampler_mode`` moves no weight at all: it asks the colocated trainer to
make room (gradients freed; optimizer state to pinned host memory only when the KV pool would not fit beside it),
re-creates the KV pool and resumes the server. A sampler that does NOT share the buffer (separate process) falls back to
pulling named tensors from its fused trainer peer."""
from __future__ import annotations

from ...controller.decorator import Dispatch, register


class SyncSamplerMixin:
    def _trainer_peer(self):
        peers = getattr(self, "_fused_peers", None) or {}
        for role, p in peers.items():
            if role != self.name and hasattr(p, "engine") and not getattr(p, "_forward_only", False) and hasattr(p, "rollout_mode"):
                return p
        return None

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def sampler_mode(self):
        peer = self._trainer_peer()
        if peer is not None:
            need = None
            eng = getattr(self, "engine", None)
            if eng is not None and getattr(eng, "_num_pages", None):
                from ..kv_cache import PagedKVCache
                need = int(eng._num_pages) * PagedKVCache.bytes_per_page(eng.cfg, eng.model.params.flat.element_size())
            peer.rollout_mode(need)
            if not self.shares_trainer_weights:
                # a trainer with parameter shards gathers whole tensors layer by layer (every rank takes part)
                gathered = getattr(peer.model, "full_named_tensors", None)
                if gathered is None and getattr(getattr(peer, "state_manager", None), "mp_group", None) is not None:
                    gathered = peer.state_manager.full_named_tensors       # tensor / expert / pipeline shards of a model-parallel trainer
                self.server.update_weights(gathered() if gathered is not None else peer.model.params.views.items())
        self.server.wake_up()

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def trainer_mode(self):
        self.server.sleep()
        peer = self._trainer_peer()
        if peer is not None:
            peer.trainer_mode()


FSDPSyncSamplerMixin = SyncSamplerMixin
MegatronSyncSamplerMixin = SyncSamplerMixin
