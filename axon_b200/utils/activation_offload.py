"""Activation offload: what a layer keeps for backward waits in pinned host memory.

The reference wraps layers in saved-tensor hooks with a synchronous and a double-buffered asynchronous
handler (``SynchronizedGroupOffloadHandler`` / ``AsyncDoubleBufferGroupOffloadHandler``,
axon/utils/fsdp/activation_offload.py:137-436; enabled by ``enable_activation_offloading``, l.537-603).
Here the model's backward is explicit, so no hooks are needed: the trunk hands each layer's kept tensors
to ``stash`` right after the layer ran and asks for them back with ``fetch`` when backward reaches the
layer. Copies run on two side streams; ``fetch(l)`` also starts bringing layer ``l - 1`` back, so at
most two layers' activations are on the device during backward, and the device copies of forward are
released as soon as their device-to-host copy has been queued behind them.
Host buffers are pinned and reused across steps (keyed by shape and dtype). On CPU tensors everything
is a pass-through.
"""
from __future__ import annotations

import torch


class ActivationOffloader:
    def __init__(self, device, min_bytes: int = 1 << 20):
        self.device = torch.device(device)
        self.active = self.device.type == "cuda"
        self.min_bytes = min_bytes            # smaller tensors (rstd, lse of short batches) stay on the device
        self._pool: dict = {}                 # (shape, dtype) -> free pinned buffers
        self._slots: dict = {}                # layer -> {"host": obj, "dev": obj | None, "event": Event | None}
        if self.active:
            self.s_out = torch.cuda.Stream(device=self.device)
            self.s_in = torch.cuda.Stream(device=self.device)
        self._pending_release: list = []      # pinned buffers whose host-to-device copy has been queued
        self.stats = dict(offloaded_bytes=0, fetched_bytes=0, kept_bytes=0)

    # ------------------------------------------------------------------ helpers
    def _host_like(self, t: torch.Tensor) -> torch.Tensor:
        key = (tuple(t.shape), t.dtype)
        free = self._pool.setdefault(key, [])
        return free.pop() if free else torch.empty(t.shape, dtype=t.dtype, pin_memory=True)

    def _release(self, h: torch.Tensor) -> None:
        self._pool.setdefault((tuple(h.shape), h.dtype), []).append(h)

    def _map(self, obj, fn):
        if isinstance(obj, torch.Tensor):
            return fn(obj)
        if isinstance(obj, dict):
            return {k: self._map(v, fn) for k, v in obj.items()}
        if isinstance(obj, (list, tuple)):
            return type(obj)(self._map(v, fn) for v in obj)
        return obj

    # ------------------------------------------------------------------ forward side
    def stash(self, layer: int, saved):
        """Queue the device-to-host copies of ``saved`` (a tensor or a nest of tensors) and give up the
        device references. Returns a token for ``fetch``."""
        if not self.active:
            self._slots[layer] = {"host": saved, "dev": saved, "event": None}
            return layer
        cur = torch.cuda.current_stream(self.device)
        self.s_out.wait_stream(cur)

        def out(t: torch.Tensor):
            if not t.is_cuda or t.numel() * t.element_size() < self.min_bytes:
                self.stats["kept_bytes"] += t.numel() * t.element_size()
                return t
            h = self._host_like(t)
            with torch.cuda.stream(self.s_out):
                h.copy_(t, non_blocking=True)
            t.record_stream(self.s_out)           # the allocator may reuse t's memory only after the copy
            self.stats["offloaded_bytes"] += t.numel() * t.element_size()
            return ("host", h, t.device)
        self._slots[layer] = {"host": self._map(saved, out), "dev": None, "event": None}
        return layer

    # ------------------------------------------------------------------ backward side
    def _start_fetch(self, layer: int) -> None:
        slot = self._slots.get(layer)
        if slot is None or slot["dev"] is not None or not self.active:
            return
        self.s_in.wait_stream(self.s_out)         # the host copy of this layer must be complete

        def walk(obj):
            if isinstance(obj, tuple) and len(obj) == 3 and obj[0] == "host":
                _, h, dev = obj
                with torch.cuda.stream(self.s_in):
                    d = torch.empty(h.shape, dtype=h.dtype, device=dev)
                    d.copy_(h, non_blocking=True)
                self.stats["fetched_bytes"] += h.numel() * h.element_size()
                self._pending_release.append(h)
                return d
            if isinstance(obj, dict):
                return {k: walk(v) for k, v in obj.items()}
            if isinstance(obj, list):
                return [walk(v) for v in obj]
            return obj
        slot["dev"] = walk(slot["host"])
        ev = torch.cuda.Event()
        ev.record(self.s_in)
        slot["event"] = ev

    def fetch(self, layer: int, prefetch: int | None = None):
        """The kept tensors of ``layer`` on the device (waits for their copy), then starts bringing
        ``prefetch`` (default ``layer - 1``) back."""
        self._start_fetch(layer)
        slot = self._slots.pop(layer)
        if self.active:
            cur = torch.cuda.current_stream(self.device)
            if slot["event"] is not None:
                cur.wait_event(slot["event"])
            # the tensors were allocated on the copy stream: tell the allocator that the compute stream uses them
            self._map(slot["dev"], lambda t: (t.record_stream(cur), t)[1] if t.is_cuda else t)
        nxt = layer - 1 if prefetch is None else prefetch
        if nxt in self._slots:
            self._start_fetch(nxt)
        return slot["dev"]

    def end_step(self) -> None:
        """Call after backward: returns the step's pinned buffers to the pool (their copies have been
        consumed by kernels that are stream-ordered before this point's synchronisation)."""
        if self.active:
            self.s_in.synchronize()
        for h in self._pending_release:
            self._release(h)
        self._pending_release = []
        self._slots.clear()
