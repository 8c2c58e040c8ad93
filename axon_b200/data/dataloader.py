"""Loader that hands out batches of a size chosen per call and can be checkpointed mid-epoch.

``next(batch_size)`` draws the next ``batch_size`` rows in sampler order; in infinite mode a new epoch
starts transparently when the sampler runs out, otherwise ``StopIteration`` is raised once nothing is
left. ``state_dict`` records the epoch, the remaining index order of the running epoch and the
sampler's own state, so a resumed run continues with exactly the rows the interrupted run would have
seen (reference behaviour: axon/data/dataloader.py:18-165, there built on torchdata's stateful
loader; here index bookkeeping is explicit and row fetch is synchronous because rows are already in
memory).
"""
from __future__ import annotations

from typing import Callable, Iterable

import torch


class DynamicDataLoader:
    def __init__(self, dataset, collate_fn: Callable | None = None, batch_size: int = 1, infinite: bool = True,
                 sampler: Iterable[int] | None = None, **_unused):
        self._dataset = dataset
        self._collate_fn = collate_fn or torch.utils.data.default_collate
        self.batch_size = batch_size
        self.infinite = infinite
        self._sampler = sampler if sampler is not None else torch.utils.data.SequentialSampler(dataset)
        self._pending: list[int] = []          # indices of the running epoch not yet handed out
        self._epoch = 0
        self._started = False
        self._exhausted = False

    # -- iteration ---------------------------------------------------------------------------
    def __iter__(self):
        self._pending, self._started, self._exhausted = [], False, False
        return self

    def _start_epoch(self) -> bool:
        order = [int(i) for i in iter(self._sampler)]
        if self._started:
            self._epoch += 1
        self._started = True
        self._pending.extend(order)
        return bool(order)

    def next(self, batch_size: int):
        assert batch_size > 0, f"batch_size must be positive, got {batch_size}"
        while len(self._pending) < batch_size and not self._exhausted:
            if self._started and not self.infinite:
                self._exhausted = True
            elif not self._start_epoch():
                self._exhausted = True
        if not self._pending:
            raise StopIteration
        take, self._pending = self._pending[:batch_size], self._pending[batch_size:]
        return self._collate_fn([self._dataset[i] for i in take])

    def __next__(self):
        return self.next(self.batch_size)

    def __len__(self) -> int:
        return len(self._dataset)

    @property
    def dataset(self):
        return self._dataset

    @property
    def sampler(self):
        return self._sampler

    @property
    def epoch(self) -> int:
        return self._epoch

    # -- checkpointing -----------------------------------------------------------------------
    def state_dict(self) -> dict:
        state = {"pending": list(self._pending), "epoch": self._epoch, "started": self._started,
                 "exhausted": self._exhausted}
        if hasattr(self._sampler, "state_dict"):
            state["sampler_state"] = self._sampler.state_dict()
        return state

    def load_state_dict(self, state: dict) -> None:
        self._pending = list(state.get("pending", []))
        self._epoch = int(state.get("epoch", 0))
        self._started = bool(state.get("started", False))
        self._exhausted = bool(state.get("exhausted", False))
        if "sampler_state" in state and hasattr(self._sampler, "load_state_dict"):
            self._sampler.load_state_dict(state["sampler_state"])
