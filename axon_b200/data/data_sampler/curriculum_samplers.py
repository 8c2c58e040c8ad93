"""Curriculum samplers driven by per-task pass rates
(reference: axon/data/data_sampler/curriculum_samplers.py:23-121)."""
from __future__ import annotations

import math
from collections.abc import Sized

import numpy as np

from .abstract_sampler import AbstractSampler


class ExpWeightedCurriculumSampler(AbstractSampler):
    """Draws rows with replacement in proportion to a weight that falls off with the pass rate:
    solved rows (> 0.8) get ``min_weight``, unsolved ones (< 0.2) ``max_weight``, the rest
    ``exp(centroid - pass_rate)``."""

    def __init__(self, data_source: Sized, min_weight: float = 0.2, max_weight: float = 1.0, seed: int | None = None):
        self.data_source = data_source
        self.num_samples = len(data_source)
        self.weights = np.ones(self.num_samples, dtype=np.float64)
        self.centroid = 0.0
        self.min_weight, self.max_weight = min_weight, max_weight
        self.rng = np.random.default_rng(seed)

    def __iter__(self):
        total = self.weights.sum()
        p = self.weights / total if total > 0 else None
        return iter(self.rng.choice(self.num_samples, size=self.num_samples, replace=True, p=p).tolist())

    def __len__(self) -> int:
        return self.num_samples

    def update(self, batch) -> None:
        idx = np.asarray(batch.non_tensor_batch["index"], dtype=np.int64)
        rate = np.asarray(batch.non_tensor_batch["pass_rate"], dtype=np.float64)
        for i, k in zip(idx, rate):
            self.weights[i] = self.min_weight if k > 0.8 else self.max_weight if k < 0.2 else math.exp(self.centroid - k)

    def state_dict(self) -> dict:
        return {"weights": self.weights.tolist(), "rng": self.rng.bit_generator.state}

    def load_state_dict(self, state: dict) -> None:
        self.weights = np.asarray(state["weights"], dtype=np.float64)
        if "rng" in state:
            self.rng.bit_generator.state = state["rng"]


class ThresholdMaskingSampler(AbstractSampler):
    """Uniform over rows that are not masked; a row is masked for good once its running mean pass
    rate reaches ``threshold``. When everything is masked the whole dataset is used again."""

    def __init__(self, data_source: Sized, threshold: float = 0.9, seed: int | None = None):
        self.data_source = data_source
        self.num_samples = len(data_source)
        self.threshold = threshold
        self.pass_sum = np.zeros(self.num_samples, dtype=np.float32)
        self.invoke_count = np.zeros(self.num_samples, dtype=np.int32)
        self.masked = np.zeros(self.num_samples, dtype=bool)
        self.rng = np.random.default_rng(seed)

    def __iter__(self):
        active = np.nonzero(~self.masked)[0]
        if active.size == 0:
            active = np.arange(self.num_samples)
        return iter(self.rng.choice(active, size=self.num_samples, replace=True).tolist())

    def __len__(self) -> int:
        return self.num_samples

    def update(self, batch) -> None:
        idx = np.asarray(batch.non_tensor_batch["index"], dtype=np.int64)
        rate = np.asarray(batch.non_tensor_batch["pass_rate"], dtype=np.float32)
        np.add.at(self.pass_sum, idx, rate)
        np.add.at(self.invoke_count, idx, 1)
        done = self.pass_sum[idx] / self.invoke_count[idx] >= self.threshold
        self.masked[idx[done]] = True

    def state_dict(self) -> dict:
        return {"masked": self.masked.tolist(), "pass_sum": self.pass_sum.tolist(),
                "invoke_count": self.invoke_count.tolist(), "rng": self.rng.bit_generator.state}

    def load_state_dict(self, state: dict) -> None:
        self.masked = np.asarray(state["masked"], dtype=bool)
        self.pass_sum = np.asarray(state["pass_sum"], dtype=np.float32)
        self.invoke_count = np.asarray(state["invoke_count"], dtype=np.int32)
        if "rng" in state:
            self.rng.bit_generator.state = state["rng"]
