"""Index samplers for the task dataset (reference: axon/data/data_sampler/__init__.py:28-120).

``create_data_sampler(config, dataset)`` reads ``data_sampler`` (a built-in name or a class spec
``pkg://module:Class`` / ``/path/file.py:Class``) and ``data_sampler_args``. A dataset that carries
per-row mixing weights forces weighted random sampling with replacement.
"""
from __future__ import annotations

import inspect
import warnings
from enum import Enum

import torch

from ...utils.module_loader import load_module
from .abstract_sampler import AbstractSampler
from .curriculum_samplers import ExpWeightedCurriculumSampler, ThresholdMaskingSampler

__all__ = ["SamplerType", "create_data_sampler", "AbstractSampler", "SeededRandomSampler",
           "ExpWeightedCurriculumSampler", "ThresholdMaskingSampler"]


class SamplerType(str, Enum):
    SEQUENTIAL = "sequential"
    RANDOM = "random"
    EXP_WEIGHTED_CURRICULUM = "exp_weighted_curriculum"
    THRESHOLD_MASK_CURRICULUM = "threshold_masking_curriculum"


class SeededRandomSampler(torch.utils.data.Sampler):
    """A fresh permutation per epoch (or weighted draws with replacement) from a generator whose
    state is part of ``state_dict`` — a resumed run draws the same future epochs."""

    def __init__(self, data_source, seed: int | None = None, weights=None):
        self.n = len(data_source)
        self.weights = torch.as_tensor(weights, dtype=torch.double) if weights is not None else None
        self.generator = torch.Generator()
        if seed is not None:
            self.generator.manual_seed(int(seed))

    def __iter__(self):
        if self.n == 0:
            return iter(())
        if self.weights is not None:
            return iter(torch.multinomial(self.weights, self.n, replacement=True, generator=self.generator).tolist())
        return iter(torch.randperm(self.n, generator=self.generator).tolist())

    def __len__(self) -> int:
        return self.n

    def state_dict(self) -> dict:
        return {"generator": self.generator.get_state()}

    def load_state_dict(self, state: dict) -> None:
        self.generator.set_state(state["generator"])


def _load_class(spec: str) -> type:
    if spec.startswith("pkg://"):
        rest = spec[len("pkg://"):]
        module_path, class_name = rest.rsplit(":", 1) if ":" in rest else (rest, rest.rsplit(".", 1)[-1])
        module_path = f"pkg://{module_path}"
    elif spec.startswith("file://"):
        module_path, class_name = spec[len("file://"):].rsplit(":", 1)
    else:
        module_path, class_name = spec.rsplit(":", 1)
    return getattr(load_module(module_path), class_name)


def _accepted(cls: type, args: dict) -> dict:
    sig = inspect.signature(cls.__init__)
    if any(p.kind == inspect.Parameter.VAR_KEYWORD for p in sig.parameters.values()):
        return dict(args)
    return {k: v for k, v in args.items() if k in sig.parameters and k != "self"}


def create_data_sampler(config, dataset):
    kind = config.get("data_sampler", "sequential") or "sequential"
    kind = kind.value if isinstance(kind, SamplerType) else str(kind)
    args = dict(config.get("data_sampler_args", {}) or {})
    weights = getattr(dataset, "sample_weights", None)
    if weights is not None and kind != "random":
        warnings.warn(f"data_mix is set, so data_sampler '{kind}' is replaced by 'random'", stacklevel=2)
        kind = "random"
    if kind == "sequential":
        return torch.utils.data.SequentialSampler(dataset)
    if kind == "random":
        return SeededRandomSampler(dataset, seed=args.get("seed"), weights=weights)
    if kind == "exp_weighted_curriculum":
        cls = ExpWeightedCurriculumSampler
    elif kind == "threshold_masking_curriculum":
        cls = ThresholdMaskingSampler
    else:
        cls = _load_class(kind)
    return cls(data_source=dataset, **_accepted(cls, args))
