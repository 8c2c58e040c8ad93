"""Interface of samplers that adapt to training feedback (curriculum learning)."""
from __future__ import annotations

from abc import abstractmethod
from collections.abc import Sized

import torch


class AbstractSampler(torch.utils.data.Sampler):
    @abstractmethod
    def __init__(self, data_source: Sized, **kwargs):
        self.data_source = data_source

    @abstractmethod
    def update(self, batch) -> None:
        """Called once per step with a DataProto whose non-tensor columns ``index`` (dataset row) and
        ``pass_rate`` (fraction of the row's rollouts that succeeded) describe the step's outcome."""
