"""Sampling-temperature schedule over training steps: linear, exponential or cosine between a start
and an end temperature (reference: axon/utils/temperature_scheduler.py:20-128)."""
from __future__ import annotations

import math

_KINDS = ("linear", "exponential", "cosine")


class TemperatureScheduler:
    def __init__(self, config):
        g = config.get if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
        self.enabled = bool(g("enable", False))
        self.scheduler_type = g("scheduler", "linear")
        self.start_temperature = float(g("start_temperature", 1.0))
        self.end_temperature = float(g("end_temperature", 1.0))
        self.num_steps = int(g("num_steps", 1000))
        self.current_step = 0
        if self.start_temperature <= 0 or self.end_temperature <= 0:
            raise ValueError("temperatures must be positive")
        if self.scheduler_type not in _KINDS:
            raise ValueError(f"invalid scheduler type '{self.scheduler_type}' (expected one of {_KINDS})")
        if self.num_steps <= 0:
            raise ValueError("num_steps must be positive")

    def get_temperature(self, step: int | None = None) -> float:
        if not self.enabled:
            return self.start_temperature
        p = min((self.current_step if step is None else step) / self.num_steps, 1.0)
        a, b = self.start_temperature, self.end_temperature
        if self.scheduler_type == "linear":
            return a + (b - a) * p
        if self.scheduler_type == "exponential":
            return a * (b / a) ** p
        return b + (a - b) * (1 + math.cos(math.pi * p)) / 2

    def step(self) -> None:
        if self.enabled:
            self.current_step += 1

    def reset(self) -> None:
        self.current_step = 0

    def set_step(self, step: int) -> None:
        if step < 0:
            raise ValueError("step must be non-negative")
        self.current_step = step
