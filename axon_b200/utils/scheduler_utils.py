"""Learning-rate schedules as step -> multiplier functions (reference: axon/utils/scheduler_utils.py).

``PolicyEngine`` evaluates ``lr_at`` directly; these factories serve code that wants a
``torch.optim.lr_scheduler.LambdaLR`` over an ordinary torch optimizer (e.g. a LoRA adapter trained
with a stock optimizer)."""
from __future__ import annotations

import math

from torch.optim.lr_scheduler import LambdaLR


def constant_with_warmup(step: int, num_warmup_steps: int) -> float:
    return min(1.0, (step + 1) / num_warmup_steps) if num_warmup_steps > 0 else 1.0


def cosine_with_warmup(step: int, num_warmup_steps: int, num_training_steps: int, min_lr_ratio: float = 0.0,
                       num_cycles: float = 0.5) -> float:
    if num_warmup_steps > 0 and step < num_warmup_steps:
        return (step + 1) / num_warmup_steps
    span = max(1, num_training_steps - num_warmup_steps)
    p = min(1.0, (step - num_warmup_steps) / span)
    return min_lr_ratio + (1 - min_lr_ratio) * 0.5 * (1 + math.cos(math.pi * 2 * num_cycles * p))


def get_constant_schedule_with_warmup(optimizer, num_warmup_steps: int, last_epoch: int = -1) -> LambdaLR:
    return LambdaLR(optimizer, lambda s: constant_with_warmup(s, num_warmup_steps), last_epoch)


def get_cosine_schedule_with_warmup(optimizer, num_warmup_steps: int, num_training_steps: int, min_lr_ratio: float = 0.0,
                                    num_cycles: float = 0.5, last_epoch: int = -1) -> LambdaLR:
    return LambdaLR(optimizer, lambda s: cosine_with_warmup(s, num_warmup_steps, num_training_steps, min_lr_ratio, num_cycles),
                    last_epoch)
