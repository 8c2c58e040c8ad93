"""Console logging helpers used by the drivers and workers (reference: axon/utils/logger/aggregate_logger.py)."""
from __future__ import annotations

import datetime
import logging
import numbers


def concat_dict_to_str(data: dict, step) -> str:
    """``step:N - key:value - ...`` over the numeric entries."""
    return " - ".join([f"step:{step}"] + [f"{k}:{v!r}" for k, v in data.items() if isinstance(v, numbers.Number)])


class LocalLogger:
    """Tracking backend that prints one line per step (``tracking: ["console"]``)."""

    def __init__(self, print_to_console: bool = True):
        self.print_to_console = print_to_console

    def flush(self) -> None:
        pass

    def log(self, data: dict, step) -> None:
        if self.print_to_console:
            print(concat_dict_to_str(data, step=step), flush=True)

    def log_with_title(self, data: dict, step, title: str) -> None:
        if self.print_to_console:
            from ..print_utils import log_metrics
            log_metrics(data, title=title)


class DecoratorLoggerBase:
    """Base of decorators that log with a role name, through ``logging`` when a logger is given, else by print;
    optionally only on rank 0."""

    def __init__(self, role: str, logger: logging.Logger | None = None, level=logging.DEBUG, rank: int = 0,
                 log_only_rank_0: bool = True):
        self.role, self.logger, self.level, self.rank, self.log_only_rank_0 = role, logger, level, rank, log_only_rank_0
        self.logging_function = self.log_by_print if logger is None else self.log_by_logging

    def _mine(self) -> bool:
        return not self.log_only_rank_0 or self.rank == 0

    def log_by_print(self, log_str: str) -> None:
        if self._mine():
            print(f"{self.role} {log_str}", flush=True)

    def log_by_logging(self, log_str: str) -> None:
        if self.logger is None:
            raise ValueError("Logger is not initialized")
        if self._mine():
            self.logger.log(self.level, f"{self.role} {log_str}")


def print_rank_0(message) -> None:
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(message, flush=True)


def print_with_rank(message: str, rank: int = 0, log_only_rank_0: bool = False) -> None:
    if not log_only_rank_0 or rank == 0:
        print(f"[Rank {rank}] {message}", flush=True)


def print_with_rank_and_timer(message: str, rank: int = 0, log_only_rank_0: bool = False) -> None:
    if not log_only_rank_0 or rank == 0:
        print(f"[{datetime.datetime.now():%Y-%m-%d %H:%M:%S}] [Rank {rank}] {message}", flush=True)


def log_with_rank(message: str, rank, logger: logging.Logger, level=logging.INFO, log_only_rank_0: bool = False) -> None:
    if not log_only_rank_0 or rank == 0:
        logger.log(level, f"[Rank {rank}] {message}")
