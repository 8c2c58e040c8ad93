"""Step metrics: batch statistics, timing, sampler/trainer mismatch, repetition, and reducers.

Every ``compute_*`` function can return "sufficient statistics" (keys starting with ``_``: counts
and sums) next to the readable values, so shards computed on different workers combine exactly with
the matching ``reduce_*`` / ``aggregate_*`` function (reference: axon/utils/metrics/*.py).
"""
from .data_metrics import compute_data_metrics, compute_response_mask, reduce_data_metrics
from .mismatch import aggregate_trainer_sampler_metrics, compute_trainer_sampler_mismatch_metrics
from .reduce import append_to_dict, reduce_metrics
from .repetition import compression_ratio, compute_repetition_metrics, has_repetition
from .timing import Timer, compute_timing_metrics, marked_timer, reduce_timing_metrics

__all__ = ["compute_data_metrics", "compute_response_mask", "reduce_data_metrics", "compute_repetition_metrics",
           "has_repetition", "compression_ratio", "compute_timing_metrics", "reduce_timing_metrics", "marked_timer",
           "Timer", "reduce_metrics", "append_to_dict", "compute_trainer_sampler_mismatch_metrics",
           "aggregate_trainer_sampler_metrics"]
