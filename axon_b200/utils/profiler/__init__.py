"""Profiling utilities: per-worker profiler control, FLOPs / MFU accounting, memory logging, timing
reducers and single-kernel microbenchmarks (``kernel_cases``)."""
from .config import NsightToolConfig, ProfilerConfig, TorchMemoryToolConfig, TorchProfilerToolConfig
from .flops_counter import FlopsCounter, get_device_flops
from .performance import GPUMemoryLogger, gather_timing, log_gpu_memory_usage, reduce_timing, topk_reduce_ratio_min_max
from .profile import (DistProfiler, DistProfilerExtension, Profiler, TorchMemoryProfiler, mark_annotate, mark_end_range,
                      mark_start_range)

__all__ = ["ProfilerConfig", "NsightToolConfig", "TorchProfilerToolConfig", "TorchMemoryToolConfig", "FlopsCounter",
           "get_device_flops", "GPUMemoryLogger", "log_gpu_memory_usage", "reduce_timing", "gather_timing",
           "topk_reduce_ratio_min_max", "DistProfiler", "DistProfilerExtension", "Profiler", "TorchMemoryProfiler",
           "mark_annotate", "mark_start_range", "mark_end_range"]
