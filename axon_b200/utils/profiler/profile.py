"""Per-worker profiler control (reference: axon/utils/profiler/profile.py:29-366).

``DistProfiler(rank, config)`` picks a backend from ``config.tool``:

* ``nsys``  — brackets the profiled region with cudaProfilerStart/Stop (for a job launched under an
  external capture tool in capture-range mode) and NVTX ranges; ``discrete`` makes every annotated
  call its own range.
* ``torch`` — ``torch.profiler`` with CPU+CUDA activities, Chrome trace written to ``save_path``.
* ``torch_memory`` — allocator history recording, snapshot pickled on stop.

Only ranks selected by ``all_ranks`` / ``ranks`` do anything. Workers expose ``start_profile`` /
``stop_profile`` through ``DistProfilerExtension``; the driver calls them around the steps listed in
``global_profiler.steps``.
"""
from __future__ import annotations

import functools
import os
from contextlib import contextmanager

import torch

from .config import ProfilerConfig, TorchMemoryToolConfig


def _cuda_live() -> bool:
    return torch.cuda.is_available() and torch.cuda.is_initialized()


def mark_start_range(message: str | None = None, color: str | None = None, domain: str | None = None,
                     category: str | None = None):
    if _cuda_live():
        torch.cuda.nvtx.range_push(message or "range")
        return message or "range"
    return None


def mark_end_range(range_id) -> None:
    if range_id is not None and _cuda_live():
        torch.cuda.nvtx.range_pop()


def mark_annotate(message: str | None = None, color: str | None = None, domain: str | None = None,
                  category: str | None = None):
    def decorator(fn):
        @functools.wraps(fn)
        def wrapped(*a, **k):
            rid = mark_start_range(message or fn.__name__, color, domain, category)
            try:
                return fn(*a, **k)
            finally:
                mark_end_range(rid)
        return wrapped
    return decorator


class _NoOp:
    def start(self, **kw):
        pass

    def stop(self):
        pass


class Profiler:
    """torch.profiler wrapper bound to a rank and an output directory."""

    def __init__(self, config: ProfilerConfig, rank: int = 0, tool_config=None):
        self.config, self.rank = config, rank
        self.tool_config = tool_config
        self.prof = None
        self.saved = False

    def check(self) -> bool:
        return self.prof is not None and not self.saved

    def start(self, **kw):
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self.prof = torch.profiler.profile(activities=acts, record_shapes=True, with_stack=False)
        self.prof.start()
        self.saved = False

    def step(self):
        if self.check():
            self.prof.step()

    def stop(self):
        if self.check():
            self.prof.stop()
            self.save()

    def save(self):
        if self.prof is None or self.saved:
            return
        path = self.config.save_path or "outputs/profile"
        os.makedirs(path, exist_ok=True)
        self.prof.export_chrome_trace(os.path.join(path, f"trace_rank{self.rank}.json"))
        self.saved = True

    stop_and_save = stop
    stop_trace = stop


class _RangeProfiler:
    """External-capture backend: profiler start/stop API calls plus an NVTX range per region."""

    def __init__(self, discrete: bool):
        self.discrete = discrete
        self._rid = None

    def start(self, role: str | None = None, profile_step: str | None = None, **kw):
        if _cuda_live():
            if not self.discrete:
                torch.cuda.profiler.start()
            self._rid = mark_start_range(f"{role or 'worker'}_step{profile_step}" if profile_step is not None else role)

    def stop(self):
        if _cuda_live():
            mark_end_range(self._rid)
            self._rid = None
            if not self.discrete:
                torch.cuda.profiler.stop()


class TorchMemoryProfiler:
    def __init__(self, rank: int, config: ProfilerConfig | None, tool_config: TorchMemoryToolConfig | None = None):
        self.rank, self.config = rank, config
        self.tool_config = tool_config or TorchMemoryToolConfig()
        self.enabled = bool(config and config.enable and (config.all_ranks or rank in (config.ranks or [])))
        self._step = 0

    def start(self, **kw):
        if self.enabled and torch.cuda.is_available():
            torch.cuda.memory._record_memory_history(max_entries=self.tool_config.trace_alloc_max_entries,
                                                     stacks="python")
            self._step = kw.get("profile_step", self._step)

    def stop(self):
        if self.enabled and torch.cuda.is_available():
            path = (self.config.save_path if self.config else None) or "outputs/profile"
            os.makedirs(path, exist_ok=True)
            torch.cuda.memory._dump_snapshot(os.path.join(path, f"memory_rank{self.rank}_step{self._step}.pickle"))
            torch.cuda.memory._record_memory_history(enabled=None)


class DistProfiler:
    def __init__(self, rank: int, config: ProfilerConfig | None = None, tool_config=None, **kw):
        self.rank = rank
        self.config = config or ProfilerConfig()
        self.enabled = bool(self.config.enable and self.config.tool and (self.config.all_ranks or rank in self.config.ranks))
        tool = self.config.tool if self.enabled else None
        gcfg = self.config.global_tool_config or {}
        sub = lambda name: (gcfg.get(name) if hasattr(gcfg, "get") else None) or {}      # noqa: E731
        if tool == "nsys":
            self.discrete = bool(sub("nsys").get("discrete", False))
            self._impl = _RangeProfiler(self.discrete)
        elif tool == "torch":
            self.discrete = False
            self._impl = Profiler(self.config, rank, tool_config)
        elif tool == "torch_memory":
            self.discrete = False
            tm = sub("torch_memory")
            self._impl = TorchMemoryProfiler(rank, self.config, TorchMemoryToolConfig(**dict(tm)) if tm else None)
        else:
            self.discrete = False
            self._impl = _NoOp()
        self.active = False

    def start(self, **kw):
        if self.enabled:
            self.active = True
            self._impl.start(**kw)

    def stop(self):
        if self.enabled and self.active:
            self._impl.stop()
            self.active = False

    @staticmethod
    def annotate(message: str | None = None, color: str | None = None, domain: str | None = None,
                 category: str | None = None, **kw):
        """Method decorator: an NVTX range around the call; in discrete mode each call is also its own
        capture range. Looks for ``self.profiler`` on the instance."""
        def decorator(fn):
            @functools.wraps(fn)
            def wrapped(self_inst, *a, **k):
                prof = getattr(self_inst, "profiler", None)
                on = bool(prof and prof.enabled and prof.active)
                if on and prof.discrete and _cuda_live():
                    torch.cuda.profiler.start()
                rid = mark_start_range(message or fn.__name__, color, domain, category) if on else None
                try:
                    return fn(self_inst, *a, **k)
                finally:
                    mark_end_range(rid)
                    if on and prof.discrete and _cuda_live():
                        torch.cuda.profiler.stop()
            return wrapped
        return decorator

    @contextmanager
    def region(self, **kw):
        self.start(**kw)
        try:
            yield
        finally:
            self.stop()


class DistProfilerExtension:
    """Mixin giving a worker ``start_profile`` / ``stop_profile`` RPCs."""

    def __init__(self, profiler: DistProfiler):
        self.profiler = profiler

    def start_profile(self, **kw) -> None:
        self.profiler.start(**kw)

    def stop_profile(self) -> None:
        self.profiler.stop()
