"""Profiler configuration dataclasses (reference: axon/utils/profiler/config.py:92-196)."""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any


class _MappingMixin:
    """Gives a dataclass the read interface of a mapping (``cfg.get("x")``, ``cfg["x"]``, ``**cfg``)."""

    def get(self, key: str, default: Any = None) -> Any:
        return getattr(self, key, default)

    def __getitem__(self, key: str):
        if not hasattr(self, key):
            raise KeyError(key)
        return getattr(self, key)

    def keys(self):
        return [f.name for f in fields(self)]

    def __iter__(self):
        return iter(self.keys())

    def __len__(self) -> int:
        return len(self.keys())


@dataclass
class NsightToolConfig(_MappingMixin):
    discrete: bool = False       # True: one capture range per annotated task; False: one per training step


@dataclass
class TorchProfilerToolConfig(_MappingMixin):
    step_start: int = -1
    step_end: int = -1

    def __post_init__(self):
        assert isinstance(self.step_start, int) and isinstance(self.step_end, int)


@dataclass
class TorchMemoryToolConfig(_MappingMixin):
    trace_alloc_max_entries: int = 100_000
    stack_depth: int = 32

    def __post_init__(self):
        assert isinstance(self.trace_alloc_max_entries, int) and self.trace_alloc_max_entries > 0
        assert isinstance(self.stack_depth, int) and self.stack_depth > 0


@dataclass
class ProfilerConfig(_MappingMixin):
    tool: str | None = None              # nsys | torch | torch_memory | None
    enable: bool = False
    all_ranks: bool = False
    ranks: list = field(default_factory=list)
    save_path: str | None = None
    tool_config: Any = None
    global_tool_config: Any = None

    def __post_init__(self):
        assert isinstance(self.ranks, (set, list, tuple)), f"ranks must be a list, got {type(self.ranks)}"
        self.ranks = list(self.ranks)

    def _combine(self, other: "ProfilerConfig", both: bool) -> "ProfilerConfig":
        assert self.tool == other.tool, f"cannot combine profiler configs of tools {self.tool} and {other.tool}"
        op = (lambda a, b: a and b) if both else (lambda a, b: a or b)
        ranks = set(self.ranks) & set(other.ranks) if both else set(self.ranks) | set(other.ranks)
        return ProfilerConfig(tool=self.tool, enable=op(self.enable, other.enable), all_ranks=op(self.all_ranks, other.all_ranks),
                              ranks=sorted(ranks), save_path=self.save_path, tool_config=self.tool_config,
                              global_tool_config=self.global_tool_config or other.global_tool_config)

    def union(self, other: "ProfilerConfig") -> "ProfilerConfig":
        return self._combine(other, both=False)

    def intersect(self, other: "ProfilerConfig") -> "ProfilerConfig":
        return self._combine(other, both=True)

    @classmethod
    def from_config(cls, cfg, global_cfg=None) -> "ProfilerConfig":
        g = lambda c, k, d=None: (c.get(k, d) if c is not None else d)   # noqa: E731
        return cls(tool=g(global_cfg, "tool", g(cfg, "tool")), enable=bool(g(cfg, "enable", False)),
                   all_ranks=bool(g(cfg, "all_ranks", False)), ranks=list(g(cfg, "ranks", []) or []),
                   save_path=g(global_cfg, "save_path", g(cfg, "save_path")), tool_config=g(cfg, "tool_config"),
                   global_tool_config=g(global_cfg, "global_tool_config"))
