"""Name -> object registries used for losses, advantages, programs, agents, envs, parsers and
rewards (reference: axon/utils/registry/, ``ClassRegistry`` and ``FunctionRegistry``)."""
from __future__ import annotations

import os

from dataclasses import dataclass
from enum import Enum
from typing import Any, Callable, Generic, TypeVar

T = TypeVar("T")


def _key(name) -> str:
    return name.value if isinstance(name, Enum) else str(name)


@dataclass
class FunctionRegistryEntry:
    name: str
    fn: Callable
    metadata: dict


class FunctionRegistry(Generic[T]):
    def __init__(self, name: str = "function"):
        self.name = name
        self._entries: dict[str, FunctionRegistryEntry] = {}

    def register(self, name_or_enum, **metadata):
        key = _key(name_or_enum)

        def deco(fn):
            if key in self._entries and self._entries[key].fn is not fn:
                raise ValueError(f"{self.name} '{key}' is already registered")
            self._entries[key] = FunctionRegistryEntry(key, fn, metadata)
            return fn
        return deco

    def get_entry(self, name_or_enum) -> FunctionRegistryEntry:
        key = _key(name_or_enum)
        if key not in self._entries:
            raise ValueError(f"unknown {self.name} '{key}'. Available: {sorted(self._entries)}")
        return self._entries[key]

    def get_fn(self, name_or_enum) -> Callable:
        return self.get_entry(name_or_enum).fn

    def compute(self, name_or_enum, *args, **kwargs):
        return self.get_fn(name_or_enum)(*args, **kwargs)

    def names(self) -> list[str]:
        return sorted(self._entries)

    def __contains__(self, name) -> bool:
        return _key(name) in self._entries


def _same_definition(a, b) -> bool:
    """Two class objects made from the same source (a recipe file imported once as a package module and once by
    path): re-registering such a class under its name is not a conflict."""
    import inspect
    try:
        return a.__qualname__ == b.__qualname__ and inspect.getsourcefile(a) is not None and \
            os.path.realpath(inspect.getsourcefile(a)) == os.path.realpath(inspect.getsourcefile(b))
    except (TypeError, OSError):
        return False


class ClassRegistry(Generic[T]):
    """Maps names to classes; ``register`` works as ``@reg.register("name")`` or ``reg.register("name", cls)``."""

    def __init__(self, name: str = "class", base: type | None = None):
        self.name = name
        self.base = base
        self._classes: dict[str, type] = {}

    def register(self, name_or_enum, cls: type | None = None, *, override: bool = False):
        key = _key(name_or_enum)

        def deco(c):
            if self.base is not None and not (isinstance(c, type) and issubclass(c, self.base)):
                raise TypeError(f"{c} is not a subclass of {self.base.__name__}")
            old = self._classes.get(key)
            if old is not None and old is not c and not override and not _same_definition(old, c):
                raise ValueError(f"{self.name} '{key}' is already registered")
            self._classes[key] = c
            return c
        return deco(cls) if cls is not None else deco

    def get(self, name_or_enum) -> type:
        key = _key(name_or_enum)
        if key not in self._classes:
            raise ValueError(f"unknown {self.name} '{key}'. Available: {sorted(self._classes)}")
        return self._classes[key]

    def create(self, name_or_enum, *args, **kwargs) -> Any:
        return self.get(name_or_enum)(*args, **kwargs)

    def names(self) -> list[str]:
        return sorted(self._classes)

    def __contains__(self, name) -> bool:
        return _key(name) in self._classes

    def __getitem__(self, name) -> type:
        return self.get(name)

    def items(self):
        return self._classes.items()
