"""Small Python helpers. ``DynamicEnum``: an enum whose members can be registered at run time
(used for the dispatch / execute modes; reference: axon/utils/py_utils.py)."""
from __future__ import annotations


class _DynamicEnumMeta(type):
    def __iter__(cls):
        return iter(cls._registry.values())

    def __contains__(cls, item):
        return item in cls._registry.values() or item in cls._registry

    def __getitem__(cls, name):
        return cls._registry[name]

    def __getattr__(cls, name):
        reg = cls.__dict__.get("_registry", {})
        if name in reg:
            return reg[name]
        raise AttributeError(name)


class DynamicEnum(metaclass=_DynamicEnumMeta):
    _registry: dict = {}
    _next_value = 0

    def __init__(self, name: str, value: int):
        self.name, self.value = name, value

    def __repr__(self):
        return f"<{self.__class__.__name__}.{self.name}: {self.value}>"

    def __reduce__(self):          # members pickle by name so identity survives process boundaries
        return (getattr, (self.__class__, self.name))

    @classmethod
    def register(cls, name: str):
        key = name.upper()
        if key in cls._registry:
            raise ValueError(f"{key} already registered in {cls.__name__}")
        member = cls(key, cls._next_value)
        cls._registry[key] = member
        cls._next_value += 1
        return member

    @classmethod
    def remove(cls, name: str):
        return cls._registry.pop(name.upper())

    @classmethod
    def from_name(cls, name: str):
        return cls._registry.get(name.upper())
