"""Import-compatibility alias: ``import axon.protocol``, ``from axon.trainer.algos.loss import register_loss`` …
resolve to the same modules as ``axon_b200.*`` (one module object under both names), so recipes and
user plug-ins written against the reference's package name load unchanged."""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

import axon_b200 as _impl

_PREFIX, _TARGET = "axon.", "axon_b200."


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, real_name: str):
        self.real_name = real_name

    def create_module(self, spec):
        return importlib.import_module(self.real_name)

    def exec_module(self, module):
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        real = _TARGET + fullname[len(_PREFIX):]
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except (ImportError, ValueError):
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(real))
        real_spec = importlib.util.find_spec(real)
        if real_spec is not None and real_spec.submodule_search_locations is not None:
            spec.submodule_search_locations = list(real_spec.submodule_search_locations)
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

__path__ = list(_impl.__path__)
__version__ = getattr(_impl, "__version__", "0.1.0")
