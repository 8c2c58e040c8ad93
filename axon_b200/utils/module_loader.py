"""Load classes by ``'pkg.module:Class'``, ``'pkg://module:Class'`` or ``'path/to/file.py:Class'``
(reference: axon/utils/module_loader.py)."""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys


def load_module(mod_path: str):
    """Import a module given a dotted name (optionally ``pkg://`` prefixed) or a ``.py`` file path
    (optionally ``file://`` prefixed)."""
    mod_path = mod_path.removeprefix("pkg://").removeprefix("file://")
    if mod_path.endswith(".py") or os.path.sep in mod_path:
        path = os.path.abspath(mod_path)
        name = "_axon_dyn_" + str(abs(hash(path)))
        if name in sys.modules:
            return sys.modules[name]
        s = importlib.util.spec_from_file_location(name, path)
        module = importlib.util.module_from_spec(s)
        sys.modules[name] = module
        s.loader.exec_module(module)
        return module
    return importlib.import_module(mod_path)


def load_class(spec: str):
    spec = spec.removeprefix("pkg://")
    mod_path, _, cls_name = spec.rpartition(":")
    if not mod_path or not cls_name:
        raise ValueError(f"expected 'module:Class', got '{spec}'")
    if mod_path.endswith(".py") or os.path.sep in mod_path:
        path = os.path.abspath(mod_path)
        name = "_axon_dyn_" + str(abs(hash(path)))
        if name in sys.modules:
            module = sys.modules[name]
        else:
            s = importlib.util.spec_from_file_location(name, path)
            module = importlib.util.module_from_spec(s)
            sys.modules[name] = module
            s.loader.exec_module(module)
    else:
        module = importlib.import_module(mod_path)
    if not hasattr(module, cls_name):
        raise AttributeError(f"module '{mod_path}' has no attribute '{cls_name}'")
    return getattr(module, cls_name)
