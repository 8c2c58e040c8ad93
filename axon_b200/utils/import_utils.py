"""Optional-dependency probes and dynamic loading (reference: axon/utils/import_utils.py:27-160)."""
from __future__ import annotations

import importlib
import importlib.util
from functools import cache

from .module_loader import load_class, load_module  # noqa: F401  (re-exported)


@cache
def _has(name: str) -> bool:
    try:
        return importlib.util.find_spec(name) is not None
    except (ImportError, ValueError):
        return False


def is_megatron_core_available() -> bool:
    return _has("megatron.core")


def is_vllm_available() -> bool:
    return _has("vllm")


def is_sglang_available() -> bool:
    return _has("sglang")


def is_nvtx_available() -> bool:
    return _has("torch")       # torch.cuda.nvtx is used for ranges


def is_trl_available() -> bool:
    return _has("trl")


def import_external_libs(external_libs=None) -> None:
    """Import user modules for their registration side effects (agents, envs, rewards, programs)."""
    if not external_libs:
        return
    for lib in ([external_libs] if isinstance(external_libs, str) else external_libs):
        importlib.import_module(lib)


def load_extern_object(module_path: str, object_name: str):
    mod = load_module(module_path)
    if not hasattr(mod, object_name):
        raise AttributeError(f"'{object_name}' not found in '{module_path}'")
    return getattr(mod, object_name)


def load_class_from_fqn(fqn: str, description: str = "class") -> type:
    mod, _, name = fqn.rpartition(".")
    if not mod:
        raise ValueError(f"{description} must be a fully qualified name, got '{fqn}'")
    return load_extern_object(mod, name)


def load_extern_type(file_path: str, type_name: str) -> type:
    return load_extern_object(file_path, type_name)
