"""Configuration objects and composition.

``Config`` is a nested mapping with attribute access, dotted ``select`` / ``set`` and ``${...}``
interpolation — the subset of OmegaConf that the framework uses. ``compose_config`` builds the run
configuration the way the reference does with Hydra (axon/cli/_hydra_bridge.py, axon/config/config.yaml):
the root yaml's ``defaults`` list grafts templates at ``group/name@target`` keys, then dotted
overrides apply: ``a.b=v`` (must exist), ``+a.b=v`` (must not exist), ``++a.b=v`` (either), ``~a.b``
(delete). Interpolations: ``${a.b}`` absolute, ``${.x}`` relative to the containing node,
``${oc.select:a.b,default}`` with a fallback. ``omega_conf_to_dataclass`` converts a sub-tree into a
dataclass (reference: axon/utils/config.py:26-136).
"""
from __future__ import annotations

import copy
import dataclasses
import re
from pathlib import Path
from typing import Any, Iterable

import yaml

_MISSING = object()
# one level of braces / brackets may appear inside (the literal defaults "{}" and "[]" of oc.select)
_INTERP = re.compile(r"\$\{((?:[^${}]|\{\})+)\}")


class ConfigError(ValueError):
    pass


class Config(dict):
    """dict with attribute access; nested dicts are converted on the way in."""

    def __init__(self, data: dict | None = None, **kw):
        super().__init__()
        for k, v in {**(data or {}), **kw}.items():
            self[k] = v

    @staticmethod
    def _wrap(v):
        if isinstance(v, Config):
            return v
        if isinstance(v, dict):
            return Config(v)
        if isinstance(v, (list, tuple)):
            return [Config._wrap(x) for x in v]
        return v

    def __setitem__(self, k, v):
        super().__setitem__(k, Config._wrap(v))

    def __getattr__(self, k):
        if k.startswith("__"):
            raise AttributeError(k)
        try:
            return self[k]
        except KeyError:
            raise AttributeError(f"config has no key '{k}'") from None

    def __setattr__(self, k, v):
        self[k] = v

    def __delattr__(self, k):
        del self[k]

    def select(self, path: str, default=None):
        node: Any = self
        for part in path.split("."):
            if isinstance(node, dict) and part in node:
                node = node[part]
            elif isinstance(node, list) and part.isdigit() and int(part) < len(node):
                node = node[int(part)]
            else:
                return default
        return node

    def set(self, path: str, value, create: bool = True) -> None:
        parts = path.split(".")
        node = self
        for p in parts[:-1]:
            if p not in node or not isinstance(node[p], dict):
                if not create:
                    raise ConfigError(f"cannot set '{path}': '{p}' does not exist")
                node[p] = Config()
            node = node[p]
        node[parts[-1]] = value

    def delete(self, path: str) -> None:
        parts = path.split(".")
        node = self.select(".".join(parts[:-1])) if len(parts) > 1 else self
        if not isinstance(node, dict) or parts[-1] not in node:
            raise ConfigError(f"cannot delete '{path}': no such key")
        del node[parts[-1]]

    def merge(self, other: dict) -> "Config":
        for k, v in other.items():
            if isinstance(v, dict) and isinstance(self.get(k), dict):
                self[k].merge(v)
            else:
                self[k] = copy.deepcopy(v)
        return self

    def to_dict(self) -> dict:
        def unwrap(v):
            if isinstance(v, dict):
                return {k: unwrap(x) for k, x in v.items()}
            if isinstance(v, list):
                return [unwrap(x) for x in v]
            return v
        return unwrap(self)

    def copy(self) -> "Config":
        return Config(copy.deepcopy(self.to_dict()))


def _parse_scalar(text: str):
    try:
        return yaml.safe_load(text)
    except yaml.YAMLError:
        return text


def resolve(cfg: Config) -> Config:
    """Resolve every ``${...}`` in place (iterates until stable; cycles raise)."""
    def lookup(expr: str, here: str):
        expr = expr.strip()
        if expr.startswith("oc.select:"):
            body = expr[len("oc.select:"):]
            key, _, default = body.partition(",")
            val = lookup_key(key.strip(), here)
            return _parse_scalar(default.strip()) if val is _MISSING else val
        if expr.startswith("oc.env:"):
            import os
            key, _, default = expr[len("oc.env:"):].partition(",")
            return os.environ.get(key.strip(), _parse_scalar(default.strip()) if default else None)
        val = lookup_key(expr, here)
        if val is _MISSING:
            raise ConfigError(f"interpolation '${{{expr}}}' (at '{here}') refers to a missing key")
        return val

    def lookup_key(key: str, here: str):
        if key.startswith("."):
            dots = len(key) - len(key.lstrip("."))
            base = here.split(".")[: -dots] if dots <= len(here.split(".")) else []
            key = ".".join(base + [key.lstrip(".")])
        v = cfg.select(key, _MISSING)
        return v

    def walk(node, path):
        changed = False
        items = node.items() if isinstance(node, dict) else enumerate(node)
        for k, v in list(items):
            here = f"{path}.{k}" if path else str(k)
            if isinstance(v, (dict, list)):
                changed |= walk(v, here)
            elif isinstance(v, str) and "${" in v:
                m = _INTERP.fullmatch(v.strip())
                if m:
                    new = lookup(m.group(1), here)
                    if isinstance(new, str) and new == v:
                        raise ConfigError(f"self-referential interpolation at '{here}'")
                else:
                    new = _INTERP.sub(lambda mm: str(lookup(mm.group(1), here)), v)
                node[k] = copy.deepcopy(new) if isinstance(new, (dict, list)) else new
                changed = True
        return changed

    for _ in range(32):
        if not walk(cfg, ""):
            return cfg
    raise ConfigError("interpolation did not converge (cycle?)")


def load_yaml(path: str | Path) -> dict:
    with open(path) as f:
        return yaml.safe_load(f) or {}


def compose_config(overrides: Iterable[str] = (), config_dir: str | Path | None = None, config_name: str = "config",
                   do_resolve: bool = True) -> Config:
    root_dir = Path(config_dir) if config_dir else Path(__file__).resolve().parent.parent / "config"
    root = load_yaml(root_dir / f"{config_name}.yaml")
    defaults = root.pop("defaults", ["_self_"])
    cfg = Config()
    for d in defaults:
        if d == "_self_":
            cfg.merge(root)
            continue
        spec = d if isinstance(d, str) else next(iter(d.items()))
        if isinstance(spec, tuple):                       # {group: name} form
            spec = f"{spec[0]}/{spec[1]}"
        src, _, target = spec.partition("@")
        sub = load_yaml(root_dir / f"{src}.yaml")
        if target:
            cfg.setdefault(target, Config())
            cfg[target].merge(sub)
        else:
            cfg.merge(sub)
    if "_self_" not in defaults:
        cfg.merge(root)
    apply_overrides(cfg, overrides)
    return resolve(cfg) if do_resolve else cfg


def apply_overrides(cfg: Config, overrides: Iterable[str]) -> Config:
    for ov in overrides:
        ov = ov.strip()
        if not ov:
            continue
        if ov.startswith("~"):
            cfg.delete(ov[1:].split("=")[0])
            continue
        if "=" not in ov:
            raise ConfigError(f"override '{ov}' is not of the form key=value")
        key, _, raw = ov.partition("=")
        force = key.startswith("++")
        add = key.startswith("+") and not force
        key = key.lstrip("+")
        exists = cfg.select(key, _MISSING) is not _MISSING
        if add and exists:
            raise ConfigError(f"'+{key}' but the key already exists (use '++{key}' to override)")
        if not add and not force and not exists:
            raise ConfigError(f"key '{key}' is not in the config (use '+{key}=...' to add it)")
        cfg.set(key, _parse_scalar(raw))
    return cfg


def flatten_yaml_to_overrides(data: dict, prefix: str = "") -> list[str]:
    """A user yaml file becomes ``++a.b=value`` overrides (lists / scalars are leaves)."""
    out = []
    for k, v in data.items():
        key = f"{prefix}.{k}" if prefix else str(k)
        if isinstance(v, dict) and v:
            out += flatten_yaml_to_overrides(v, key)
        else:
            out.append(f"++{key}={yaml.safe_dump(v, default_flow_style=True).strip().removesuffix('...').strip()}")
    return out


def omega_conf_to_dataclass(config, dataclass_type=None):
    """Mapping -> dataclass instance (nested dataclass fields are converted recursively; unknown keys
    raise). With no type, a plain dict copy is returned."""
    if config is None:
        return None
    data = config.to_dict() if isinstance(config, Config) else dict(config)
    if dataclass_type is None:
        return data
    if not dataclasses.is_dataclass(dataclass_type):
        raise TypeError(f"{dataclass_type} is not a dataclass")
    fields = {f.name: f for f in dataclasses.fields(dataclass_type)}
    unknown = set(data) - set(fields)
    if unknown:
        raise ConfigError(f"unknown keys for {dataclass_type.__name__}: {sorted(unknown)}")
    kw = {}
    for k, v in data.items():
        ft = fields[k].type
        if dataclasses.is_dataclass(ft) and isinstance(v, dict):
            v = omega_conf_to_dataclass(v, ft)
        kw[k] = v
    return dataclass_type(**kw)


def validate_config(cfg, required: Iterable[str]) -> None:
    missing = [k for k in required if Config(cfg).select(k, _MISSING) is _MISSING]
    if missing:
        raise ConfigError(f"missing required config keys: {missing}")
