"""A small batch-of-tensors container with the subset of the ``tensordict.TensorDict`` API that
the data protocol needs (the reference depends on the external ``tensordict`` package:
axon/protocol.py:362, axon/utils/tensordict_utils.py). Every value shares the leading batch
dimension(s) given by ``batch_size``."""
from __future__ import annotations

from typing import Iterable, Mapping

import torch


class TensorDict:
    def __init__(self, source: Mapping[str, torch.Tensor] | None = None, batch_size=None, device=None):
        self._d: dict[str, torch.Tensor] = {}
        src = dict(source or {})
        if batch_size is None:
            first = next(iter(src.values()), None)
            batch_size = (first.shape[0],) if first is not None and first.dim() > 0 else ()
        if isinstance(batch_size, int):
            batch_size = (batch_size,)
        self.batch_size = torch.Size(batch_size)
        for k, v in src.items():
            self[k] = v if device is None else v.to(device)

    # ------------------------------------------------------------------ mapping protocol
    def __setitem__(self, key: str, value: torch.Tensor) -> None:
        if not isinstance(value, torch.Tensor):
            value = torch.as_tensor(value)
        nb = len(self.batch_size)
        if tuple(value.shape[:nb]) != tuple(self.batch_size):
            raise ValueError(f"tensor '{key}' has leading shape {tuple(value.shape[:nb])}, "
                             f"expected batch size {tuple(self.batch_size)}")
        self._d[key] = value

    def __getitem__(self, idx):
        if isinstance(idx, str):
            return self._d[idx]
        out = {k: v[idx] for k, v in self._d.items()}
        probe = torch.empty(self.batch_size, device="meta")[idx]
        return TensorDict(out, batch_size=probe.shape)

    def __delitem__(self, key: str) -> None:
        del self._d[key]

    def __contains__(self, key) -> bool:
        return key in self._d

    def __iter__(self):
        return iter(self._d)

    def __len__(self) -> int:
        return self.batch_size[0] if len(self.batch_size) else 0

    def keys(self):
        return self._d.keys()

    def values(self):
        return self._d.values()

    def items(self):
        return self._d.items()

    def get(self, key, default=None):
        return self._d.get(key, default)

    def pop(self, key, *default):
        return self._d.pop(key, *default)

    def set(self, key, value):
        self[key] = value
        return self

    def update(self, other: Mapping[str, torch.Tensor]):
        for k, v in other.items():
            self[k] = v
        return self

    # ------------------------------------------------------------------ transforms
    @property
    def device(self):
        v = next(iter(self._d.values()), None)
        return None if v is None else v.device

    def to(self, device, non_blocking: bool = False) -> "TensorDict":
        return TensorDict({k: v.to(device, non_blocking=non_blocking) for k, v in self._d.items()},
                          batch_size=self.batch_size)

    def clone(self) -> "TensorDict":
        return TensorDict({k: v.clone() for k, v in self._d.items()}, batch_size=self.batch_size)

    def contiguous(self) -> "TensorDict":
        return TensorDict({k: v.contiguous() for k, v in self._d.items()}, batch_size=self.batch_size)

    def select(self, *keys: str, strict: bool = True) -> "TensorDict":
        if strict:
            missing = [k for k in keys if k not in self._d]
            if missing:
                raise KeyError(f"keys not found: {missing}")
        return TensorDict({k: self._d[k] for k in keys if k in self._d}, batch_size=self.batch_size)

    def exclude(self, *keys: str) -> "TensorDict":
        return TensorDict({k: v for k, v in self._d.items() if k not in keys}, batch_size=self.batch_size)

    def rename_key_(self, old: str, new: str) -> "TensorDict":
        self._d[new] = self._d.pop(old)
        return self

    def chunk(self, chunks: int, dim: int = 0) -> list["TensorDict"]:
        assert dim == 0
        n = len(self)
        size = (n + chunks - 1) // chunks
        return [self[i:i + size] for i in range(0, n, size)]

    def split(self, split_size: int, dim: int = 0) -> list["TensorDict"]:
        assert dim == 0
        return [self[i:i + split_size] for i in range(0, len(self), split_size)]

    def view(self, *shape) -> "TensorDict":
        nb = len(self.batch_size)
        new = torch.empty(self.batch_size, device="meta").view(*shape).shape
        return TensorDict({k: v.reshape(*new, *v.shape[nb:]) for k, v in self._d.items()}, batch_size=new)

    def to_dict(self) -> dict[str, torch.Tensor]:
        return dict(self._d)

    def __repr__(self) -> str:
        body = ", ".join(f"{k}: {tuple(v.shape)} {str(v.dtype).replace('torch.', '')}" for k, v in self._d.items())
        return f"TensorDict(batch_size={tuple(self.batch_size)}, {{{body}}})"

    # pickling through plain dicts keeps files loadable without this class's internals changing
    def __getstate__(self):
        return {"d": self._d, "batch_size": tuple(self.batch_size)}

    def __setstate__(self, st):
        self._d = st["d"]
        self.batch_size = torch.Size(st["batch_size"])


def cat(tds: Iterable[TensorDict], dim: int = 0) -> TensorDict:
    tds = list(tds)
    assert dim == 0 and tds
    keys = list(tds[0].keys())
    for t in tds[1:]:
        if set(t.keys()) != set(keys):
            raise KeyError(f"cannot concatenate TensorDicts with different keys: {sorted(keys)} vs {sorted(t.keys())}")
    n = sum(len(t) for t in tds)
    return TensorDict({k: torch.cat([t[k] for t in tds], 0) for k in keys},
                      batch_size=(n, *tds[0].batch_size[1:]))


def stack(tds: Iterable[TensorDict], dim: int = 0) -> TensorDict:
    tds = list(tds)
    assert dim == 0 and tds
    return TensorDict({k: torch.stack([t[k] for t in tds], 0) for k in tds[0].keys()},
                      batch_size=(len(tds), *tds[0].batch_size))
