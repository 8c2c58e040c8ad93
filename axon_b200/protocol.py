"""``DataProto``: the batch container exchanged between the controller and the workers.

Three parts with one shared leading batch dimension: ``batch`` (tensors), ``non_tensor_batch``
(numpy object arrays) and ``meta_info`` (free-form dict, not batched). API-compatible with the
reference container (axon/protocol.py:362-1099): indexing, select/pop/rename/union, chunk/split/
concat (``metrics`` in meta_info are merged), repeat variants, padding helpers, iterators and
(de)serialisation. The tensor part is the in-house ``TensorDict`` (no external dependency).
"""
from __future__ import annotations

import copy
import io
import os
import pickle
from dataclasses import dataclass, field
from typing import Any, Callable

import numpy as np
import torch

from .utils.tensordict_lite import TensorDict
from .utils.tensordict_lite import cat as _td_cat

__all__ = ["DataProto", "DataProtoItem", "DataProtoFuture", "DataProtoConfig", "pad_dataproto_to_divisor",
           "unpad_dataproto", "union_tensor_dict", "union_numpy_dict", "collate_fn", "fold_batch_dim",
           "unfold_batch_dim", "all_gather_data_proto", "list_of_dict_to_dict_of_list"]


class _ConfigMeta(type):
    _auto_padding = False

    @property
    def auto_padding(cls) -> bool:
        return cls._auto_padding or os.environ.get("AXON_AUTO_PADDING", "").lower() in ("1", "true")

    @auto_padding.setter
    def auto_padding(cls, enabled: bool) -> None:
        cls._auto_padding = bool(enabled)


class DataProtoConfig(metaclass=_ConfigMeta):
    """Process-wide switches (``DataProtoConfig.auto_padding`` / env ``AXON_AUTO_PADDING``)."""


def list_of_dict_to_dict_of_list(items: list[dict]) -> dict:
    if not items:
        return {}
    out = {k: [] for k in items[0]}
    for it in items:
        for k in out:
            out[k].append(it[k])
    return out


def _as_object_array(values) -> np.ndarray:
    if isinstance(values, np.ndarray):
        return values
    arr = np.empty(len(values), dtype=object)
    for i, v in enumerate(values):
        arr[i] = v
    return arr


def _same(a, b) -> bool:
    if isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor):
        return a.shape == b.shape and bool(torch.equal(a, b))
    if isinstance(a, np.ndarray) and isinstance(b, np.ndarray):
        if a.shape != b.shape:
            return False
        if a.dtype == object or b.dtype == object:
            return all(_same(x, y) for x, y in zip(a.ravel(), b.ravel()))
        return bool(np.array_equal(a, b, equal_nan=a.dtype.kind == "f"))
    if isinstance(a, (list, tuple)) and isinstance(b, (list, tuple)):
        return len(a) == len(b) and all(_same(x, y) for x, y in zip(a, b))
    if isinstance(a, dict) and isinstance(b, dict):
        return a.keys() == b.keys() and all(_same(a[k], b[k]) for k in a)
    try:
        return bool(a == b)
    except Exception:  # noqa: BLE001
        return a is b


def union_tensor_dict(td1: TensorDict, td2: TensorDict) -> TensorDict:
    """Merge td2 into td1 (in place). Keys present in both must hold equal tensors."""
    assert td1.batch_size == td2.batch_size, f"batch sizes differ: {td1.batch_size} vs {td2.batch_size}"
    for k, v in td2.items():
        if k in td1:
            assert _same(td1[k], v), f"key '{k}' holds different values in the two batches"
        else:
            td1[k] = v
    return td1


def union_numpy_dict(d1: dict, d2: dict) -> dict:
    for k, v in d2.items():
        if k in d1:
            assert _same(d1[k], v), f"key '{k}' holds different values in the two dicts"
        d1[k] = v
    return d1


@dataclass
class DataProtoItem:
    batch: TensorDict | None = None
    non_tensor_batch: dict = field(default_factory=dict)
    meta_info: dict = field(default_factory=dict)


@dataclass
class DataProto:
    batch: TensorDict | None = None
    non_tensor_batch: dict = field(default_factory=dict)
    meta_info: dict = field(default_factory=dict)

    def __post_init__(self):
        self.check_consistency()

    # ------------------------------------------------------------------ basics
    def __len__(self) -> int:
        if self.batch is not None:
            return self.batch.batch_size[0] if len(self.batch.batch_size) else 0
        for v in self.non_tensor_batch.values():
            return v.shape[0]
        return 0

    def __getitem__(self, item):
        if isinstance(item, slice):
            return self.slice(item.start, item.stop, item.step)
        if isinstance(item, (list, np.ndarray, torch.Tensor)):
            return self.select_idxs(item)
        if isinstance(item, (int, np.integer)):
            b = None if self.batch is None else self.batch[int(item)]
            nt = {k: v[item] for k, v in self.non_tensor_batch.items()}
            return DataProtoItem(batch=b, non_tensor_batch=nt, meta_info=self.meta_info)
        raise TypeError(f"indexing with {type(item)} is not supported")

    def check_consistency(self) -> None:
        if self.batch is not None:
            assert len(self.batch.batch_size) == 1, "only one batch dimension is supported"
        n = None if self.batch is None else self.batch.batch_size[0]
        for k, v in self.non_tensor_batch.items():
            assert isinstance(v, np.ndarray), f"non_tensor_batch['{k}'] must be a numpy array, got {type(v)}"
            if n is None:
                n = v.shape[0]
            assert v.shape[0] == n, f"non_tensor_batch['{k}'] has {v.shape[0]} rows, expected {n}"

    # ------------------------------------------------------------------ constructors
    @classmethod
    def from_single_dict(cls, data: dict, meta_info: dict | None = None, auto_padding: bool = False):
        tensors = {k: v for k, v in data.items() if isinstance(v, torch.Tensor)}
        others = {k: v for k, v in data.items() if isinstance(v, np.ndarray)}
        bad = [k for k, v in data.items() if not isinstance(v, (torch.Tensor, np.ndarray))]
        if bad:
            raise ValueError(f"unsupported value types for keys {bad}")
        return cls.from_dict(tensors, others, meta_info, auto_padding=auto_padding)

    @classmethod
    def from_dict(cls, tensors: dict | None = None, non_tensors: dict | None = None,
                  meta_info: dict | None = None, num_batch_dims: int = 1, auto_padding: bool = False):
        assert num_batch_dims > 0
        tensors = tensors or {}
        non_tensors = {k: _as_object_array(v) for k, v in (non_tensors or {}).items()}
        bs = None
        for k, v in tensors.items():
            cur = tuple(v.shape[:num_batch_dims])
            if bs is None:
                bs = cur
            assert cur == bs, f"tensor '{k}' has batch shape {cur}, expected {bs}"
        td = TensorDict(tensors, batch_size=bs) if tensors else None
        meta = dict(meta_info or {})
        if auto_padding:
            meta["_axon_auto_padding"] = True
        return cls(batch=td, non_tensor_batch=non_tensors, meta_info=meta)

    @classmethod
    def from_tensordict(cls, td: TensorDict, meta_info: dict | None = None, num_batch_dims: int = 1):
        return cls(batch=td, non_tensor_batch={}, meta_info=dict(meta_info or {}))

    def to_tensordict(self) -> TensorDict:
        td = TensorDict(dict(self.batch.items()) if self.batch is not None else {}, batch_size=(len(self),))
        return td

    # ------------------------------------------------------------------ (de)serialisation
    def __getstate__(self):
        method = os.environ.get("AXON_DATAPROTO_SERIALIZATION_METHOD", "torch")
        if self.batch is None:
            payload = None
        elif method == "numpy":
            payload = ("numpy", tuple(self.batch.batch_size),
                       {k: (str(v.dtype), v.detach().cpu().contiguous().view(torch.uint8).numpy()
                            if v.dtype == torch.bfloat16 else v.detach().cpu().numpy(), tuple(v.shape))
                        for k, v in self.batch.items()})
        else:
            buf = io.BytesIO()
            torch.save({"d": {k: v.detach().cpu() for k, v in self.batch.items()},
                        "bs": tuple(self.batch.batch_size)}, buf)
            payload = ("torch", buf.getvalue())
        return payload, self.non_tensor_batch, self.meta_info

    def __setstate__(self, state):
        payload, self.non_tensor_batch, self.meta_info = state
        if payload is None:
            self.batch = None
        elif payload[0] == "numpy":
            _, bs, items = payload
            d = {}
            for k, (dt, arr, shape) in items.items():
                if dt == "torch.bfloat16":
                    d[k] = torch.from_numpy(arr.copy()).view(torch.bfloat16).view(shape)
                else:
                    d[k] = torch.from_numpy(np.ascontiguousarray(arr))
            self.batch = TensorDict(d, batch_size=bs)
        else:
            obj = torch.load(io.BytesIO(payload[1]), weights_only=False)
            self.batch = TensorDict(obj["d"], batch_size=obj["bs"])

    def save_to_disk(self, filepath: str) -> None:
        with open(filepath, "wb") as f:
            pickle.dump(self, f)

    @staticmethod
    def load_from_disk(filepath: str) -> "DataProto":
        with open(filepath, "rb") as f:
            return pickle.load(f)

    def print_size(self, prefix: str = "") -> None:
        tb = sum(v.numel() * v.element_size() for v in (self.batch.values() if self.batch is not None else []))
        nb = sum(v.nbytes for v in self.non_tensor_batch.values())
        print(f"{prefix}DataProto: tensors {tb / 2**30:.3f} GiB, non-tensors {nb / 2**30:.3f} GiB")

    # ------------------------------------------------------------------ device / selection
    def to(self, device) -> "DataProto":
        if self.batch is not None:
            self.batch = self.batch.to(device)
        return self

    def select(self, batch_keys=None, non_tensor_batch_keys=None, meta_info_keys=None, deepcopy=False):
        b = self.batch
        if batch_keys is not None and b is not None:
            b = b.select(*batch_keys)
        nt = self.non_tensor_batch
        if non_tensor_batch_keys is not None:
            nt = {k: nt[k] for k in non_tensor_batch_keys}
        mi = self.meta_info
        if meta_info_keys is not None:
            mi = {k: mi[k] for k in meta_info_keys}
        if deepcopy:
            b, nt, mi = copy.deepcopy(b), copy.deepcopy(nt), copy.deepcopy(mi)
        return type(self)(batch=b, non_tensor_batch=dict(nt), meta_info=dict(mi))

    def select_idxs(self, idxs) -> "DataProto":
        if isinstance(idxs, list):
            idxs = torch.tensor(idxs)
        if isinstance(idxs, np.ndarray):
            np_idx, t_idx = idxs, torch.from_numpy(idxs)
        else:
            t_idx, np_idx = idxs, idxs.detach().cpu().numpy()
        b = None if self.batch is None else self.batch[t_idx.to(self.batch.device) if self.batch.device is not None else t_idx]
        nt = {k: v[np_idx] for k, v in self.non_tensor_batch.items()}
        return type(self)(batch=b, non_tensor_batch=nt, meta_info=self.meta_info)

    def slice(self, start=None, end=None, step=None) -> "DataProto":
        sl = slice(start, end, step)
        b = None if self.batch is None else self.batch[sl]
        nt = {k: v[sl] for k, v in self.non_tensor_batch.items()}
        return type(self)(batch=b, non_tensor_batch=nt, meta_info=self.meta_info)

    def pop(self, batch_keys=None, non_tensor_batch_keys=None, meta_info_keys=None) -> "DataProto":
        tensors = {k: self.batch.pop(k) for k in (batch_keys or [])}
        nts = {k: self.non_tensor_batch.pop(k) for k in (non_tensor_batch_keys or [])}
        mis = {k: self.meta_info.pop(k) for k in (meta_info_keys or [])}
        return DataProto.from_dict(tensors, nts, mis)

    def rename(self, old_keys=None, new_keys=None) -> "DataProto":
        as_list = lambda k: [k] if isinstance(k, str) else list(k or [])  # noqa: E731
        old_keys, new_keys = as_list(old_keys), as_list(new_keys)
        assert len(old_keys) == len(new_keys), "old_keys and new_keys must have the same length"
        for o, n in zip(old_keys, new_keys):
            self.batch.rename_key_(o, n)
        return self

    def union(self, other: "DataProto") -> "DataProto":
        if self.batch is None:
            self.batch = other.batch
        elif other.batch is not None:
            union_tensor_dict(self.batch, other.batch)
        union_numpy_dict(self.non_tensor_batch, other.non_tensor_batch)
        for k, v in other.meta_info.items():
            if k in self.meta_info:
                assert _same(self.meta_info[k], v), f"conflicting meta_info for '{k}'"
            self.meta_info[k] = v
        return self

    # ------------------------------------------------------------------ iteration / batching
    def make_iterator(self, mini_batch_size: int, epochs: int, seed: int | None = None, dataloader_kwargs=None):
        """Yield ``epochs`` passes of shuffled mini-batches (len must divide by mini_batch_size)."""
        assert len(self) % mini_batch_size == 0, f"{len(self)} % {mini_batch_size} != 0"
        shuffle = (dataloader_kwargs or {}).get("shuffle", True)
        gen = torch.Generator()
        if seed is not None:
            gen.manual_seed(seed)

        def it():
            for _ in range(epochs):
                order = torch.randperm(len(self), generator=gen) if shuffle else torch.arange(len(self))
                for s in range(0, len(self), mini_batch_size):
                    d = self.select_idxs(order[s:s + mini_batch_size])
                    d.meta_info = self.meta_info
                    yield d
        return iter(it())

    def is_padding_enabled(self) -> bool:
        return bool(self.meta_info.get("_axon_auto_padding", False)) or DataProtoConfig.auto_padding

    def padding(self, padding_size: int, padding_candidate: str = "") -> None:
        """Append ``padding_size`` rows copied from the first ('first') or last (default) row, in place."""
        if padding_size == 0:
            return
        idx = 0 if padding_candidate == "first" else len(self) - 1
        pad = self.select_idxs([idx]).repeat(padding_size)
        merged = DataProto.concat([self, pad])
        self.batch, self.non_tensor_batch = merged.batch, merged.non_tensor_batch

    def chunk(self, chunks: int) -> list["DataProto"]:
        if not self.is_padding_enabled():
            assert len(self) % chunks == 0, f"only equal chunks are supported: {len(self)} rows into {chunks}"
        n = len(self)
        size = (n + chunks - 1) // chunks
        out = []
        for i in range(chunks):
            out.append(self.slice(i * size, min(n, (i + 1) * size)))
        return out

    def split(self, split_size: int) -> list["DataProto"]:
        return [self.slice(i, i + split_size) for i in range(0, len(self), split_size)]

    @staticmethod
    def concat(data: list["DataProto"]) -> "DataProto":
        """Concatenate along the batch dim. ``meta_info['metrics']`` entries are gathered into a
        dict of lists; every other meta key must agree across the inputs."""
        if not data:
            return DataProto()
        batch = _td_cat([d.batch for d in data]) if data[0].batch is not None else None
        nt = {}
        for k in data[0].non_tensor_batch:
            parts = [d.non_tensor_batch[k] for d in data]
            try:
                nt[k] = np.concatenate(parts, axis=0)
            except ValueError:
                nt[k] = _as_object_array([x for p in parts for x in p])
        meta, metrics = {}, []
        for d in data:
            for k, v in d.meta_info.items():
                if k == "metrics":
                    if v is not None:
                        metrics.extend(v if isinstance(v, list) else [v])
                elif k not in meta:
                    meta[k] = v
                else:
                    assert _same(meta[k], v), f"conflicting meta_info for '{k}'"
        if metrics:
            meta["metrics"] = list_of_dict_to_dict_of_list(metrics)
        return type(data[0])(batch=batch, non_tensor_batch=nt, meta_info=meta)

    def reorder(self, indices: torch.Tensor) -> None:
        self.batch = self.batch[indices]
        idx = indices.detach().cpu().numpy()
        self.non_tensor_batch = {k: v[idx] for k, v in self.non_tensor_batch.items()}

    def repeat(self, repeat_times: int = 2, interleave: bool = True) -> "DataProto":
        """interleave=True: a a b b; False: a b a b."""
        n = len(self)
        base = torch.arange(n)
        order = base.repeat_interleave(repeat_times) if interleave else base.repeat(repeat_times)
        return self.select_idxs(order)

    def unfold_column_chunks(self, n_split: int, split_keys=None) -> "DataProto":
        split_keys = set(split_keys or [])
        new = len(self) * n_split
        b = None
        if self.batch is not None:
            d = {}
            for k, v in self.batch.items():
                d[k] = v.reshape(new, v.shape[1] // n_split, *v.shape[2:]) if k in split_keys \
                    else v.repeat_interleave(n_split, 0)
            b = TensorDict(d, batch_size=(new,))
        nt = {}
        for k, v in self.non_tensor_batch.items():
            nt[k] = v.reshape(new, v.shape[1] // n_split, *v.shape[2:]) if k in split_keys else np.repeat(v, n_split, 0)
        return type(self)(batch=b, non_tensor_batch=nt, meta_info=self.meta_info)

    def sample_level_repeat(self, repeat_times) -> "DataProto":
        if isinstance(repeat_times, torch.Tensor):
            counts = repeat_times.to(torch.long).cpu()
        else:
            counts = torch.tensor(list(repeat_times), dtype=torch.long)
        assert counts.dim() == 1 and counts.numel() == len(self)
        return self.select_idxs(torch.arange(len(self)).repeat_interleave(counts))

    def repeat_by_counts(self, repeat_counts: list[int], interleave: bool = True) -> "DataProto":
        assert len(repeat_counts) == len(self)
        if interleave:
            return self.sample_level_repeat(repeat_counts)
        order = [i for r in range(max(repeat_counts, default=0)) for i, c in enumerate(repeat_counts) if r < c]
        return self.select_idxs(torch.tensor(order, dtype=torch.long))

    def get_data_info(self) -> str:
        lines = [f"DataProto(len={len(self)})"]
        for k, v in (self.batch.items() if self.batch is not None else []):
            lines.append(f"  batch[{k}]: {tuple(v.shape)} {v.dtype} {v.device}")
        for k, v in self.non_tensor_batch.items():
            lines.append(f"  non_tensor[{k}]: {v.shape} {v.dtype}")
        for k, v in self.meta_info.items():
            lines.append(f"  meta[{k}]: {type(v).__name__}")
        return "\n".join(lines)


def pad_dataproto_to_divisor(data: DataProto, size_divisor: int) -> tuple[DataProto, int]:
    """Pad by cycling rows from the start until len % size_divisor == 0. Returns (padded, pad_size)."""
    assert isinstance(data, DataProto)
    n = len(data)
    rem = n % size_divisor
    if rem == 0 or n == 0:
        return data, 0
    pad = size_divisor - rem
    idx = torch.arange(pad) % n
    return DataProto.concat([data, copy.deepcopy(data.select_idxs(idx))]), pad


def unpad_dataproto(data: DataProto, pad_size: int) -> DataProto:
    return data[:-pad_size] if pad_size else data


def fold_batch_dim(data: DataProto, new_batch_size: int) -> DataProto:
    """[B, ...] -> [new_batch_size, B / new_batch_size, ...]."""
    b = data.batch.view(new_batch_size, -1) if data.batch is not None else None
    nt = {k: v.reshape(new_batch_size, -1, *v.shape[1:]) for k, v in data.non_tensor_batch.items()}
    out = DataProto.__new__(DataProto)
    out.batch, out.non_tensor_batch, out.meta_info = b, nt, data.meta_info
    return out


def unfold_batch_dim(data: DataProto, batch_dims: int = 2) -> DataProto:
    n = 1
    for s in data.batch.batch_size[:batch_dims]:
        n *= s
    b = data.batch.view(n)
    nt = {k: v.reshape(n, *v.shape[batch_dims:]) for k, v in data.non_tensor_batch.items()}
    return DataProto(batch=b, non_tensor_batch=nt, meta_info=data.meta_info)


def collate_fn(items: list[DataProtoItem]) -> DataProto:
    from .utils.tensordict_lite import stack
    batch = stack([it.batch for it in items]) if items and items[0].batch is not None else None
    nt = list_of_dict_to_dict_of_list([it.non_tensor_batch for it in items])
    nt = {k: _as_object_array(v) for k, v in nt.items()}
    return DataProto(batch=batch, non_tensor_batch=nt)


class DataProtoFuture:
    """A lazily collected DataProto: ``futures`` resolve to per-worker results that ``collect_fn``
    merges; ``dispatch_fn`` then selects this consumer's share. ``resolve`` turns one future into a
    value (identity for plain values, ``.result()`` for concurrent futures)."""

    def __init__(self, collect_fn: Callable, futures: list, dispatch_fn: Callable | None = None,
                 resolve: Callable | None = None):
        self.collect_fn, self.futures, self.dispatch_fn = collect_fn, futures, dispatch_fn
        self.resolve = resolve or (lambda f: f.result() if hasattr(f, "result") else f)

    @staticmethod
    def concat(data: list) -> "DataProtoFuture":
        return DataProtoFuture(collect_fn=DataProto.concat, futures=data)

    def chunk(self, chunks: int) -> list["DataProtoFuture"]:
        def make(i):
            return lambda x: x.chunk(chunks)[i]
        return [DataProtoFuture(self.collect_fn, self.futures, make(i), self.resolve) for i in range(chunks)]

    def get(self):
        out = self.collect_fn([self.resolve(f) for f in self.futures])
        return self.dispatch_fn(out) if self.dispatch_fn is not None else out


def all_gather_data_proto(data: DataProto, process_group) -> None:
    """In place all-gather of every tensor / array along the batch dim over ``process_group``."""
    import torch.distributed as dist
    ws = dist.get_world_size(group=process_group)
    if data.batch is not None:
        out = {}
        for k in sorted(data.batch.keys()):
            v = data.batch[k].contiguous()
            parts = [torch.empty_like(v) for _ in range(ws)]
            dist.all_gather(parts, v, group=process_group)
            out[k] = torch.cat(parts, 0)
        data.batch = TensorDict(out, batch_size=(next(iter(out.values())).shape[0],))
    gathered: list[Any] = [None] * ws
    dist.all_gather_object(gathered, data.non_tensor_batch, group=process_group)
    data.non_tensor_batch = {k: np.concatenate([g[k] for g in gathered]) for k in data.non_tensor_batch}
