"""Layout-independent ("distributed") checkpoints: every tensor is one array in GLOBAL coordinates, written as
chunks by whichever ranks hold a piece of it, and read back by boxes, so a checkpoint written under one parallel
layout (tp / ep / pp / dp sizes) loads under any other.

This is the role megatron's ``dist_checkpointing`` plays for the reference, with its asynchronous zarr strategy
(axon/utils/megatron/async_zarr_dist_checkpointing.py:61-150 save / preload / finalize functions, :152-400 the
strategy: one array per tensor key chunked by shard, objects as ``shard_<offset>_<shape>.pt`` files, only the main
replica of a shard writes; used by axon/utils/state/megatron_state_manager.py:177-300). The store here is a plain
directory tree with no third-party array library:

    <dir>/metadata.json                         format tag, per key: dtype, global shape, list of chunks
    <dir>/arrays/<key>/c_<o0.o1>_<s0.s1>.bin    raw little-endian bytes of one box (offset o, shape s)
    <dir>/objects/<key>/shard_<o>_<s>.pt        pickled python objects (optimizer scalars, rng, ...)
    <dir>/manifests/rank_<R>.json               what rank R wrote (merged into metadata.json by rank 0)

Saving is asynchronous in the same three stages as the reference's strategy: *preload* (device -> pinned host
copies, enqueued on the current stream; the training step may go on once they are synchronised), *save* (a
background thread writes the chunk files and this rank's manifest) and *finalize* (join, barrier, rank 0 merges
the manifests). bfloat16 travels as its 16-bit pattern.
"""
from __future__ import annotations

import json
import os
import pickle
import threading
from dataclasses import dataclass, field

import numpy as np
import torch

FORMAT = "axon_b200.sharded_arrays"
VERSION = 1

_NP = {torch.float32: "<f4", torch.float64: "<f8", torch.float16: "<f2", torch.bfloat16: "<u2", torch.int64: "<i8",
       torch.int32: "<i4", torch.int16: "<i2", torch.int8: "|i1", torch.uint8: "|u1", torch.bool: "|b1"}
_TORCH = {str(k): k for k in _NP}


@dataclass
class ShardedTensor:
    """A rank's piece of the array ``key``: ``data`` covers ``boxes`` (in order, concatenated along dim 0 of a 2-D
    view) of the global array. A box is (offset tuple, shape tuple). ``replica_id`` 0 marks the copy that is written;
    other holders of the same box (data-parallel replicas) pass a non-zero id."""
    key: str
    data: torch.Tensor | None
    global_shape: tuple
    boxes: list = field(default_factory=list)
    replica_id: int = 0

    @classmethod
    def whole(cls, key: str, data: torch.Tensor, replica_id: int = 0) -> "ShardedTensor":
        return cls(key, data, tuple(data.shape), [((0,) * data.dim(), tuple(data.shape))], replica_id)

    @classmethod
    def slice_1d(cls, key: str, data: torch.Tensor, global_numel: int, offset: int, replica_id: int = 0) -> "ShardedTensor":
        return cls(key, data, (int(global_numel),), [((int(offset),), (int(data.numel()),))], replica_id)


@dataclass
class ShardedObject:
    key: str
    obj: object
    global_shape: tuple = (1,)
    global_offset: tuple = (0,)
    replica_id: int = 0


def shard_file(offset, shape, prefix: str = "shard", ext: str = "pt") -> str:
    """``shard_<o1.o2>_<s1.s2>.pt``: dots between dimensions, an underscore between offset and shape."""
    return f"{prefix}_{'.'.join(str(int(o)) for o in offset)}_{'.'.join(str(int(s)) for s in shape)}.{ext}"


def _rank_world(group=None):
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def _barrier(group=None):
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.barrier(group=group)


def _as_numpy(t: torch.Tensor) -> np.ndarray:
    t = t.contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view("<u2")
    return t.numpy()


def _key_dir(key: str) -> str:
    return key.replace("/", "__")


class AsyncSaveRequest:
    """Handle of a running save. ``finalize()`` joins the writer, synchronises the ranks and lets rank 0 publish
    ``metadata.json`` (a checkpoint without that file is incomplete and refused by ``load_sharded``)."""

    def __init__(self, ckpt_dir: str, thread: threading.Thread | None, group, errors: list):
        self.ckpt_dir, self._thread, self._group, self._errors = ckpt_dir, thread, group, errors
        self.finalized = False

    def done(self) -> bool:
        return self._thread is None or not self._thread.is_alive()

    def finalize(self) -> None:
        if self.finalized:
            return
        if self._thread is not None:
            self._thread.join()
        if self._errors:
            raise RuntimeError("asynchronous sharded save failed") from self._errors[0]
        _barrier(self._group)
        rank, world = _rank_world(self._group)
        if rank == 0:
            _merge_manifests(self.ckpt_dir, world)
        _barrier(self._group)
        self.finalized = True


def _merge_manifests(ckpt_dir: str, world: int) -> None:
    tensors: dict = {}
    objects: dict = {}
    for r in range(world):
        with open(os.path.join(ckpt_dir, "manifests", f"rank_{r}.json")) as f:
            m = json.load(f)
        for key, rec in m["tensors"].items():
            cur = tensors.setdefault(key, {"dtype": rec["dtype"], "global_shape": rec["global_shape"], "chunks": []})
            if cur["dtype"] != rec["dtype"] or cur["global_shape"] != rec["global_shape"]:
                raise ValueError(f"ranks disagree about array '{key}': {cur['dtype']} {cur['global_shape']} vs "
                                 f"{rec['dtype']} {rec['global_shape']}")
            cur["chunks"].extend(rec["chunks"])
        for key, rec in m["objects"].items():
            objects.setdefault(key, []).extend(rec)
    tmp = os.path.join(ckpt_dir, "metadata.json.tmp")
    with open(tmp, "w") as f:
        json.dump({"format": FORMAT, "version": VERSION, "world_size": world, "tensors": tensors, "objects": objects}, f)
    os.replace(tmp, os.path.join(ckpt_dir, "metadata.json"))


def save_sharded(state: dict, ckpt_dir: str, group=None, async_save: bool = True) -> AsyncSaveRequest:
    """``state``: key -> ShardedTensor | ShardedObject. Returns after the preload stage; call ``finalize()`` on the
    result before relying on the checkpoint (and before the next save into the same directory)."""
    rank, _ = _rank_world(group)
    for sub in ("arrays", "objects", "manifests"):
        os.makedirs(os.path.join(ckpt_dir, sub), exist_ok=True)
    stale = os.path.join(ckpt_dir, "metadata.json")
    if rank == 0 and os.path.exists(stale):
        os.remove(stale)
    # ---- preload: host copies of what this rank writes
    work, objs = [], []
    manifest = {"tensors": {}, "objects": {}}
    on_gpu = False
    for key, item in state.items():
        if isinstance(item, ShardedObject):
            if item.replica_id == 0:
                objs.append((item, pickle.dumps(_strip_device(item.obj))))
            continue
        assert isinstance(item, ShardedTensor), f"'{key}': expected ShardedTensor or ShardedObject, got {type(item)}"
        if item.replica_id != 0 or item.data is None:
            continue
        t = item.data.detach()
        rows = sum(int(np.prod(s)) for _, s in item.boxes)
        assert rows == t.numel(), f"'{key}': boxes cover {rows} elements, data has {t.numel()}"
        if t.is_cuda:
            host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            host.copy_(t, non_blocking=True)
            on_gpu = True
        else:
            host = t.clone()
        work.append((item, host))
    if on_gpu:
        torch.cuda.current_stream().synchronize()

    errors: list = []

    def write():
        try:
            for item, host in work:
                d = os.path.join(ckpt_dir, "arrays", _key_dir(item.key))
                os.makedirs(d, exist_ok=True)
                flat = _as_numpy(host).reshape(-1)
                rec = manifest["tensors"].setdefault(item.key, {"dtype": str(item.data.dtype), "global_shape": list(item.global_shape),
                                                                "chunks": []})
                pos = 0
                for off, shp in item.boxes:
                    n = int(np.prod(shp))
                    name = shard_file(off, shp, "c", "bin")
                    tmp = os.path.join(d, name + f".tmp{rank}")
                    flat[pos:pos + n].tofile(tmp)
                    os.replace(tmp, os.path.join(d, name))
                    rec["chunks"].append({"offset": [int(o) for o in off], "shape": [int(s) for s in shp], "file": name})
                    pos += n
            for item, blob in objs:
                d = os.path.join(ckpt_dir, "objects", _key_dir(item.key))
                os.makedirs(d, exist_ok=True)
                name = shard_file(item.global_offset, item.global_shape)
                with open(os.path.join(d, name), "wb") as f:
                    f.write(blob)
                manifest["objects"].setdefault(item.key, []).append({"offset": list(item.global_offset), "shape": list(item.global_shape),
                                                                     "file": name})
            with open(os.path.join(ckpt_dir, "manifests", f"rank_{rank}.json"), "w") as f:
                json.dump(manifest, f)
        except BaseException as e:          # noqa: BLE001 - surfaced by finalize()
            errors.append(e)

    if async_save:
        th = threading.Thread(target=write, name="sharded-ckpt-writer", daemon=True)
        th.start()
        return AsyncSaveRequest(ckpt_dir, th, group, errors)
    write()
    req = AsyncSaveRequest(ckpt_dir, None, group, errors)
    req.finalize()
    return req


def _strip_device(obj):
    """Tensors to the host, generators to their state (a CUDA generator cannot be unpickled on another machine)."""
    if isinstance(obj, torch.Tensor):
        return obj.detach().cpu()
    if isinstance(obj, torch.Generator):
        return {"__generator_state__": obj.get_state().cpu()}
    if isinstance(obj, dict):
        return {k: _strip_device(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_strip_device(v) for v in obj)
    return obj


def read_metadata(ckpt_dir: str) -> dict:
    path = os.path.join(ckpt_dir, "metadata.json")
    if not os.path.exists(path):
        raise FileNotFoundError(f"{ckpt_dir} has no metadata.json: the save was not finalized (or this is another layout)")
    with open(path) as f:
        meta = json.load(f)
    if meta.get("format") != FORMAT:
        raise ValueError(f"{path}: format {meta.get('format')!r}, expected {FORMAT!r}")
    return meta


def _read_box(ckpt_dir: str, key: str, rec: dict, off, shp) -> np.ndarray:
    """The box (off, shp) of array ``key`` assembled from every chunk that overlaps it."""
    dt = np.dtype(_NP[_TORCH[rec["dtype"]]])
    out = np.empty(tuple(int(s) for s in shp), dtype=dt)
    filled = 0
    nd = len(shp)
    for ch in rec["chunks"]:
        co, cs = ch["offset"], ch["shape"]
        lo = [max(int(off[d]), co[d]) for d in range(nd)]
        hi = [min(int(off[d]) + int(shp[d]), co[d] + cs[d]) for d in range(nd)]
        if any(h <= l for l, h in zip(lo, hi)):
            continue
        src = np.memmap(os.path.join(ckpt_dir, "arrays", _key_dir(key), ch["file"]), dtype=dt, mode="r", shape=tuple(cs))
        s_idx = tuple(slice(lo[d] - co[d], hi[d] - co[d]) for d in range(nd))
        d_idx = tuple(slice(lo[d] - int(off[d]), hi[d] - int(off[d])) for d in range(nd))
        out[d_idx] = src[s_idx]
        filled += int(np.prod([h - l for l, h in zip(lo, hi)]))
    want = int(np.prod(shp))
    if filled < want:
        raise ValueError(f"array '{key}': box offset {tuple(off)} shape {tuple(shp)} is only covered for {filled} of {want} elements")
    return out


def load_sharded(template: dict, ckpt_dir: str, group=None, strict: bool = True) -> dict:
    """Fill ``template`` (key -> ShardedTensor whose ``data`` is the destination, or ShardedObject) from the
    checkpoint: each rank reads exactly its boxes, whatever layout wrote them. Returns key -> loaded object for the
    ShardedObject entries. Chunks written twice (overlapping replicas) are fine; gaps raise."""
    meta = read_metadata(ckpt_dir)
    out = {}
    for key, item in template.items():
        if isinstance(item, ShardedObject):
            recs = meta["objects"].get(key)
            if not recs:
                if strict:
                    raise KeyError(f"object '{key}' is not in {ckpt_dir}")
                continue
            name = shard_file(item.global_offset, item.global_shape)
            rec = next((r for r in recs if r["file"] == name), recs[0])
            with open(os.path.join(ckpt_dir, "objects", _key_dir(key), rec["file"]), "rb") as f:
                out[key] = pickle.load(f)
            continue
        rec = meta["tensors"].get(key)
        if rec is None:
            if strict:
                raise KeyError(f"array '{key}' is not in {ckpt_dir}")
            continue
        if tuple(rec["global_shape"]) != tuple(int(s) for s in item.global_shape):
            raise ValueError(f"array '{key}': checkpoint has global shape {rec['global_shape']}, this run expects {list(item.global_shape)}")
        dst = item.data
        parts = [_read_box(ckpt_dir, key, rec, off, shp).reshape(-1) for off, shp in item.boxes]
        flat = np.concatenate(parts) if len(parts) > 1 else parts[0]
        src_dtype = _TORCH[rec["dtype"]]
        t = torch.from_numpy(np.ascontiguousarray(flat))
        if src_dtype == torch.bfloat16:
            t = t.view(torch.int16).view(torch.bfloat16)
        dst.copy_(t.view(dst.shape).to(dst.dtype))
    if group is not False:               # False: a single rank reads on its own (no collective)
        _barrier(group)
    return out
