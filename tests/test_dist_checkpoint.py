"""Layout-independent sharded checkpoints: boxes written under one layout are read back under another, objects,
asynchronous save and refusal of unfinished or incomplete checkpoints."""
import os
import subprocess
import sys

import pytest
import torch

from axon_b200.utils.state.dist_checkpoint import (ShardedObject, ShardedTensor, load_sharded, read_metadata,
                                                   save_sharded, shard_file)


def test_boxes_written_by_rows_are_read_by_columns(tmp_path):
    full = torch.randn(12, 10).to(torch.bfloat16)
    vec = torch.arange(100, dtype=torch.float32)
    # "two ranks" with row shards (the first one in two boxes, as a fused qkv shard is), written by one process
    a = ShardedTensor("w", torch.cat([full[0:2], full[6:8]]), (12, 10), [((0, 0), (2, 10)), ((6, 0), (2, 10))])
    d = str(tmp_path / "ck")
    save_sharded({"w": a, "v": ShardedTensor.slice_1d("v", vec[:60], 100, 0),
                  "meta": ShardedObject("meta", {"step": 3, "t": torch.ones(2)})}, d, async_save=False)
    # metadata is only that of the last writer here; emulate the second rank by a second manifest
    b = ShardedTensor("w", torch.cat([full[2:6], full[8:12]]), (12, 10), [((2, 0), (4, 10)), ((8, 0), (4, 10))])
    import json
    from axon_b200.utils.state import dist_checkpoint as DC
    os.rename(os.path.join(d, "manifests", "rank_0.json"), os.path.join(d, "manifests", "rank_1.json"))
    save_sharded({"w": b, "v": ShardedTensor.slice_1d("v", vec[60:], 100, 60)}, d, async_save=False)
    DC._merge_manifests(d, 2)
    meta = read_metadata(d)
    assert len(meta["tensors"]["w"]["chunks"]) == 4 and meta["tensors"]["w"]["dtype"] == "torch.bfloat16"
    # read back by COLUMN shards and as one piece
    left, right, whole = torch.empty(12, 4, dtype=torch.bfloat16), torch.empty(12, 6, dtype=torch.bfloat16), torch.empty(12, 10, dtype=torch.bfloat16)
    v2 = torch.empty(30)
    objs = load_sharded({"w": ShardedTensor("w", left, (12, 10), [((0, 0), (12, 4))])}, d)
    load_sharded({"w": ShardedTensor("w", right, (12, 10), [((0, 4), (12, 6))]), "v": ShardedTensor.slice_1d("v", v2, 100, 45)}, d)
    objs = load_sharded({"w": ShardedTensor.whole("w", whole), "meta": ShardedObject("meta", None)}, d)
    assert torch.equal(left, full[:, :4]) and torch.equal(right, full[:, 4:]) and torch.equal(whole, full)
    assert torch.equal(v2, vec[45:75])
    assert objs["meta"]["step"] == 3 and torch.equal(objs["meta"]["t"], torch.ones(2))
    assert shard_file((47, 96), (94, 128)) == "shard_47.96_94.128.pt"
    # a box that no chunk covers is an error, not silent garbage
    os.remove(os.path.join(d, "arrays", "v", meta["tensors"]["v"]["chunks"][1]["file"]))
    meta["tensors"]["v"]["chunks"].pop(1)
    json.dump(meta, open(os.path.join(d, "metadata.json"), "w"))
    with pytest.raises(ValueError, match="only covered"):
        load_sharded({"v": ShardedTensor.slice_1d("v", torch.empty(100), 100, 0)}, d)


def test_async_save_is_incomplete_until_finalized(tmp_path):
    d = str(tmp_path / "ck")
    x = torch.randn(1000, 64)
    req = save_sharded({"x": ShardedTensor.whole("x", x)}, d, async_save=True)
    with pytest.raises(FileNotFoundError):
        if not os.path.exists(os.path.join(d, "metadata.json")):
            read_metadata(d)
    req.finalize()
    y = torch.empty_like(x)
    load_sharded({"x": ShardedTensor.whole("x", y)}, d)
    assert torch.equal(x, y)


_WORKER = r"""
import os, sys, json, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[3])
from axon_b200.models.config import tiny_qwen3
from axon_b200.models.dense import DenseModel
from axon_b200.models.params import FlatParams
from axon_b200.utils.state.dist_checkpoint import ShardedTensor, save_sharded, load_sharded
from axon_b200.utils.p2p.param_mapper import shard_rows
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
mode, d = sys.argv[1], sys.argv[2]
cfg = tiny_qwen3()
full = FlatParams(cfg, "cpu", torch.float32); full.init_random(seed=11)
def entries(tp, r, fill):
    out = {}
    for name, v in full.views.items():
        g2 = (v.shape[0], v[0].numel() if v.dim() > 1 else 1)
        rows = shard_rows(cfg, name, tp, r)
        boxes = [((r0, c0), (r1 - r0, c1 - c0)) for (r0, r1, c0, c1) in rows]
        v2 = v.reshape(g2)
        data = torch.cat([v2[r0:r1, c0:c1].reshape(-1) for (r0, r1, c0, c1) in rows]) if fill else torch.empty(sum((r1-r0)*(c1-c0) for (r0,r1,c0,c1) in rows))
        whole = len(rows) == 1 and rows[0] == (0, g2[0], 0, g2[1])
        out[name] = ShardedTensor(name, data, g2, boxes, 0 if (not whole or r == 0) else 1)
    return out
if mode == "save":                       # tensor-parallel layout over the two ranks
    save_sharded(entries(world, rank, True), d, async_save=True).finalize()
else:                                    # every rank reads the WHOLE model (tp = 1) and a 2-way layout again
    for tp, r in ((1, 0), (world, world - 1 - rank)):
        e = entries(tp, r, False)
        load_sharded(e, d)
        ref = entries(tp, r, True)
        for k in e:
            assert torch.equal(e[k].data, ref[k].data), k
dist.barrier()
if rank == 0: print("OK", mode)
"""


def test_tensor_parallel_save_then_load_under_other_layouts(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "w.py"
    script.write_text(_WORKER)
    d = str(tmp_path / "ck")
    for mode in ("save", "load"):
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                            "--master-port", "29641", str(script), mode, d, root], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0 and f"OK {mode}" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
