"""DataProto behaviours: construction, slicing, concat with metrics, padding, repeat, serialisation."""
import os
import pickle

import numpy as np
import pytest
import torch

from axon_b200.protocol import (DataProto, DataProtoFuture, fold_batch_dim, pad_dataproto_to_divisor,
                                unfold_batch_dim, unpad_dataproto)


def make(n=6):
    return DataProto.from_dict(
        {"a": torch.arange(n * 3).view(n, 3).float(), "b": torch.arange(n)},
        {"uid": np.array([f"u{i}" for i in range(n)], dtype=object)}, {"tag": 1})


def test_basic_indexing_and_select():
    d = make()
    assert len(d) == 6
    assert d[2].batch["b"].item() == 2 and d[2].non_tensor_batch["uid"] == "u2"
    s = d[1:4]
    assert len(s) == 3 and s.non_tensor_batch["uid"].tolist() == ["u1", "u2", "u3"]
    p = d.select_idxs([5, 0])
    assert p.batch["b"].tolist() == [5, 0]
    sel = d.select(batch_keys=["a"], non_tensor_batch_keys=[])
    assert list(sel.batch.keys()) == ["a"] and sel.non_tensor_batch == {}
    popped = d.pop(batch_keys=["b"], non_tensor_batch_keys=["uid"])
    assert "b" not in d.batch and "uid" not in d.non_tensor_batch and len(popped) == 6
    d.rename("a", "c")
    assert "c" in d.batch


def test_consistency_errors():
    with pytest.raises(AssertionError):
        DataProto.from_dict({"a": torch.zeros(3, 2), "b": torch.zeros(4)})
    with pytest.raises(AssertionError):
        DataProto.from_dict({"a": torch.zeros(3)}, {"x": np.zeros(2)})


def test_union_and_conflict():
    d1, d2 = make(), DataProto.from_dict({"c": torch.ones(6)}, meta_info={"tag": 1, "new": 2})
    d1.union(d2)
    assert "c" in d1.batch and d1.meta_info["new"] == 2
    with pytest.raises(AssertionError):
        d1.union(DataProto.from_dict({"c": torch.zeros(6)}))


def test_chunk_concat_metrics_roundtrip():
    d = make()
    chunks = d.chunk(3)
    assert [len(c) for c in chunks] == [2, 2, 2]
    for i, c in enumerate(chunks):
        c.meta_info = {"tag": 1, "metrics": {"loss": float(i)}}
    back = DataProto.concat(chunks)
    assert torch.equal(back.batch["a"], d.batch["a"])
    assert back.meta_info["metrics"] == {"loss": [0.0, 1.0, 2.0]} and back.meta_info["tag"] == 1
    with pytest.raises(AssertionError):
        d.chunk(4)
    assert [len(x) for x in d.split(4)] == [4, 2]


def test_padding_helpers():
    d = make(5)
    padded, pad = pad_dataproto_to_divisor(d, 4)
    assert len(padded) == 8 and pad == 3
    assert padded.batch["b"].tolist() == [0, 1, 2, 3, 4, 0, 1, 2]
    assert len(unpad_dataproto(padded, pad)) == 5
    same, pad0 = pad_dataproto_to_divisor(d, 5)
    assert pad0 == 0 and same is d
    big, padn = pad_dataproto_to_divisor(make(2), 7)
    assert len(big) == 7 and padn == 5


def test_repeat_variants():
    d = make(3)
    assert d.repeat(2, interleave=True).batch["b"].tolist() == [0, 0, 1, 1, 2, 2]
    assert d.repeat(2, interleave=False).batch["b"].tolist() == [0, 1, 2, 0, 1, 2]
    assert d.sample_level_repeat([1, 0, 2]).batch["b"].tolist() == [0, 2, 2]
    assert d.repeat_by_counts([2, 1, 0], interleave=False).batch["b"].tolist() == [0, 1, 0]
    u = DataProto.from_dict({"x": torch.arange(12).view(2, 6), "y": torch.tensor([7, 8])})
    un = u.unfold_column_chunks(3, split_keys=["x"])
    assert un.batch["x"].shape == (6, 2) and un.batch["y"].tolist() == [7, 7, 7, 8, 8, 8]


def test_iterator_and_reorder():
    d = make(8)
    seen = []
    for mb in d.make_iterator(4, epochs=2, seed=1):
        assert len(mb) == 4
        seen.extend(mb.batch["b"].tolist())
    assert sorted(seen) == sorted(list(range(8)) * 2)
    d.reorder(torch.tensor([7, 6, 5, 4, 3, 2, 1, 0]))
    assert d.batch["b"].tolist()[0] == 7 and d.non_tensor_batch["uid"][0] == "u7"


@pytest.mark.parametrize("method", ["torch", "numpy"])
def test_pickle_roundtrip(method, tmp_path, monkeypatch):
    monkeypatch.setenv("AXON_DATAPROTO_SERIALIZATION_METHOD", method)
    d = make()
    d.batch["h"] = torch.randn(6, 2).to(torch.bfloat16)
    e = pickle.loads(pickle.dumps(d))
    assert torch.equal(e.batch["a"], d.batch["a"]) and torch.equal(e.batch["h"], d.batch["h"])
    assert e.non_tensor_batch["uid"].tolist() == d.non_tensor_batch["uid"].tolist() and e.meta_info == d.meta_info
    d.save_to_disk(str(tmp_path / "x.pkl"))
    assert len(DataProto.load_from_disk(str(tmp_path / "x.pkl"))) == 6


def test_fold_unfold_and_future():
    d = make(6)
    f = fold_batch_dim(d, 2)
    assert f.batch["a"].shape == (2, 3, 3)
    assert torch.equal(unfold_batch_dim(f).batch["a"], d.batch["a"])
    fut = DataProtoFuture.concat([d[:3], d[3:]])
    parts = fut.chunk(2)
    assert torch.equal(parts[1].get().batch["b"], torch.tensor([3, 4, 5]))


def test_auto_padding_chunk():
    d = DataProto.from_dict({"a": torch.arange(5)}, auto_padding=True)
    assert [len(c) for c in d.chunk(2)] == [3, 2]
    d2 = make(3)
    d2.padding(2)
    assert d2.batch["b"].tolist() == [0, 1, 2, 2, 2]
