"""Dataset, dynamic loader (mid-epoch resume) and data samplers."""
import json

import numpy as np
import pytest
import torch

from axon_b200.data import DynamicDataLoader, RLDataset, collate_rl_dataset, create_data_sampler
from axon_b200.data.data_sampler import ExpWeightedCurriculumSampler, SeededRandomSampler, ThresholdMaskingSampler
from axon_b200.protocol import DataProto


def _write(tmp_path, name, n, tag):
    p = tmp_path / name
    with open(p, "w") as f:
        for i in range(n):
            f.write(json.dumps({"q": f"{tag}{i}", "answer": i}) + "\n")
    return str(p)


def test_dataset_jsonl_parquet_and_mix(tmp_path):
    a = _write(tmp_path, "a.jsonl", 4, "a")
    import pyarrow as pa
    import pyarrow.parquet as pq
    b = str(tmp_path / "b.parquet")
    pq.write_table(pa.table({"q": [f"b{i}" for i in range(6)], "answer": list(range(6))}), b)
    ds = RLDataset([a, b], file_weights=[0.75, 0.25])
    assert len(ds) == 10 and ds[5]["data"]["q"] == "b1" and ds[5]["index"] == 5
    assert abs(sum(ds.sample_weights) - 1.0) < 1e-9 and abs(ds.sample_weights[0] - 0.75 / 4) < 1e-12
    with pytest.raises(ValueError):
        RLDataset([a], file_weights=[1.0, 2.0])
    with pytest.raises(ValueError):
        RLDataset([str(tmp_path / "x.csv")])
    out = collate_rl_dataset([ds[0], ds[9]])
    assert out["env_args"][1]["q"] == "b5" and out["index"].tolist() == [0, 9]
    with pytest.warns(UserWarning):
        s = create_data_sampler({"data_sampler": "sequential", "data_sampler_args": {"seed": 1}}, ds)
    assert isinstance(s, SeededRandomSampler) and s.weights is not None


def test_dynamic_loader_wraps_and_resumes(tmp_path):
    ds = RLDataset(_write(tmp_path, "a.jsonl", 7, "a"))
    make = lambda: DynamicDataLoader(ds, collate_fn=collate_rl_dataset, sampler=SeededRandomSampler(ds, seed=3), infinite=True)  # noqa: E731
    ld = make()
    seen = [ld.next(3)["index"].tolist() for _ in range(2)]
    state = ld.state_dict()
    rest = [ld.next(4)["index"].tolist() for _ in range(3)]              # crosses the epoch boundary twice
    assert sorted(seen[0] + seen[1] + rest[0][:1]) == list(range(7)) and ld.epoch >= 1
    ld2 = make()
    ld2.load_state_dict(state)
    assert [ld2.next(4)["index"].tolist() for _ in range(3)] == rest
    fin = DynamicDataLoader(ds, collate_fn=collate_rl_dataset, infinite=False)
    assert fin.next(5)["index"].tolist() == [0, 1, 2, 3, 4] and fin.next(5)["index"].tolist() == [5, 6]
    with pytest.raises(StopIteration):
        fin.next(1)


def test_curriculum_samplers(tmp_path):
    ds = RLDataset(_write(tmp_path, "a.jsonl", 6, "a"))
    fb = DataProto.from_dict(tensors={"x": torch.zeros(3, 1)}, non_tensors={"index": np.array([0, 1, 2]),
                                                                            "pass_rate": np.array([1.0, 0.0, 0.5])})
    ew = create_data_sampler({"data_sampler": "exp_weighted_curriculum", "data_sampler_args": {"min_weight": 0.1, "max_weight": 2.0, "seed": 0}}, ds)
    assert isinstance(ew, ExpWeightedCurriculumSampler)
    ew.update(fb)
    assert ew.weights[0] == 0.1 and ew.weights[1] == 2.0 and abs(ew.weights[2] - np.exp(-0.5)) < 1e-12
    st = ew.state_dict()
    ew2 = ExpWeightedCurriculumSampler(ds)
    ew2.load_state_dict(st)
    assert list(ew2) == list(ew) or len(list(ew2)) == 6
    tm = create_data_sampler({"data_sampler": "threshold_masking_curriculum", "data_sampler_args": {"threshold": 0.9, "seed": 0}}, ds)
    assert isinstance(tm, ThresholdMaskingSampler)
    tm.update(fb)
    assert tm.masked.tolist() == [True, False, False, False, False, False] and 0 not in set(tm)
    tm.update(DataProto.from_dict(tensors={"x": torch.zeros(5, 1)}, non_tensors={"index": np.arange(1, 6), "pass_rate": np.ones(5)}))
    assert not tm.masked[1] and tm.masked[3]                    # row 1 averages 0.5; rows 3.. reach the threshold
    tm.masked[:] = True
    assert len(list(tm)) == 6                                   # everything masked: fall back to the whole set
