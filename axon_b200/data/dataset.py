"""Task dataset for RL: rows of arbitrary dictionaries that become environment arguments.

Reads ``.parquet`` (pyarrow) and ``.jsonl`` files; several files concatenate in order, and optional
per-file mixing weights become per-row sampling weights (each file's weight spread evenly over its
rows) that the random data sampler honours. With no files the dataset is empty and the loader yields
nothing (reference behaviour: axon/data/dataset.py:29-85).
"""
from __future__ import annotations

import json
from typing import Optional, Sequence

import torch


def collate_rl_dataset(batch: list[dict]) -> dict:
    """Rows stay a list of dicts (``env_args``); the dataset indices become one tensor."""
    return {"env_args": [item["data"] for item in batch],
            "index": torch.tensor([item["index"] for item in batch], dtype=torch.long)}


def _read_parquet(path: str) -> list[dict]:
    import pyarrow.parquet as pq
    return pq.read_table(path).to_pylist()


def _read_jsonl(path: str) -> list[dict]:
    rows = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line:
                rows.append(json.loads(line))
    return rows


class RLDataset(torch.utils.data.Dataset):
    def __init__(self, data_files: Optional[str | Sequence[str]] = None, file_weights: Optional[Sequence[float]] = None,
                 rows: Optional[list[dict]] = None):
        self.sample_weights: Optional[list[float]] = None
        self.data: list[dict] = list(rows) if rows is not None else []
        if data_files:
            self._load(data_files, file_weights)

    def _load(self, data_files, file_weights) -> None:
        files = [data_files] if isinstance(data_files, str) else [str(p) for p in data_files]
        if file_weights is not None and len(file_weights) != len(files):
            raise ValueError(f"data_mix has {len(file_weights)} weights for {len(files)} files")
        weights: list[float] = []
        for i, path in enumerate(files):
            if path.endswith(".parquet"):
                rows = _read_parquet(path)
            elif path.endswith(".jsonl") or path.endswith(".json"):
                rows = _read_jsonl(path)
            else:
                raise ValueError(f"unsupported data file '{path}': expected .parquet or .jsonl")
            self.data.extend(rows)
            if file_weights is not None:
                weights.extend([file_weights[i] / len(rows) if rows else 0.0] * len(rows))
        if file_weights is not None:
            self.sample_weights = weights

    def __len__(self) -> int:
        return len(self.data)

    def __getitem__(self, index: int) -> dict:
        if not 0 <= index < len(self.data):
            raise IndexError(f"index {index} out of range for dataset of {len(self.data)} rows")
        return {"data": self.data[index], "index": int(index)}
