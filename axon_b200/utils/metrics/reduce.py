"""Reduce lists of per-micro-batch values to one number per key
(reference: axon/utils/metrics/reduce_metrics.py:30-64)."""
from __future__ import annotations

import re
from typing import Any

import numpy as np

_MAX = re.compile(r"(?<![A-Za-z0-9])max(?![A-Za-z0-9])")
_MIN = re.compile(r"(?<![A-Za-z0-9])min(?![A-Za-z0-9])")


def append_to_dict(data: dict, new_data: dict) -> None:
    for k, v in new_data.items():
        data.setdefault(k, [])
        if isinstance(v, (list, tuple)):
            data[k].extend(v)
        else:
            data[k].append(v)


def reduce_metrics(metrics: dict[str, list[Any]]) -> dict[str, Any]:
    """Mean of each list — except keys with a stand-alone ``max`` / ``min`` token
    (``grad_norm/max``, ``max_reward``), which take the maximum / minimum."""
    out = {}
    for key, vals in metrics.items():
        flat = np.concatenate([np.atleast_1d(np.asarray(v, dtype=np.float64)) for v in vals]) if len(vals) else np.zeros(0)
        if flat.size == 0:
            continue
        out[key] = float(flat.max() if _MAX.search(key) else flat.min() if _MIN.search(key) else flat.mean())
    return out
