"""Named benchmark datasets and loaders for prepared task files
(reference: axon/utils/dataset_utils.py:50-203). ``load_dataset`` reads
``<root>/<category>/<split>/<name>.{json,jsonl,parquet}`` produced by the data-preparation
scripts; nothing is downloaded."""
from __future__ import annotations

import enum
import json
import os

from .system_prompts import (LCB_FORMATTING_MESSAGE_WITH_STARTER_CODE, LCB_FORMATTING_WITHOUT_STARTER_CODE,
                             LCB_SYSTEM_MESSAGE_GENERIC)


class TrainDataset:
    class Math(enum.Enum):
        AIME = "AIME"
        AMC = "AMC"
        OMNI_MATH = "OMNI_MATH"
        NUMINA_OLYMPIAD = "OLYMPIAD"
        MATH = "MATH"
        STILL = "STILL"
        DEEPSCALER = "DEEPSCALER"

    class Code(enum.Enum):
        TACO = "TACO"
        APPS = "APPS"
        CODEFORCES = "CODEFORCES"
        CODE_CONTESTS = "CODE_CONTESTS"
        LIVECODEBENCH = "LIVECODEBENCH"
        LEETCODE = "LEETCODE"
        PRIMEINTELLECT = "PRIMEINTELLECT"
        KODCODE = "KODCODE"

    class Web(enum.Enum):
        GAIA = "GAIA"


class TestDataset:
    class Math(enum.Enum):
        AIME = "AIME"
        AMC = "AMC"
        MATH = "MATH"
        MINERVA = "MINERVA"
        OLYMPIAD_BENCH = "OLYMPIAD_BENCH"

    class Code(enum.Enum):
        TACO = "TACO"
        CODEFORCES = "CODEFORCES"
        LIVECODEBENCH = "LIVECODEBENCH"
        LEETCODE = "LEETCODE"
        HUMANEVALPLUS = "HUMANEVALPLUS"

    class Web(enum.Enum):
        GAIA = "GAIA"


def load_dataset(dataset: enum.Enum, root: str | None = None) -> list[dict]:
    root = root or os.environ.get("AXON_DATA_ROOT", os.path.join(os.getcwd(), "data"))
    split = "train" if dataset.__class__.__qualname__.startswith("TrainDataset") else "test"
    category = dataset.__class__.__name__.lower()
    base = os.path.join(root, category, split, dataset.value.lower())
    for ext in (".json", ".jsonl", ".parquet"):
        path = base + ext
        if not os.path.exists(path):
            continue
        if ext == ".json":
            return json.load(open(path))
        if ext == ".jsonl":
            return [json.loads(line) for line in open(path) if line.strip()]
        import pyarrow.parquet as pq
        return pq.read_table(path).to_pylist()
    raise FileNotFoundError(f"no prepared file for {dataset} under {base}.(json|jsonl|parquet)")


def fetch_live_code_bench_system_prompt(prompt: str, starter_code: str | None = None) -> str:
    out = LCB_SYSTEM_MESSAGE_GENERIC + "\n\n" + prompt + "\n\n"
    if starter_code:
        return out + LCB_FORMATTING_MESSAGE_WITH_STARTER_CODE + f"\n```python\n{starter_code}\n```\n\n"
    return out + LCB_FORMATTING_WITHOUT_STARTER_CODE + "\n```python\n# YOUR CODE HERE\n```\n\n"
