"""Turns question / answer files into the rows the driver reads (reference: recipes/math/data.py, which pulls
GSM8K / MATH / DeepScaleR from the hub). There is no hub access here, so the input is a local ``.jsonl`` or
``.parquet`` with a question column and an answer column; without an input a small arithmetic set is generated,
enough to smoke-test the recipe end to end.

    python recipes/math/data.py --input gsm8k_train.jsonl --question question --answer answer --out data/math/train.parquet
"""
from __future__ import annotations

import argparse
import json
import os
import re

import numpy as np


def final_answer(text: str) -> str:
    """GSM8K-style answers end in ``#### 42``; boxed answers and plain values pass through."""
    m = re.search(r"####\s*(.+)$", str(text).strip())
    return (m.group(1) if m else str(text)).strip().replace(",", "")


def synthetic(n: int, seed: int) -> list[dict]:
    rng = np.random.default_rng(seed)
    rows = []
    for _ in range(n):
        a, b, c = (int(x) for x in rng.integers(2, 60, 3))
        rows.append({"question": f"Compute {a} * {b} + {c}.", "answer": str(a * b + c)})
    return rows


def to_rows(items: list[dict], q_col: str, a_col: str, source: str, split: str) -> list[dict]:
    return [{"data_source": source, "index": i, "split": split, "env_name": "math", "agent_name": "math",
             "question": str(it[q_col]), "ground_truth": final_answer(it[a_col]), "reward_fn": "math",
             "prompt": [{"role": "user", "content": str(it[q_col])}]} for i, it in enumerate(items)]


def read(path: str) -> list[dict]:
    if path.endswith(".parquet"):
        import pandas as pd
        return pd.read_parquet(path).to_dict("records")
    with open(path) as f:
        return [json.loads(line) for line in f if line.strip()]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", default=None)
    ap.add_argument("--question", default="question")
    ap.add_argument("--answer", default="answer")
    ap.add_argument("--source", default="math")
    ap.add_argument("--split", default="train")
    ap.add_argument("--out", default="data/math/train.parquet")
    ap.add_argument("--synthetic_size", type=int, default=512)
    args = ap.parse_args()
    items = read(args.input) if args.input else synthetic(args.synthetic_size, 0)
    rows = to_rows(items, args.question, args.answer, args.source, args.split)
    os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
    try:
        import pandas as pd
        pd.DataFrame(rows).to_parquet(args.out)
        out = args.out
    except Exception:  # noqa: BLE001
        out = os.path.splitext(args.out)[0] + ".jsonl"
        with open(out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    print(f"wrote {len(rows)} rows to {out}")


if __name__ == "__main__":
    main()
