"""Dataset generator for the FrozenLake recipe: every row is an environment configuration (seed, size, p) plus the
program columns the driver expects (reference: recipes/frozenlake/data.py).

    python recipes/frozenlake/data.py --train_size 10000 --test_size 100 --out data/frozenlake
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np


def make_rows(n: int, rng: np.random.Generator, split: str) -> list[dict]:
    rows = []
    for i in range(n):
        env = {"seed": int(rng.integers(0, 2 ** 31 - 1)), "size": int(rng.integers(2, 10)), "p": float(rng.uniform(0.6, 0.85)),
               "is_slippery": False}
        rows.append({"data_source": "frozenlake", "index": i, "split": split, "env_name": "frozenlake", "agent_name": "frozenlake",
                     "env_args": env, "prompt": [{"role": "user", "content": "frozenlake"}]})
    return rows


def write(rows: list[dict], path: str) -> None:
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    try:
        import pandas as pd
        pd.DataFrame(rows).to_parquet(path)
    except Exception:  # noqa: BLE001 - no parquet engine: fall back to json lines beside the requested name
        path = os.path.splitext(path)[0] + ".jsonl"
        with open(path, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    print(f"wrote {len(rows)} rows to {path}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--train_size", type=int, default=10000)
    ap.add_argument("--test_size", type=int, default=100)
    ap.add_argument("--out", default="data/frozenlake")
    ap.add_argument("--seed", type=int, default=42)
    args = ap.parse_args()
    rng = np.random.default_rng(args.seed)
    write(make_rows(args.train_size, rng, "train"), os.path.join(args.out, "train.parquet"))
    write(make_rows(args.test_size, rng, "test"), os.path.join(args.out, "test.parquet"))


if __name__ == "__main__":
    main()
