"""Degenerate-repetition detector: text that compresses extremely well is looping
(reference: axon/utils/metrics/repetition.py:35-141)."""
from __future__ import annotations

import bz2
import gzip
import lzma
import zlib
from typing import Any

_COMPRESSORS = {"zlib": lambda b, lv: zlib.compress(b, lv), "gzip": lambda b, lv: gzip.compress(b, compresslevel=lv),
                "bz2": lambda b, lv: bz2.compress(b, compresslevel=lv), "lzma": lambda b, lv: lzma.compress(b, preset=lv)}


def compression_ratio(data, *, encoding: str = "utf-8", algorithm: str = "zlib", level: int = 9) -> tuple[float, float]:
    """(original/compressed size, percent saved)."""
    raw = data.encode(encoding) if isinstance(data, str) else bytes(data)
    if not raw:
        return float("inf"), 0.0
    if algorithm not in _COMPRESSORS:
        raise ValueError(f"unsupported algorithm '{algorithm}'")
    n = len(_COMPRESSORS[algorithm](raw, level))
    return (float("inf"), 100.0) if n == 0 else (len(raw) / n, 100.0 * (1.0 - n / len(raw)))


def has_repetition(text: str, *, tail_chars: int = 10000, threshold: float = 10.0) -> bool:
    return len(text) > tail_chars and compression_ratio(text[-tail_chars:])[0] > threshold


def compute_repetition_metrics(batch, tokenizer) -> dict[str, Any]:
    ids, rm = batch.batch["input_ids"], batch.batch["response_mask"].bool()
    rows = [ids[i][rm[i]].tolist() for i in range(ids.size(0))]
    if hasattr(tokenizer, "batch_decode"):
        texts = tokenizer.batch_decode(rows, skip_special_tokens=False)
    else:
        texts = [tokenizer.decode(r) for r in rows]
    return {"response/repetition_frac": sum(map(has_repetition, texts)) / len(texts) if texts else 0.0}
