"""Offline check of weight-sync plans.

The reference ships a tool that reads the send / receive logs of a P2P sync and verifies that both sides issue
matching operations in the same order (axon/utils/p2p/verify_p2p_order.py) - with NCCL send / recv a mismatch is a
deadlock. The sync here is a list of slice-copy descriptors executed by one kernel per sender, so order cannot
deadlock; what can go wrong is coverage: an element of a sampler buffer written twice (two senders racing) or
never (stale weights). ``verify_plans`` checks exactly that from the compiled plans, before anything runs.
"""
from __future__ import annotations

import numpy as np

from .plan import SyncPlan


def coverage(plans: dict[int, SyncPlan], sampler_sizes: dict[int, int]) -> dict[int, np.ndarray]:
    """How many times each element of every sampler rank's flat buffer is written, over all senders."""
    hits = {r: np.zeros(n, dtype=np.int32) for r, n in sampler_sizes.items()}
    for plan in plans.values():
        for d in plan.descs:
            h = hits[int(d["dst_rank"])]
            rows, cols, stride, off = int(d["rows"]), int(d["cols"]), int(d["dst_stride"]), int(d["dst_off"])
            for r in range(rows):
                h[off + r * stride:off + r * stride + cols] += 1
    return hits


def verify_plans(plans: dict[int, SyncPlan], sampler_expected: dict[int, list[tuple[int, int]]], verbose: bool = False) -> dict:
    """``plans``: sender rank -> its plan. ``sampler_expected``: sampler rank -> [(offset, numel)] spans that must be
    written (its parameters' shards inside the flat buffer; padding between them must stay untouched).
    Returns {"ok", "missing", "duplicated", "stray", "bytes_per_sender"}; element counts per sampler rank."""
    sizes = {r: max((o + n for o, n in spans), default=0) for r, spans in sampler_expected.items()}
    for plan in plans.values():
        for d in plan.descs:
            r = int(d["dst_rank"])
            end = int(d["dst_off"]) + (int(d["rows"]) - 1) * int(d["dst_stride"]) + int(d["cols"])
            sizes[r] = max(sizes.get(r, 0), end)
    hits = coverage(plans, sizes)
    report = {"missing": {}, "duplicated": {}, "stray": {}, "bytes_per_sender": {s: p.total_bytes for s, p in plans.items()}}
    for r, h in hits.items():
        want = np.zeros_like(h, dtype=bool)
        for o, n in sampler_expected.get(r, []):
            want[o:o + n] = True
        report["missing"][r] = int(np.count_nonzero(want & (h == 0)))
        report["duplicated"][r] = int(np.count_nonzero(h > 1))
        report["stray"][r] = int(np.count_nonzero(~want & (h > 0)))
    report["ok"] = not any(v for k in ("missing", "duplicated", "stray") for v in report[k].values())
    if verbose:
        for k in ("missing", "duplicated", "stray"):
            print(k, report[k])
        print("bytes per sender", report["bytes_per_sender"])
    return report
