"""Moving the slices of a sync plan between processes that do not share memory.

The fused path (one kernel writing through peer pointers, ``plan.execute_plan``) needs the
destination buffers mapped into the sender — same node, symmetric memory. Everywhere else (CPU
ranks, gloo, different nodes) the same plan is carried by point-to-point messages: per destination
rank the sender packs all of that rank's slices into one contiguous staging buffer and sends it
once; the receiver, which derives the identical descriptor list from the routing table, unpacks it
into its parameter shards. One message per (sender, receiver) pair instead of one per slice.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from .plan import SyncPlan


def descs_for_rank(plan: SyncPlan, dst_rank: int) -> np.ndarray:
    return plan.descs[plan.descs["dst_rank"] == dst_rank]


def staging_numel(descs: np.ndarray) -> int:
    return int((descs["rows"].astype(np.int64) * descs["cols"].astype(np.int64)).sum())


def pack(descs: np.ndarray, src_flat: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    n = staging_numel(descs)
    out = out if out is not None else torch.empty(n, dtype=src_flat.dtype, device=src_flat.device)
    pos = 0
    for d in descs:
        r, c = int(d["rows"]), int(d["cols"])
        out[pos:pos + r * c].view(r, c).copy_(src_flat[int(d["src_off"]):].as_strided((r, c), (int(d["src_stride"]), 1)))
        pos += r * c
    return out


def unpack(descs: np.ndarray, staging: torch.Tensor, dst_flat: torch.Tensor) -> None:
    pos = 0
    for d in descs:
        r, c = int(d["rows"]), int(d["cols"])
        dst_flat[int(d["dst_off"]):].as_strided((r, c), (int(d["dst_stride"]), 1)).copy_(staging[pos:pos + r * c].view(r, c))
        pos += r * c


def send_plan(plan: SyncPlan, src_flat: torch.Tensor, group, rank_offset: int, cache: dict | None = None) -> int:
    """Sender side: one isend per destination rank (bridge rank = ``rank_offset + sampler rank``)."""
    reqs, sent = [], 0
    for dst in sorted(set(plan.descs["dst_rank"].tolist())):
        descs = descs_for_rank(plan, dst)
        buf = None
        if cache is not None:
            buf = cache.get(dst)
            if buf is None or buf.numel() != staging_numel(descs):
                buf = cache[dst] = torch.empty(staging_numel(descs), dtype=src_flat.dtype, device=src_flat.device)
        buf = pack(descs, src_flat, buf)
        reqs.append(dist.isend(buf, dst=rank_offset + int(dst), group=group))
        sent += buf.numel() * buf.element_size()
    for r in reqs:
        r.wait()
    return sent


def recv_plans(plans_by_src: dict[int, np.ndarray], dst_flat: torch.Tensor, group, cache: dict | None = None) -> int:
    """Receiver side: ``plans_by_src[bridge rank of the sender]`` = descriptors aimed at this rank."""
    reqs, got = [], 0
    for src, descs in sorted(plans_by_src.items()):
        n = staging_numel(descs)
        buf = None
        if cache is not None:
            buf = cache.get(src)
        if buf is None or buf.numel() != n:
            buf = torch.empty(n, dtype=dst_flat.dtype, device=dst_flat.device)
            if cache is not None:
                cache[src] = buf
        reqs.append((dist.irecv(buf, src=int(src), group=group), descs, buf))
    for req, descs, buf in reqs:
        req.wait()
        unpack(descs, buf, dst_flat)
        got += buf.numel() * buf.element_size()
    return got
