"""``RoutingTable``: who sends which parameter shard to whom when trainer weights are pushed to a
sampler fleet with a different parallel layout.

Inputs are per-rank lists of ``ParameterMetadata`` (name, shard shape, full shape, split dim, split
index) for the trainer ("actor") and for the sampler. For every parameter name the shards of each side
are ordered by ``split_idx``; tensor-parallel sizes must be integer multiples of each other:

  equal          actor shard i           -> sampler shard i
  actor smaller  actor shard i           -> sampler shards [i*r, (i+1)*r)      (r = sampler_tp / actor_tp)
  actor larger   actor shards [j*r, ..)  -> sampler shard j                    (each fills its slice)

A shard held by several actor ranks (data-parallel replicas) is sent by exactly ONE of them per
destination, chosen greedily by (transfers already on this actor->sampler pair, total transfers of the
actor). Every (sampler rank, sampler shard, actor split) is covered exactly once, which
``_verify_routing_completeness`` re-checks. Reference: axon/utils/p2p/routing_table.py:20-667.
"""
from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass, field
from typing import Any

import torch


@dataclass
class ParameterMetadata:
    param_name: str
    original_param_name: str
    param_shape: tuple
    full_param_shape: tuple
    param_dtype: torch.dtype
    split_dim: int = -1          # -1: replicated
    split_idx: int = 0
    expert_idx: int = -1
    metadata: dict = field(default_factory=dict)

    def __hash__(self):
        return hash((self.param_name, self.split_idx))

    @property
    def numel(self) -> int:
        n = 1
        for s in self.param_shape:
            n *= s
        return n


@dataclass
class FusedParameterMetadata:
    """A sampler-side fused tensor (qkv_proj, gate_up_proj, w13) and the logical parameters inside it."""
    param_name: str
    param_shape: tuple
    param_dtype: torch.dtype
    full_param_shape: tuple
    split_dim: int = -1
    split_idx: int = 0
    params: list = field(default_factory=list)

    def __hash__(self):
        return hash((self.param_name, self.split_idx))


@dataclass
class RankMapping:
    rank: int
    params: list = field(default_factory=list)


class RoutingTable:
    def __init__(self, actor_rank_mapping: list[RankMapping], sampler_rank_mapping: list[RankMapping], verbose: bool = False):
        self.actor_rank_mapping = [x for x in actor_rank_mapping if x.params]
        self.sampler_rank_mapping = [x for x in sampler_rank_mapping if x.params]
        self.verbose = verbose
        self.actor_param_to_rank = self._build_param_to_rank_map(self.actor_rank_mapping)
        self.sampler_param_to_rank = self._build_param_to_rank_map(self.sampler_rank_mapping)
        self.routing_map = self._build_routing_map()

    @staticmethod
    def _build_param_to_rank_map(mappings: list[RankMapping]) -> dict:
        out = defaultdict(list)
        for rm in mappings:
            for meta in rm.params:
                out[(meta.param_name, meta.split_idx)].append((rm.rank, meta))
        return dict(out)

    def _build_routing_map(self) -> dict:
        a_names = {k[0] for k in self.actor_param_to_rank}
        s_names = {k[0] for k in self.sampler_param_to_rank}
        if a_names != s_names:
            lines = [f"Parameter name mismatch! Actor: {len(a_names)}, Sampler: {len(s_names)}, Common: {len(a_names & s_names)}"]
            for label, names in (("Actor-only", a_names - s_names), ("Sampler-only", s_names - a_names)):
                if names:
                    lines.append(f"  {label} ({len(names)}):")
                    lines += [f"    - {n}" for n in sorted(names)[:10]]
                    if len(names) > 10:
                        lines.append(f"    ... and {len(names) - 10} more")
            raise ValueError("\n".join(lines))
        if not a_names:
            raise ValueError("No common parameters found between actor and sampler workers!")
        a_by_name, s_by_name = defaultdict(list), defaultdict(list)
        for name, idx in self.actor_param_to_rank:
            a_by_name[name].append(idx)
        for name, idx in self.sampler_param_to_rank:
            s_by_name[name].append(idx)
        routing = defaultdict(list)
        pair_load, actor_load = defaultdict(int), defaultdict(int)
        done = set()
        for name in sorted(a_names):
            a_idx, s_idx = sorted(a_by_name[name]), sorted(s_by_name[name])
            na, ns = len(a_idx), len(s_idx)
            if max(na, ns) % min(na, ns) != 0:
                raise ValueError(f"'{name}': shard counts {na} (actor) and {ns} (sampler) are not multiples of each other")
            for pos, ai in enumerate(a_idx):
                if na == ns:
                    targets = [s_idx[pos]]
                elif na < ns:
                    r = ns // na
                    targets = s_idx[pos * r:(pos + 1) * r]
                else:
                    targets = [s_idx[pos // (na // ns)]]
                holders = sorted(self.actor_param_to_rank[(name, ai)], key=lambda x: x[0])
                receivers = sorted((rk for t in targets for rk in self.sampler_param_to_rank[(name, t)]), key=lambda x: x[0])
                for s_rank, s_meta in receivers:
                    key = (s_rank, s_meta.param_name, s_meta.split_idx, ai)
                    if key in done:
                        continue
                    a_rank, a_meta = min(holders, key=lambda h: (pair_load[(h[0], s_rank)], actor_load[h[0]], h[0]))
                    routing[(a_rank, s_rank)].append({"actor": a_meta, "sampler": s_meta})
                    done.add(key)
                    pair_load[(a_rank, s_rank)] += 1
                    actor_load[a_rank] += 1
        self._verify_routing_completeness(routing)
        return dict(routing)

    def _verify_routing_completeness(self, routing) -> None:
        """Every sampler (rank, shard) must be fully covered: the element counts of the actor slices
        routed to it add up to the shard's size (several actor shards may fill one sampler shard)."""
        got = defaultdict(int)
        for (_, s_rank), items in routing.items():
            for it in items:
                a, s = it["actor"], it["sampler"]
                got[(s_rank, s.param_name, s.split_idx)] += min(a.numel, s.numel)
        missing = []
        for (name, idx), holders in self.sampler_param_to_rank.items():
            for s_rank, meta in holders:
                if got.get((s_rank, name, idx), 0) != meta.numel:
                    missing.append((s_rank, name, idx, got.get((s_rank, name, idx), 0), meta.numel))
        if missing:
            head = "; ".join(f"rank {r} {n}[{i}] got {g}/{w}" for r, n, i, g, w in missing[:5])
            raise ValueError(f"incomplete routing for {len(missing)} sampler shards: {head}")

    def get_transfers_for_actor_rank(self, rank: int) -> dict:
        return {s: items for (a, s), items in self.routing_map.items() if a == rank}

    def get_transfers_for_sampler_rank(self, rank: int) -> dict:
        return {a: items for (a, s), items in self.routing_map.items() if s == rank}

    def get_load_statistics(self) -> dict[str, Any]:
        sent, recv = defaultdict(int), defaultdict(int)
        for (a, s), items in self.routing_map.items():
            for it in items:
                nbytes = min(it["actor"].numel, it["sampler"].numel) * it["actor"].param_dtype.itemsize
                sent[a] += nbytes
                recv[s] += nbytes
        tot = sum(sent.values())
        return {"bytes_sent_per_actor": dict(sent), "bytes_recv_per_sampler": dict(recv), "total_bytes": tot,
                "max_actor_bytes": max(sent.values(), default=0), "min_actor_bytes": min(sent.values(), default=0),
                "num_pairs": len(self.routing_map)}

    def print_routing_table(self, max_items: int = 5) -> str:
        lines = ["RoutingTable:"]
        for (a, s), items in sorted(self.routing_map.items()):
            lines.append(f"  actor {a} -> sampler {s}: {len(items)} transfers")
            for it in items[:max_items]:
                lines.append(f"    {it['actor'].param_name}[{it['actor'].split_idx}] {tuple(it['actor'].param_shape)} -> "
                             f"[{it['sampler'].split_idx}] {tuple(it['sampler'].param_shape)}")
        text = "\n".join(lines)
        if self.verbose:
            print(text)
        return text
