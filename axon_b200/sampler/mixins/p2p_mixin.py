"""Sampler side of the disaggregated weight push
(reference: axon/sampler/mixins/p2p_mixin.py:60-757).

The sampler publishes what each of its ranks needs (``get_parameter_mapping``: per fused parameter
the tensor-/expert-parallel shard this rank owns). With tensor parallel size 1 the shard layout equals
the engine's flat parameter buffer, so pushed bytes land directly in the live weights.

On CUDA within one node the sampler moves its parameters into an IPC-exportable allocation at connect
time and hands the handle to the trainers; a push is then the trainers' plan kernel storing into that
buffer, and this side only waits for the bridge all-reduce that follows the stores. Elsewhere it posts
one receive per sending trainer and unpacks the messages.
"""
from __future__ import annotations

import socket
import time

import numpy as np
import torch
import torch.distributed as dist

from ...controller.decorator import Dispatch, register
from ...utils.p2p.distributed import init_trainer_sampler_process_group
from ...utils.p2p.param_mapper import get_param_metadata
from ...utils.p2p.plan import compile_plan
from ...utils.p2p.transport import recv_plans


def _cfg(cfg, key, default=None):
    if isinstance(cfg, dict):
        return cfg.get(key, default)
    return getattr(cfg, key, default)


class SamplerP2PMixin:
    bridge_pg = None
    _recv_plans = None
    _recv_stage: dict | None = None
    _peer_path = False
    _ipc_buffer = None

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def connect_sampler_to_trainer(self, master_addr: str, master_port: int, world_size: int, rank_offset: int):
        from ...trainer.mixins.p2p_mixin import exchange_peer_info, peer_store_path_possible
        self._n_trainers = rank_offset
        self.bridge_pg = init_trainer_sampler_process_group(master_addr, master_port, rank_offset + self.rank, world_size,
                                                            backend="nccl" if self.device.type == "cuda" else "gloo")
        self._bridge_token = torch.zeros(1, device=self.device)
        dist.all_reduce(self._bridge_token, group=self.bridge_pg)
        mine = {"role": "sampler", "rank": self.rank, "host": socket.gethostname(), "cuda": self.device.type == "cuda",
                "tp": self.tp, "handle": None, "offsets": None}
        if self.device.type == "cuda" and self.tp == 1 and getattr(self, "pp", 1) == 1 and not getattr(self, "shares_trainer_weights", False):
            mine["handle"], mine["offsets"] = self._export_parameters()
        infos = exchange_peer_info(self.bridge_pg, mine)
        self._peer_path = peer_store_path_possible(infos)
        return self.bridge_pg.rank()

    def _export_parameters(self):
        """Move the live parameters into an allocation other processes can map; returns (handle, offsets)."""
        from ...parallel.ipc import IpcBuffer
        p = self.model.params
        if self._ipc_buffer is None:
            buf = IpcBuffer(p.flat.numel(), p.flat.dtype, self.device)
            buf.tensor.copy_(p.flat)
            torch.cuda.current_stream().synchronize()
            p.rebind(buf.tensor)
            self._ipc_buffer = buf
            if getattr(self, "engine", None) is not None:
                self.engine._graphs.clear()                  # captured decode graphs hold the old addresses
        return self._ipc_buffer.handle(), {n: o for n, (o, _) in p.offsets.items()}

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def get_parameter_mapping(self):
        tp_rank = self.rank % self.tp
        cfg = getattr(self.model, "full_cfg", self.model.cfg)       # a sharded model computes on its local configuration
        ep = self.tp if getattr(cfg, "num_experts", 0) > 0 else 1   # experts are divided whole over the group
        whole = ("model.embed_tokens.weight", "lm_head.weight") if self.tp > 1 else ()      # every rank of a group holds these in full
        mapping = get_param_metadata(cfg, rank=self.rank, tp=self.tp, tp_rank=tp_rank, ep=ep, ep_rank=tp_rank if ep > 1 else 0,
                                     dtype=self.model.params.dtype, replicated_names=whole)
        local_name = getattr(self.model, "local_name", None)
        if local_name is not None:                      # a pipeline stage: its own layers (under the full model's names) only
            mapping.params = [m for m in mapping.params if local_name(m.param_name) is not None]
        return mapping

    def _shard_offsets(self, metas) -> dict:
        local_name = getattr(self.model, "local_name", None)
        if local_name is not None:                      # full-model names -> where the stage keeps the tensor
            return {m.param_name: self.model.params.offsets[local_name(m.param_name)][0] for m in metas}
        if self.tp == 1:
            return {n: o for n, (o, _) in self.model.params.offsets.items()}
        off, table = 0, {}
        for m in metas:
            table[m.param_name] = off
            off += (m.numel + 127) // 128 * 128
        return table

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def receive_trainer_to_sampler_weights(self, routing_table=None):
        if routing_table is not None:
            self.routing_table = routing_table
            self._recv_plans = None
        assert getattr(self, "routing_table", None) is not None, "no routing table: the first push must carry it"
        t0 = time.monotonic()
        if getattr(self, "server", None) is not None:
            self.server.reset_prefix_cache()         # cached keys / values belong to the weights being replaced
        if self._peer_path:
            # the trainers' kernels store into this rank's live buffer; generation must not read it meanwhile
            with self.server._ctl_lock, torch.cuda.device(self.device):
                torch.cuda.current_stream().synchronize()
                dist.all_reduce(self._bridge_token, group=self.bridge_pg)     # completes after every trainer's stores
                torch.cuda.current_stream().synchronize()
            return {"bytes": self.model.params.numel * self.model.params.flat.element_size(), "seconds": time.monotonic() - t0,
                    "transport": "peer-store kernel"}
        if self._recv_plans is None:
            mine = next(m for m in self.routing_table.sampler_rank_mapping if m.rank == self.rank).params
            my_off = self._shard_offsets(mine)
            # bridge rank of trainer rank a is a (trainers come first in the bridge group)
            self._recv_plans = {a_rank: _pair_descs(self.routing_table, a_rank, self.rank, my_off)
                                for a_rank in sorted(self.routing_table.get_transfers_for_sampler_rank(self.rank))}
            self._recv_stage = {}
        with self.server._ctl_lock:
            got = recv_plans(self._recv_plans, self.model.params.flat, self.bridge_pg, self._recv_stage)
        if _cfg(self.scfg, "offload_p2p_buffer", False):
            self._recv_stage = {}
        return {"bytes": got, "seconds": time.monotonic() - t0, "transport": "messages"}

    @staticmethod
    def _print_p2p_mismatch(actor_map, sampler_map) -> str:
        a = {p.param_name: p.full_param_shape for m in actor_map for p in m.params}
        s = {p.param_name: p.full_param_shape for m in sampler_map for p in m.params}
        lines = [f"only on trainer: {n}" for n in sorted(set(a) - set(s))] + [f"only on sampler: {n}" for n in sorted(set(s) - set(a))]
        lines += [f"shape differs: {n}: {a[n]} vs {s[n]}" for n in sorted(set(a) & set(s)) if tuple(a[n]) != tuple(s[n])]
        return "\n".join(lines)


class _Zero(dict):
    """Offset table that answers 0 for every name (for the side of a plan whose offsets are unused)."""

    def __getitem__(self, k):
        return 0


def _pair_descs(table, a_rank: int, s_rank: int, s_off: dict) -> np.ndarray:
    """Descriptors of the (a_rank -> s_rank) pair in the order the sender packs them; destination
    offsets are this rank's, source offsets are irrelevant on the receiving side."""
    dsts = {s for (a, s) in table.routing_map if a == a_rank}
    plan = compile_plan(table, a_rank, _Zero(), {r: (s_off if r == s_rank else _Zero()) for r in dsts})
    return plan.descs[plan.descs["dst_rank"] == s_rank]


FSDPSamplerP2PMixin = SamplerP2PMixin
MegatronSamplerP2PMixin = SamplerP2PMixin
