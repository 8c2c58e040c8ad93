"""Trainer side of the disaggregated weight push
(reference: axon/trainer/mixins/p2p_mixin.py:58-703).

``get_parameter_mapping`` describes what this rank holds: the full fused parameters on a data-parallel
trainer (any rank can serve any sampler shard and the routing table spreads the load), this rank's
slices on a tensor- or expert-parallel one.

``send_trainer_to_sampler_weights`` compiles the routing table into a copy plan once (cached across
steps) and executes it. Two transports:

* **peer stores** (CUDA, all ranks on one node): at connect time every sampler process exports its live
  parameter buffer as a CUDA IPC handle and every trainer process maps it. A push is then ONE launch of the
  plan kernel (``csrc/comm.cu``: ``p2p_copy_plan_kernel``) that re-slices this rank's shards and stores
  them straight into the samplers' weights over NVLink - no packing, no staging buffer, no send / receive
  pair - followed by one tiny all-reduce on the bridge group that tells the samplers the stores are done.
* **messages** (CPU ranks, gloo, ranks on different nodes): one packed message per destination over the
  bridge process group, unpacked by the receiver.
"""
from __future__ import annotations

import socket
import time

import torch
import torch.distributed as dist

from ...controller.decorator import Dispatch, register
from ...utils.p2p.distributed import init_trainer_sampler_process_group
from ...utils.p2p.param_mapper import get_param_metadata
from ...utils.p2p.plan import compile_plan, execute_plan
from ...utils.p2p.transport import send_plan


def slice_for_tp(t: torch.Tensor, dim: int, tp_rank: int, tp_size: int) -> torch.Tensor:
    """The ``tp_rank``-th of ``tp_size`` equal slices along ``dim`` (``dim`` < 0: replicated)."""
    if dim < 0 or tp_size == 1:
        return t
    n = t.shape[dim] // tp_size
    return t.narrow(dim, tp_rank * n, n)


def exchange_peer_info(bridge_pg, mine: dict) -> list[dict]:
    """Every bridge rank learns every other rank's role, host and (for samplers) the IPC handle and layout of
    its parameter buffer. Called by both mixins at connect time."""
    out = [None] * dist.get_world_size(group=bridge_pg)
    dist.all_gather_object(out, mine, group=bridge_pg)
    return out


def peer_store_path_possible(infos: list[dict]) -> bool:
    """The one-launch path needs every rank on CUDA, on one host, and every sampler to have exported a buffer
    whose layout is the plain parameter layout (tensor-parallel sampler shards take the message path)."""
    if not infos or any(i is None for i in infos):
        return False
    if len({i["host"] for i in infos}) != 1 or not all(i["cuda"] for i in infos):
        return False
    return all(i["role"] != "sampler" or (i.get("handle") is not None and i.get("tp", 1) == 1) for i in infos)


class TrainerP2PMixin:
    bridge_pg = None
    _p2p_plan = None
    _p2p_stage: dict | None = None
    _bridge_offset = 0
    _peer_infos: list | None = None
    _peer_ptrs: list | None = None
    _peer_path = False

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def connect_trainer_to_sampler(self, master_addr: str, master_port: int, world_size: int, rank_offset: int = 0):
        self._bridge_world = world_size
        self._n_trainers = self.world_size
        self.bridge_pg = init_trainer_sampler_process_group(master_addr, master_port, rank_offset + self.rank, world_size,
                                                            backend="nccl" if self.device.type == "cuda" else "gloo")
        self._bridge_token = torch.zeros(1, device=self.device)
        dist.all_reduce(self._bridge_token, group=self.bridge_pg)          # warm-up: connections exist before the first push
        infos = exchange_peer_info(self.bridge_pg, {"role": "trainer", "rank": self.rank, "host": socket.gethostname(),
                                                    "cuda": self.device.type == "cuda"})
        self._peer_infos = infos
        self._peer_path = peer_store_path_possible(infos)
        if self._peer_path:
            from ...parallel.ipc import open_handle
            samplers = sorted((i for i in infos if i["role"] == "sampler"), key=lambda i: i["rank"])
            self._peer_ptrs = [open_handle(i["handle"], self.device) for i in samplers]
            self._peer_offsets = {i["rank"]: i["offsets"] for i in samplers}
        return self.bridge_pg.rank()

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def get_parameter_mapping(self):
        # a tensor- or expert-parallel trainer describes its own slices; the routing table then matches
        # them against the sampler's slices box by box
        inner = getattr(self.model, "inner", self.model)
        tp, ep = getattr(self.model, "tp", None), getattr(self.model, "ep", None) or getattr(inner, "ep", None)
        if getattr(inner, "etp_world", 1) > 1:
            raise NotImplementedError("the trainer -> sampler push does not describe experts that are cut over the tensor-parallel "
                                      "group (expert_tensor_parallel_size > 1); use the colocated deployment, which gathers whole tensors")
        rep = ()
        if tp is not None and tp.world > 1:
            from ...utils.p2p.param_mapper import split_kind
            rep = [n for n in inner.replicated_names() if split_kind(n) != "replicated"]
        mapping = get_param_metadata(self.model.cfg, rank=self.rank, dtype=self.model.params.dtype,
                                     tp=tp.world if tp is not None else 1, tp_rank=tp.rank if tp is not None else 0,
                                     ep=ep.world if ep is not None else 1, ep_rank=ep.rank if ep is not None else 0,
                                     replicated_names=rep)
        held = self.model.params.layout                 # a pipeline stage holds (and sends) its own layers only
        mapping.params = [m for m in mapping.params if m.param_name in held]
        return mapping

    def _local_offsets(self) -> dict:
        return {n: o for n, (o, _) in self.model.params.offsets.items()}

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def send_trainer_to_sampler_weights(self, routing_table=None):
        if routing_table is not None:
            self.routing_table = routing_table
            self._p2p_plan = None
        assert getattr(self, "routing_table", None) is not None, "no routing table: the first push must carry it"
        t0 = time.monotonic()
        dsts = {s for (a, s) in self.routing_table.routing_map if a == self.rank}
        if self._peer_path:
            if self._p2p_plan is None:
                self._p2p_plan = compile_plan(self.routing_table, self.rank, self._local_offsets(),
                                              {s: self._peer_offsets[s] for s in dsts},
                                              elem_bytes=self.model.params.flat.element_size())
            with torch.cuda.device(self.device):
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
                execute_plan(self._p2p_plan, self.model.params.flat, [None] * len(self._peer_ptrs), dst_ptrs=self._peer_ptrs)
                ev1.record()
                # stream-ordered after the stores: when this completes on a sampler, every trainer's kernel has finished
                dist.all_reduce(self._bridge_token, group=self.bridge_pg)
                torch.cuda.current_stream().synchronize()
            return {"bytes": self._p2p_plan.total_bytes, "seconds": time.monotonic() - t0, "transport": "peer-store kernel",
                    "kernel_ms": ev0.elapsed_time(ev1)}
        if self._p2p_plan is None:
            from ...sampler.mixins.p2p_mixin import _Zero
            # message path: only source offsets matter to the sender (the receiver owns its layout)
            self._p2p_plan = compile_plan(self.routing_table, self.rank, self._local_offsets(), {s: _Zero() for s in dsts},
                                          elem_bytes=self.model.params.flat.element_size())
            self._p2p_stage = {}
        sent = send_plan(self._p2p_plan, self.model.params.flat, self.bridge_pg, self._n_trainers, self._p2p_stage)
        if getattr(self, "offload_p2p_buffer", False):
            self._p2p_stage = {}
        return {"bytes": sent, "seconds": time.monotonic() - t0, "transport": "messages"}


FSDPTrainerP2PMixin = TrainerP2PMixin
MegatronTrainerP2PMixin = TrainerP2PMixin
