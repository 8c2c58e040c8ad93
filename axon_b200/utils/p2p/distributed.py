"""Process group that spans the trainer ranks and the sampler ranks (the "bridge"), independent of
each side's own default group (reference: axon/utils/p2p/distributed.py:30-104).

Ranks rendezvous through a dedicated TCP store at ``master_addr:master_port``; trainer rank r becomes
bridge rank r, sampler rank s becomes ``n_trainers + s``. The group is created with the c10d helper
behind ``new_group`` but against its own store, so neither side needs to know the other's default
group.
"""
from __future__ import annotations

import datetime

import torch
import torch.distributed as dist
from torch.distributed.distributed_c10d import Backend, PrefixStore, _new_process_group_helper, _world


def init_trainer_sampler_process_group(master_addr: str, master_port: int, rank: int, world_size: int,
                                       backend: str | None = None, group_name: str = "trainer_sampler_bridge",
                                       timeout_s: float = 600.0):
    assert 0 <= rank < world_size
    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    timeout = datetime.timedelta(seconds=timeout_s)
    store = dist.TCPStore(master_addr, int(master_port), world_size, is_master=(rank == 0), timeout=timeout,
                          wait_for_workers=False)
    store = PrefixStore(group_name, store)
    kwargs = {}
    if backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
    pg, _ = _new_process_group_helper(world_size, rank, [], Backend(backend), store, group_name=group_name,
                                      timeout=timeout, **kwargs)
    _world.pg_group_ranks[pg] = {i: i for i in range(world_size)}
    return pg
