"""Dispatch decorator, worker groups (inline and spawned processes), fused roles, failure detection."""
import os
import threading
import time

import numpy as np
import pytest
import torch

from axon_b200.controller.decorator import Dispatch, Execute, make_nd_compute_dataproto_dispatch_fn, register
from axon_b200.controller.worker_group import (ClassWithInitArgs, LocalWorkerGroup, RPCTimeoutError, WorkerDiedError,
                                               init_worker_group)
from axon_b200.core.resource_pool import ResourcePool, split_trainer_sampler_pools
from axon_b200.core.role import Role
from axon_b200.core.worker import Worker
from axon_b200.protocol import DataProto


class ToyWorker(Worker):
    def __init__(self, scale=1.0, tp=1):
        super().__init__()
        self.scale = scale
        # mesh "trainer": dp index = rank // tp; only tp-rank 0 returns results
        self._register_dispatch_collect_info("trainer", self.rank // tp, self.rank % tp == 0)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def whoami(self):
        return (self.rank, self.world_size, os.environ.get("RANK"))

    @register(dispatch_mode=Dispatch.DP_COMPUTE_PROTO_WITH_FUNC)
    def double(self, data: DataProto):
        return DataProto.from_dict({"y": data.batch["x"] * 2 * self.scale + self.rank * 1000})

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("trainer"))
    def mesh_op(self, data: DataProto):
        return DataProto.from_dict({"y": data.batch["x"] + self.rank * 1000}, meta_info={"metrics": {"r": self.rank}})

    @register(dispatch_mode=Dispatch.ONE_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def only_zero(self, v):
        return v + self.rank

    @register(dispatch_mode=Dispatch.ONE_TO_ALL, blocking=False)
    def slow(self, secs):
        time.sleep(secs)
        return self.rank

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def boom(self):
        raise ValueError("kaboom")

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def die(self):
        os._exit(3)

    @register(dispatch_mode=Dispatch.DIRECT_SAMPLER_METHOD)
    def direct(self):
        return "direct"


def data(n=8):
    return DataProto.from_dict({"x": torch.arange(n).float()})


@pytest.mark.parametrize("backend", ["inline", "process"])
def test_dispatch_modes(backend):
    wg = LocalWorkerGroup(ResourcePool([4]), ClassWithInitArgs(ToyWorker, scale=1.0, tp=2), backend=backend)
    try:
        who = wg.whoami()
        assert [w[0] for w in who] == [0, 1, 2, 3] and all(w[1] == 4 for w in who)
        if backend == "process":
            assert [w[2] for w in who] == ["0", "1", "2", "3"]
        out = wg.double(data())
        assert out.batch["y"].tolist() == [0, 2, 1004, 1006, 2008, 2010, 3012, 3014]
        m = wg.mesh_op(data())           # dp=2 (tp=2): collected from ranks 0 and 2 only
        assert m.batch["y"].tolist() == [0, 1, 2, 3, 2004, 2005, 2006, 2007]
        assert m.meta_info["metrics"] == {"r": [0, 2]}
        assert wg.only_zero(5) == 5
        futs = wg.slow(0.05)
        got = [f.result(5) if hasattr(f, "result") else f for f in futs]
        assert got == [0, 1, 2, 3]
        with pytest.raises((RuntimeError, ValueError)):
            wg.boom()
        assert not hasattr(wg, "nonexistent")
        with pytest.raises(NotImplementedError):
            wg.direct()
    finally:
        wg.shutdown()


def test_dead_worker_is_detected_and_rpc_times_out():
    wg = LocalWorkerGroup(world_size=2, cls_with_init=ClassWithInitArgs(ToyWorker), backend="process", rpc_timeout=1.0)
    try:
        with pytest.raises(RPCTimeoutError):
            [f.result(10) for f in wg.slow(3.0)]
    finally:
        wg.shutdown()
    wg = LocalWorkerGroup(world_size=2, cls_with_init=ClassWithInitArgs(ToyWorker), backend="process", rpc_timeout=20.0)
    dead = []
    hit = threading.Event()
    wg.start_worker_aliveness_check(0.1, on_failure=lambda r: (dead.append(r), hit.set()))
    try:
        with pytest.raises(WorkerDiedError):
            wg.execute_all_sync("die")
        assert hit.wait(5) and dead and dead[0] in (0, 1)
    finally:
        wg.shutdown()


class ToySampler(Worker):
    def __init__(self):
        super().__init__()
        self._register_dispatch_collect_info("sampler", self.rank, True)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def peer_scale(self):
        return self._fused_peers["actor"].scale      # colocated roles share the process

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("sampler"))
    def gen(self, data: DataProto):
        return DataProto.from_dict({"t": data.batch["x"] + 0.5})

    @register(dispatch_mode=Dispatch.DIRECT_SAMPLER_METHOD)
    def wake_up(self):
        return "awake"


def test_fused_worker_group_and_role_proxy():
    groups = init_worker_group({"actor": ClassWithInitArgs(ToyWorker, scale=3.0), "sampler": ClassWithInitArgs(ToySampler)},
                               ResourcePool([2]), backend="inline")
    actor, sampler = groups["actor"], groups["sampler"]
    assert actor.world_size == 2 and sampler.peer_scale() == [3.0, 3.0]
    assert sampler.gen(data(4)).batch["t"].tolist() == [0.5, 1.5, 2.5, 3.5]
    assert actor.mesh_op(data(4)).batch["y"].tolist() == [0, 1, 1002, 1003]
    fused_obj = actor.workers[0]
    assert fused_obj.wake_up() == "awake" and hasattr(fused_obj, "actor_double") and not hasattr(fused_obj, "sampler_wake_up")


def test_roles_and_pools():
    assert Role.from_string("actor") is Role.Actor and Role.from_string("ref") is Role.RefPolicy
    assert Role.Actor.is_trainable and not Role.Sampler.is_trainable
    p = ResourcePool([8, 8])
    assert p.world_size == 16 and p.local_rank_list()[8] == 0 and p.node_rank_list()[9] == 1
    pools = split_trainer_sampler_pools(1, 8, ratio=1, hybrid=False)
    assert pools["trainer"].world_size == 4 and pools["sampler"].world_size == 4 and pools["sampler"].device_offset == 4
    assert split_trainer_sampler_pools(2, 8, 1, hybrid=True)["global"].world_size == 16
    pools = split_trainer_sampler_pools(1, 8, ratio=3, hybrid=False)
    assert pools["trainer"].world_size == 2 and pools["sampler"].world_size == 6
