"""Base class of every distributed worker (trainer, sampler, critic ...): rank bookkeeping from the
environment and the per-mesh dispatch/collect tables that the controller queries
(reference: axon/core/worker.py:30-232)."""
from __future__ import annotations

import os
import socket

from ..controller.decorator import Dispatch, Execute, register


class Worker:
    ENV_KEYS = ("WORLD_SIZE", "RANK", "LOCAL_WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT",
                "CUDA_VISIBLE_DEVICES")

    def __init__(self, *args, **kwargs):
        self._rank = int(os.environ.get("RANK", "0"))
        self._world_size = int(os.environ.get("WORLD_SIZE", "1"))
        self._local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self._master_addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        self._master_port = os.environ.get("MASTER_PORT", "29500")
        self._dispatch_info: dict[str, int] = {}
        self._collect_info: dict[str, bool] = {}

    @property
    def rank(self) -> int:
        return self._rank

    @property
    def world_size(self) -> int:
        return self._world_size

    @property
    def local_rank(self) -> int:
        return self._local_rank

    def get_master_addr_port(self):
        return self._master_addr, self._master_port

    @staticmethod
    def get_availale_master_addr_port():
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            return "127.0.0.1", str(s.getsockname()[1])

    def _register_dispatch_collect_info(self, mesh_name: str, dp_rank: int, is_collect: bool) -> None:
        """Declare, for one device mesh, which data-parallel shard this worker consumes and whether its
        output is the one to collect (e.g. only TP rank 0 / last PP stage)."""
        if mesh_name in self._dispatch_info:
            raise ValueError(f"mesh '{mesh_name}' is already registered on rank {self._rank}")
        self._dispatch_info[mesh_name] = int(dp_rank)
        self._collect_info[mesh_name] = bool(is_collect)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def _query_dispatch_info(self, mesh_name: str) -> int:
        assert mesh_name in self._dispatch_info, f"mesh '{mesh_name}' not registered on rank {self._rank}"
        return self._dispatch_info[mesh_name]

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def _query_collect_info(self, mesh_name: str) -> bool:
        assert mesh_name in self._collect_info, f"mesh '{mesh_name}' not registered on rank {self._rank}"
        return self._collect_info[mesh_name]

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def ping(self) -> int:
        return self._rank

    @register(dispatch_mode=Dispatch.ONE_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def execute_func_rank_zero(self, func, *args, **kwargs):
        return func(*args, **kwargs)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def execute_with_func_generator(self, func, *args, **kwargs):
        return func(self, *args, **kwargs)
