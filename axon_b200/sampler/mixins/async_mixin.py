"""Worker-resident rollout pipeline for the asynchronous driver
(reference: axon/sampler/mixins/async_mixin.py:60-438).

The rank-0 sampler worker hosts the Engine, the program runner and the replay buffer, so a step's
data never has to pass through the driver process: programs run next to the servers, advantages are
computed where the batch is, and the per-rank shards go straight to the trainer ranks over the
bridge process group as (size, pickled bytes) pairs.
"""
from __future__ import annotations

import asyncio
import io
import os
import pickle

import numpy as np
import torch
import torch.distributed as dist

from ...controller.decorator import Dispatch, Execute, register
from ...protocol import DataProto


def encode_object(obj, device) -> torch.Tensor:
    buf = io.BytesIO()
    pickle.dump(obj, buf, protocol=pickle.HIGHEST_PROTOCOL)
    return torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8).to(device)


def decode_object(t: torch.Tensor):
    return pickle.loads(t.cpu().numpy().tobytes())


class AsyncSamplerMixin:
    replay_buffer: DataProto | None = None

    @register(dispatch_mode=Dispatch.ONE_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def initialize_sampler(self, server_addresses: list, config, actor_world_size: int):
        from ...driver.components.program_component import create_program_components
        from ...utils.tokenizer import hf_tokenizer
        self.full_config = config
        self.actor_world_size = int(actor_world_size)
        self.tokenizer = hf_tokenizer(config.get("model_path"))
        # this worker's own server is used in-process; the others are reached over HTTP
        servers = [self.server if (a is None or a == self.address) else a for a in server_addresses]
        comps = create_program_components(config, self.tokenizer, None, [], servers, hybrid_engine=False,
                                          thread_name_prefix="SamplerPipeline")
        self.sampling_client, self.rollout_engine = comps.sampling_client, comps.engine
        self.program_processor, self.program_runner, self._tasks_loop = comps.program_processor, comps.program_runner, comps.tasks_loop
        out = config.get("output_dir", "outputs")
        self.experiment_dir = os.path.join(os.path.abspath(out), str(config.get("project_name", "axon")),
                                           str(config.get("experiment_name", "run")), "samplers")
        os.makedirs(self.experiment_dir, exist_ok=True)
        self.replay_buffer = None
        self._uid_to_index = {}
        return True

    @register(dispatch_mode=Dispatch.ONE_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def pause_all(self, strategy: str = "drain"):
        asyncio.run(self.sampling_client.pause_all(strategy))

    @register(dispatch_mode=Dispatch.ONE_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def continue_all(self):
        asyncio.run(self.sampling_client.continue_all())

    @register(dispatch_mode=Dispatch.ONE_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def add_batch_to_engine(self, batch: DataProto, global_steps: int) -> bool:
        """False when the sampler already has too many requests in flight (caller retries)."""
        limit = self.full_config.get("max_sampler_queue_size", None) or 10 ** 9
        if sum(self.sampling_client.load_statistics()["inflight"]) >= limit:
            return False
        _, self._uid_to_index = self.program_runner.create_programs(batch, global_steps)
        self.original_batch = batch
        return True

    @register(dispatch_mode=Dispatch.ONE_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def generate_programs(self, global_steps: int = -1) -> dict:
        cfg = self.full_config
        if cfg.get("use_dummy_batch", False):
            self.replay_buffer = self.program_processor.create_dummy_batch(self.original_batch, global_steps=global_steps)
            return {}
        finished, engine_metrics = asyncio.run(self.program_runner.run_and_collect())
        strict = bool(cfg.get("filter_program_errors", False))
        programs = [p for p in finished if p.is_trainable(strict=strict) and p.training_steps]
        engine_metrics["engine/training_programs"] = len(programs)
        if not programs:
            self.replay_buffer = None
            return {"skip": True, **engine_metrics}
        batch, tm = self.program_processor.transform_programs(programs, self.experiment_dir, global_steps, self._uid_to_index)
        temp = (self.original_batch.meta_info.get("sample_params", {}) or {}).get("temperature")
        batch.meta_info["temperature"] = float(temp if temp is not None else cfg.get("decoding", {}).get("temperature", 1.0))
        self.replay_buffer = batch
        return {**engine_metrics, **tm, "skip": False}

    @register(dispatch_mode=Dispatch.ONE_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def evaluate_programs(self, global_steps: int = 0) -> list[dict]:
        finished, _ = asyncio.run(self.program_runner.run_and_collect(val=True))
        return [{"reward": (p.metadata or {}).get("raw_score", p.reward), "group_id": p.group_id,
                 "data_source": (p.metadata or {}).get("data_source", "unknown")} for p in finished]

    @register(dispatch_mode=Dispatch.ONE_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def compute_advantage_on_replay_buffer(self) -> dict:
        from ...driver.components.advantage_component import compute_advantage_component
        from ...driver.driver_utils import balance_batch, pad_dataproto_to_world_size
        cfg = self.full_config
        metrics: dict = {}
        adv_cfg = {"advantage": cfg.get("advantage", "grpo"), "advantage_args": dict(cfg.get("advantage_args", {}) or {}),
                   "drop_zero_advantage_samples": bool(cfg.get("drop_zero_advantage_samples", False))}
        meta = dict(self.replay_buffer.meta_info)
        rb = compute_advantage_component(self.replay_buffer, adv_cfg, metrics)
        rb = pad_dataproto_to_world_size(rb, [self.world_size, self.actor_world_size])
        rb = balance_batch(rb, world_size=self.actor_world_size, metrics=metrics)
        rb.meta_info.update(meta)
        self.replay_buffer = rb
        return metrics

    @register(dispatch_mode=Dispatch.ONE_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def get_replay_buffer(self) -> DataProto:
        assert self.replay_buffer is not None, "no replay buffer: generate_programs() has not produced one"
        return self.replay_buffer

    @register(dispatch_mode=Dispatch.ONE_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def send_batch_to_actor(self, dp_rank_mapping: list[int], batch_uid: str) -> int:
        """Two messages per trainer rank over the bridge group: byte count (int64), then the pickled
        shard (uint8). Trainer ranks of one data-parallel shard receive the same payload."""
        assert self.bridge_pg is not None, "bridge process group is not connected"
        dp_size = max(dp_rank_mapping) + 1
        shards = self.replay_buffer.chunk(dp_size)
        for sh in shards:
            sh.meta_info = dict(self.replay_buffer.meta_info)
        payloads = {dp: encode_object(sh, self.device) for dp, sh in enumerate(shards)}
        reqs, keep = [], []
        for actor_rank, dp in enumerate(dp_rank_mapping):
            size = torch.tensor([payloads[dp].numel()], dtype=torch.int64, device=self.device)
            keep.append(size)
            reqs.append(dist.isend(size, dst=actor_rank, group=self.bridge_pg))
        for r in reqs:
            r.wait()
        reqs = [dist.isend(payloads[dp], dst=actor_rank, group=self.bridge_pg) for actor_rank, dp in enumerate(dp_rank_mapping)]
        for r in reqs:
            r.wait()
        return sum(p.numel() for p in payloads.values())
