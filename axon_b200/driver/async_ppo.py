"""Asynchronous PPO driver for disaggregated trainer / sampler pools
(reference: axon/driver/async_ppo.py:50-399).

A producer thread keeps the samplers busy: it queues a batch of tasks, runs the programs inside the
sampler worker, computes advantages there and ships the per-rank shards to the trainer ranks (bridge
process group, ``sampler_channel=nccl``) or hands the batch to the driver (``ray``: host objects).
A bounded queue (two entries) caps how far sampling may run ahead of training — the staleness bound.
The consumer (main thread) trains on each delivered batch, pauses the servers with the configured
strategy, pushes the new weights over the P2P path and lets generation continue; requests that were
in flight keep the tokens they already produced under the old policy (partial rollout).
"""
from __future__ import annotations

import queue
import threading
import time
import uuid

import numpy as np

from ..protocol import DataProto
from ..utils.metrics import aggregate_trainer_sampler_metrics, marked_timer, reduce_data_metrics, reduce_timing_metrics
from .base import PPODriverBase, cfg_get
from .driver_utils import ValidationResult, convert_batch_dict_to_dataproto


class AsyncPPO(PPODriverBase):
    QUEUE_DEPTH = 2

    def _retry_add_batch(self, batch: DataProto, step: int, max_retries: int = 600, delay: float = 0.5) -> None:
        for _ in range(max_retries):
            if self.sampler_wg.add_batch_to_engine(batch, step):
                return
            time.sleep(delay)
        raise RuntimeError(f"sampler refused the batch of step {step} {max_retries} times (queue full)")

    def _init_mode(self) -> None:
        cfg = self.config
        for bad, why in ((self.use_critic, "a critic"), (self.use_ref, "a reference policy"), (bool(cfg_get(cfg, "kl_reward")), "kl_reward")):
            if bad:
                raise ValueError(f"the asynchronous driver does not support {why}")
        if hasattr(self.train_sampler, "update") and str(cfg_get(cfg, "data_sampler", "")).endswith("curriculum"):
            raise ValueError("curriculum samplers need the synchronous driver (feedback would arrive steps late)")
        if self.hybrid_engine:
            raise ValueError("the asynchronous driver needs disaggregated pools (hybrid_engine=false)")
        self.channel = str(cfg_get(cfg, "sampler_channel", "nccl"))
        sp = int(cfg_get(cfg, "actor.fsdp.ulysses_sequence_parallel_size", 1))
        if str(cfg_get(cfg, "strategy", "fsdp")) == "megatron":
            # ranks of one tensor- / pipeline- / context-parallel block work on the same rows (expert-parallel ranks do not)
            sp = 1
            for key in ("tensor_model_parallel_size", "pipeline_model_parallel_size", "context_parallel_size"):
                sp *= int(cfg_get(cfg, f"actor.megatron.{key}", 1) or 1)
        self.dp_rank_mapping = [r // sp for r in range(self.actor_wg.world_size)]
        plain = cfg.to_dict() if hasattr(cfg, "to_dict") else dict(cfg)
        addrs = self.server_addresses or [None] * self.sampler_wg.world_size
        self.sampler_wg.initialize_sampler(addrs, plain, self.actor_wg.world_size)
        self._sampler_lock = threading.Lock()         # serialises producer-side and consumer-side sampler RPC groups
        self._weights_lock = threading.Lock()

    # ------------------------------------------------------------------ main loop
    def _run_training_loop(self) -> None:
        q: queue.Queue = queue.Queue(maxsize=self.QUEUE_DEPTH)
        stop = threading.Event()
        first, last = self.global_steps, self.total_training_steps
        temp_default = float(cfg_get(self.config, "decoding.temperature", 1.0) or 1.0)

        def producer():
            try:
                for step in range(first, last + 1):
                    if stop.is_set():
                        return
                    timing: dict = {}
                    t0 = time.time()
                    batch = self._prepare_batch(self.train_dataloader.next(self.train_batch_size), step)
                    self._retry_add_batch(batch, step)
                    metrics = dict(self.sampler_wg.generate_programs(step) or {})
                    if metrics.pop("skip", False):
                        q.put(("skip", step, metrics, timing))
                        continue
                    metrics.update(self.sampler_wg.compute_advantage_on_replay_buffer())
                    uid = str(uuid.uuid4())
                    if self.channel == "nccl":
                        with self._weights_lock:                 # the bridge group carries one exchange at a time
                            self._nonblocking(self.actor_wg, "receive_batch_from_sampler", uid)
                            self.sampler_wg.send_batch_to_actor(self.dp_rank_mapping, uid)
                            self._join_nonblocking()
                        payload = uid
                    else:
                        payload = self.sampler_wg.get_replay_buffer()
                    timing["gen"] = time.time() - t0
                    temp = (batch.meta_info.get("sample_params", {}) or {}).get("temperature", temp_default)
                    q.put(("batch", step, metrics, timing, payload, temp))
                q.put(None)
            except BaseException as e:       # noqa: BLE001
                q.put(e)

        th = threading.Thread(target=producer, daemon=True, name="async-producer")
        th.start()
        try:
            while True:
                item = q.get()
                if item is None:
                    break
                if isinstance(item, BaseException):
                    raise item
                if item[0] == "skip":
                    _, step, metrics, timing = item
                    metrics["batch/skipped"] = 1
                    self._post_step(metrics, timing)
                    continue
                _, step, metrics, timing, payload, temp = item
                metrics["async/staleness_steps"] = step - self.global_steps if step >= self.global_steps else 0
                metrics["async/queue_depth"] = q.qsize()
                with marked_timer("step", timing):
                    if self.channel == "nccl":
                        ok = all(self.actor_wg.set_batch_from_uid(payload))
                        assert ok, f"batch {payload} did not reach every trainer rank"
                    else:
                        self.actor_wg.set_batch(payload)
                    self._train_on_actor(metrics, timing, temp)
                    with marked_timer("sync_weights", timing), self._weights_lock:
                        self.sampler_wg.pause_all(str(cfg_get(self.config, "sampler_pausing_strategy", "continue")))
                        self._broadcast_weights()
                        self.sampler_wg.continue_all()
                    metrics.update(self.weight_sync_metrics())
                shards = self.actor_wg.get_batch_metrics_and_clear(timing)
                metrics.update(reduce_data_metrics([s["data"] for s in shards]))
                metrics.update(reduce_timing_metrics([s["timing"] for s in shards]))
                self._post_step(metrics, timing)
        finally:
            stop.set()

    def _train_on_actor(self, metrics: dict, timing: dict, temperature: float) -> None:
        cfg = self.config
        with marked_timer("old_log_prob", timing):
            if cfg_get(cfg, "use_sampler_logprobs", False):
                mm = self.actor_wg.use_sampler_log_probs(temperature)
            else:
                mm = self.actor_wg.compute_log_prob_on_batch(temperature)
        metrics.update(aggregate_trainer_sampler_metrics(mm if isinstance(mm, list) else [mm]))
        with marked_timer("forward_backward", timing):
            outs = self.actor_wg.train_on_batch(cfg_get(cfg, "loss", "ppo"), self._loss_args(), epochs=int(cfg_get(cfg, "ppo_epochs", 1)),
                                                mini_batch_size=int(cfg_get(cfg, "mini_batch_size", 0) or 0),
                                                mini_batch_shuffle=bool(cfg_get(cfg, "mini_batch_shuffle", False)),
                                                mini_batch_seed=cfg_get(cfg, "mini_batch_seed"))
        first = outs[0] if isinstance(outs, list) else outs
        metrics.update(first.meta_info["metrics"])

    # ------------------------------------------------------------------ validation
    def _validation_step(self) -> dict:
        if self.val_dataloader is None:
            return {}
        n = int(cfg_get(self.config, "validation.decoding.n", 1) or 1)
        vdec = cfg_get(self.config, "validation.decoding", {}) or {}
        vdec = vdec.to_dict() if hasattr(vdec, "to_dict") else dict(vdec)
        res = ValidationResult(n_samples=n)
        it = iter(self.val_dataloader)
        while True:
            try:
                bd = it.next(len(self.val_dataset))
            except StopIteration:
                break
            vb = convert_batch_dict_to_dataproto(bd, self.global_steps, val=True, val_n_samples=n)
            vb.meta_info["sample_params"] = {k: v for k, v in vdec.items() if k != "n"}
            self._retry_add_batch(vb, self.global_steps)
            for r in self.sampler_wg.evaluate_programs(self.global_steps):
                res.add(r["reward"], r["group_id"], r.get("data_source", "unknown"))
        return res.compute_metrics()
