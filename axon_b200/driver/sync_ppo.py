"""Synchronous PPO driver (reference: axon/driver/sync_ppo.py:60-524).

One step: draw tasks -> run programs on the sampler -> flatten to a training batch -> (critic values,
reward model, KL-in-reward) -> advantages -> pad / balance over data-parallel ranks -> (critic
update, reference log-probs) -> old log-probs -> PPO mini-batch updates -> validation / checkpoint /
log. With ``enable_one_off_pipeline`` (disaggregated pools) a background thread prepares step N+1
while step N trains, bounded by a queue of depth 1, and weights reach the sampler by the P2P push
instead of the colocated mode switch.
"""
from __future__ import annotations

import asyncio
import queue
import threading
import time

import numpy as np
import torch

from ..protocol import DataProto
from ..utils.metrics import (aggregate_trainer_sampler_metrics, compute_data_metrics, compute_timing_metrics,
                             compute_trainer_sampler_mismatch_metrics, marked_timer)
from ..utils.rl.kl import apply_kl_penalty
from .base import PPODriverBase, cfg_get
from .components.advantage_component import compute_advantage_component
from .driver_utils import balance_batch, pad_dataproto_to_world_size, process_mini_batch, update_trainer


class SyncPPO(PPODriverBase):
    def _init_mode(self) -> None:
        cfg = self.config
        self.one_off = bool(cfg_get(cfg, "enable_one_off_pipeline", False))
        if self.one_off and self.hybrid_engine:
            raise ValueError("enable_one_off_pipeline needs disaggregated trainer / sampler pools (hybrid_engine=false)")
        if cfg_get(cfg, "kl_reward") and not self.use_ref:
            raise ValueError("kl_reward needs a reference-policy role")
        self.use_sampler_logprobs = bool(cfg_get(cfg, "use_sampler_logprobs", False))
        self._uid_to_index: dict = {}

    # ------------------------------------------------------------------ loops
    def _run_training_loop(self) -> None:
        (self._run_pipelined if self.one_off else self._run_sequential)()

    def _run_sequential(self) -> None:
        while self.global_steps <= self.total_training_steps:
            timing: dict[str, float] = {}
            metrics: dict = {}
            with marked_timer("step", timing):
                batch_dict = self.train_dataloader.next(self.train_batch_size)
                batch = self._sample_and_prepare(batch_dict, self.global_steps, metrics, timing)
                self._train_on_actor(batch, metrics, timing)
            self._finish_step(batch, metrics, timing)

    def _run_pipelined(self) -> None:
        """Producer thread samples step N+1 with the weights of step N-1 (one step stale at most: the
        queue holds a single prepared batch) while the main thread trains step N."""
        q: queue.Queue = queue.Queue(maxsize=1)
        stop = threading.Event()
        first, last = self.global_steps, self.total_training_steps

        def producer():
            try:
                for step in range(first, last + 1):
                    if stop.is_set():
                        return
                    metrics, timing = {}, {}
                    batch_dict = self.train_dataloader.next(self.train_batch_size)
                    batch = self._sample_and_prepare(batch_dict, step, metrics, timing)
                    q.put((batch, metrics, timing))
                q.put(None)
            except BaseException as e:      # noqa: BLE001
                q.put(e)

        th = threading.Thread(target=producer, daemon=True, name="one-off-producer")
        th.start()
        try:
            while True:
                item = q.get()
                if item is None:
                    break
                if isinstance(item, BaseException):
                    raise item
                batch, metrics, timing = item
                with marked_timer("step", timing):
                    self._train_on_actor(batch, metrics, timing)
                    with marked_timer("sync_weights", timing):
                        asyncio.run(self.sampling_client.pause_all(cfg_get(self.config, "sampler_pausing_strategy", "continue")))
                        self._broadcast_weights()
                        asyncio.run(self.sampling_client.continue_all())
                    metrics.update(self.weight_sync_metrics())
                self._finish_step(batch, metrics, timing)
        finally:
            stop.set()

    def _finish_step(self, batch: DataProto, metrics: dict, timing: dict) -> None:
        metrics.update(compute_data_metrics(batch, use_critic=self.use_critic))
        metrics.update(compute_timing_metrics(batch, timing))
        n_tok = float(batch.batch["attention_mask"].sum())
        if timing.get("step"):
            metrics["perf/throughput_tokens_per_s"] = n_tok / timing["step"]
            metrics["perf/throughput_tokens_per_s_per_gpu"] = n_tok / timing["step"] / max(1, self._total_gpus())
        if hasattr(self.train_sampler, "update"):
            self.train_sampler.update(batch)
        self._post_step(metrics, timing)

    def _total_gpus(self) -> int:
        n = self.actor_wg.world_size
        if self.disaggregated:
            n += self.sampler_wg.world_size
        return n

    # ------------------------------------------------------------------ rollout + batch preparation
    def _sample_and_prepare(self, batch_dict: dict, step: int, metrics: dict, timing: dict) -> DataProto:
        cfg = self.config
        gen_batch = self._prepare_batch(batch_dict, step)
        if self._use_dummy_batch:
            batch = self.program_processor.create_dummy_batch(gen_batch, global_steps=step)
        else:
            with marked_timer("gen", timing):
                if self.hybrid_engine:
                    self.sampler_wg.sampler_mode()           # trainer vacates the device, KV pool comes back
                programs, uid_to_index = self.program_runner.create_programs(gen_batch, step)
                self._uid_to_index = uid_to_index
                finished, engine_metrics = self._run_coro(self.program_runner.run_and_collect())
                if self.hybrid_engine:
                    self.sampler_wg.trainer_mode()
            metrics.update(engine_metrics)
            if cfg_get(cfg, "filter_program_errors", False):
                from ..programs.base_program import FAILED_PROGRAM_REWARD
                finished = [p for p in finished if p.reward > FAILED_PROGRAM_REWARD / 2]
            finished = [p for p in finished if p.training_steps]
            if not finished:
                raise RuntimeError("no trainable program finished in this step")
            with marked_timer("transform", timing):
                batch, pm = self.program_processor.transform_programs(finished, self.experiment_dir, step, uid_to_index)
            metrics.update(pm)
        batch.meta_info["temperature"] = float(gen_batch.meta_info.get("sample_params", {}).get(
            "temperature", cfg_get(cfg, "decoding.temperature", 1.0)) or 1.0)
        batch.meta_info["global_steps"] = step
        world_sizes = self._collect_world_sizes()
        if self.use_critic or self.use_rm or cfg_get(cfg, "kl_reward"):
            batch = pad_dataproto_to_world_size(batch, world_sizes)
        if self.use_rm:
            with marked_timer("reward_model", timing):
                rm = self.rm_wg.forward(batch)
                batch.batch["token_level_scores"] = batch.batch["token_level_scores"] + rm.batch["rm_scores"]
        if self.use_critic:
            with marked_timer("values", timing):
                batch.batch["values"] = self.critic_wg.forward(batch).batch["values"]
        if cfg_get(cfg, "kl_reward"):
            with marked_timer("ref", timing):
                batch.batch["ref_log_probs"] = self.ref_policy_wg.forward(batch).batch["log_probs"]
                batch.batch["old_log_probs"] = self.actor_wg.forward(batch).batch["log_probs"]
            rewards, kl_metrics = apply_kl_penalty(batch.batch["token_level_scores"], batch.batch["old_log_probs"],
                                                   batch.batch["ref_log_probs"], batch.batch["response_mask"], self.kl_ctrl,
                                                   cfg_get(cfg, "kl_reward", "kl"))
            batch.batch["token_level_rewards"] = rewards
            metrics.update(kl_metrics)
        with marked_timer("adv", timing):
            batch = compute_advantage_component(batch, self._adv_config(), metrics)
        batch = pad_dataproto_to_world_size(batch, world_sizes)
        batch = balance_batch(batch, self.actor_wg.world_size, metrics)
        if self.use_critic:
            with marked_timer("update_critic", timing):
                mb = batch.select(deepcopy=False)
                process_mini_batch(mb)
                out = self.critic_wg.forward_backward(mb, loss_fn="value", loss_fn_args=self._loss_args())
                metrics.update(out.meta_info["metrics"])
                metrics.update(self.critic_wg.optim_step(step_lr=True).meta_info["metrics"])
        if self.use_ref and "ref_log_probs" not in batch.batch:
            with marked_timer("ref", timing):
                batch.batch["ref_log_probs"] = self.ref_policy_wg.forward(batch).batch["log_probs"]
        return batch

    def _run_coro(self, coro):
        """Run a coroutine to completion from this (synchronous) thread."""
        return asyncio.run(coro)

    # ------------------------------------------------------------------ policy update
    def _train_on_actor(self, batch: DataProto, metrics: dict, timing: dict) -> None:
        cfg = self.config
        critic_warmup = int(cfg_get(cfg, "critic_warmup", 0) or 0)
        if self.use_sampler_logprobs:
            batch.batch["old_log_probs"] = batch.batch["sampler_log_probs"].clone()
        elif "old_log_probs" not in batch.batch:
            with marked_timer("old_log_prob", timing):
                out = self.actor_wg.forward(batch)
                batch.batch["old_log_probs"] = out.batch["log_probs"]
                if "entropy" in out.batch:
                    rm = batch.batch["response_mask"]
                    metrics["actor/old_entropy"] = float((out.batch["entropy"] * rm).sum() / rm.sum().clamp_min(1))
        if "sampler_log_probs" in batch.batch and not self.use_sampler_logprobs:
            metrics.update(aggregate_trainer_sampler_metrics([compute_trainer_sampler_mismatch_metrics(batch)]))
        if self.global_steps <= critic_warmup:
            return
        with marked_timer("forward_backward", timing):
            out = update_trainer(batch, self.training_client, cfg_get(cfg, "loss", "ppo"), self._loss_args(),
                                 epochs=int(cfg_get(cfg, "ppo_epochs", 1)), mini_batch_size=int(cfg_get(cfg, "mini_batch_size", 0) or 0),
                                 mini_batch_shuffle=bool(cfg_get(cfg, "mini_batch_shuffle", False)),
                                 mini_batch_seed=cfg_get(cfg, "mini_batch_seed"), world_size=self.actor_wg.world_size)
        metrics.update(out)

    # ------------------------------------------------------------------ validation
    def _validation_step(self) -> dict:
        if self.val_dataloader is None:
            return {}
        n = int(cfg_get(self.config, "validation.decoding.n", 1) or 1)
        vdec = cfg_get(self.config, "validation.decoding", {}) or {}
        vdec = vdec.to_dict() if hasattr(vdec, "to_dict") else dict(vdec)
        programs_all = []
        it = iter(self.val_dataloader)
        if self.hybrid_engine:
            self.sampler_wg.sampler_mode()
        try:
            while True:
                try:
                    batch_dict = it.next(len(self.val_dataset))
                except StopIteration:
                    break
                from .driver_utils import convert_batch_dict_to_dataproto
                vb = convert_batch_dict_to_dataproto(batch_dict, self.global_steps, val=True, val_n_samples=n)
                vb.meta_info["sample_params"] = {k: v for k, v in vdec.items() if k != "n"}
                self.program_runner.create_programs(vb, self.global_steps)
                finished, _ = self._run_coro(self.program_runner.run_and_collect(val=True))
                programs_all.extend(finished)
        finally:
            if self.hybrid_engine:
                self.sampler_wg.trainer_mode()
        return self._compute_validation_metrics(programs_all, n)
