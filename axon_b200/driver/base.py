"""Common machinery of the PPO drivers: dataloaders, worker groups, sampler servers, the program
pipeline, weight broadcast, validation, checkpoints and per-step logging
(reference: axon/driver/base.py:60-781). ``SyncPPO`` and ``AsyncPPO`` supply the training loop.
"""
from __future__ import annotations

import asyncio
import os
import re
import time
import warnings
from abc import ABC, abstractmethod

import numpy as np
import torch

from ..controller.worker_group import ClassWithInitArgs, init_worker_group
from ..core.role import Role
from ..data import DynamicDataLoader, RLDataset, collate_rl_dataset, create_data_sampler
from ..protocol import DataProto
from ..tinker.training_client import TrainingClient
from ..utils.metrics import aggregate_trainer_sampler_metrics
from ..utils.rl.kl import get_kl_controller
from ..utils.state import find_latest_ckpt_path
from ..utils.temperature_scheduler import TemperatureScheduler
from ..utils.tracking import Tracking
from .components.program_component import create_program_components
from .driver_utils import RoleWorkerConfig, ValidationResult, convert_batch_dict_to_dataproto


def cfg_get(cfg, key, default=None):
    cur = cfg
    for part in key.split("."):
        if isinstance(cur, dict) and part in cur:
            cur = cur[part]
        elif cur is not None and not isinstance(cur, dict) and hasattr(cur, part):
            cur = getattr(cur, part)
        else:
            return default
    return default if cur is None else cur


class PPODriverBase(ABC):
    def __init__(self, config, tokenizer, role_worker_mapping: dict, processor=None, backend: str = "process"):
        self.config = config
        self.tokenizer, self.processor = tokenizer, processor
        self.role_worker_mapping: dict[Role, RoleWorkerConfig] = role_worker_mapping
        self.backend = backend
        self.hybrid_engine = bool(cfg_get(config, "hybrid_engine", True))
        self.disaggregated = not self.hybrid_engine
        self.use_critic = Role.Critic in role_worker_mapping
        self.use_ref = Role.RefPolicy in role_worker_mapping
        self.use_rm = Role.RewardModel in role_worker_mapping
        self.global_steps = 1
        self._eval_only = cfg_get(config, "mode", "train") == "eval"
        self._use_dummy_batch = bool(cfg_get(config, "use_dummy_batch", False))
        self._memory_stress_test = bool(cfg_get(config, "memory_stress_test", False))
        self.experiment_dir = os.path.join(str(cfg_get(config, "output_dir", "outputs")), str(cfg_get(config, "project_name", "axon")),
                                           str(cfg_get(config, "experiment_name", "run")))
        os.makedirs(self.experiment_dir, exist_ok=True)
        self.tracking = Tracking(cfg_get(config, "project_name", "axon"), cfg_get(config, "experiment_name", "run"),
                                 list(cfg_get(config, "logger", ["console"])), config=config)
        self.temperature_scheduler = TemperatureScheduler(cfg_get(config, "decoding.temperature_schedule", {}) or {})
        self.kl_ctrl = None
        self.routing_table = None
        self.actor_wg = self.sampler_wg = self.critic_wg = self.ref_policy_wg = self.rm_wg = None
        self._all_wgs: list = []
        self._init_dataloader()

    # ------------------------------------------------------------------ abstract
    @abstractmethod
    def _init_mode(self) -> None: ...

    @abstractmethod
    def _run_training_loop(self) -> None: ...

    @abstractmethod
    def _validation_step(self) -> dict: ...

    # ------------------------------------------------------------------ data
    def _init_dataloader(self) -> None:
        cfg = self.config
        self.train_dataset = RLDataset(cfg_get(cfg, "train_files"), cfg_get(cfg, "data_mix"))
        self.val_dataset = RLDataset(cfg_get(cfg, "val_files"))
        self.train_sampler = create_data_sampler(cfg, self.train_dataset)
        self.train_batch_size = int(cfg_get(cfg, "train_batch_size", 1))
        self.train_dataloader = DynamicDataLoader(self.train_dataset, sampler=self.train_sampler, collate_fn=collate_rl_dataset,
                                                  batch_size=self.train_batch_size, infinite=True)
        self.val_dataloader = None
        if len(self.val_dataset) > 0:
            self.val_dataloader = DynamicDataLoader(self.val_dataset, collate_fn=collate_rl_dataset,
                                                    batch_size=len(self.val_dataset), infinite=False)
        if not self._eval_only:
            assert len(self.train_dataset) >= 1, "the training dataset is empty (config.train_files)"
        self.steps_per_epoch = None
        if cfg_get(cfg, "total_epochs") is not None:
            self.steps_per_epoch = max(1, len(self.train_dataset) // self.train_batch_size)
            self.total_training_steps = self.steps_per_epoch * int(cfg_get(cfg, "total_epochs"))
        elif cfg_get(cfg, "total_training_steps") is not None:
            self.total_training_steps = int(cfg_get(cfg, "total_training_steps"))
        else:
            warnings.warn("neither total_training_steps nor total_epochs is set; defaulting to 1e9 steps", stacklevel=2)
            self.total_training_steps = int(1e9)
        for role in ("actor", "critic"):
            sub = cfg_get(cfg, f"{role}.lr_scheduler")
            if isinstance(sub, dict) and not sub.get("total_steps"):
                sub["total_steps"] = self.total_training_steps
            args = cfg_get(cfg, f"{role}.lr_scheduler_args")
            if isinstance(args, dict) and int(args.get("total_training_steps") or -1) <= 0:
                args["total_training_steps"] = self.total_training_steps

    def _prepare_batch(self, batch_dict: dict, global_steps: int) -> DataProto:
        return convert_batch_dict_to_dataproto(batch_dict, global_steps=global_steps, n_samples=int(cfg_get(self.config, "decoding.n", 1)),
                                               temperature_scheduler=self.temperature_scheduler,
                                               temperature_config=cfg_get(self.config, "decoding.temperature_schedule"))

    @staticmethod
    def _collect_metrics(result, *aggregators) -> dict:
        if isinstance(result, list):
            merged = {}
            for agg in (aggregators or (aggregate_trainer_sampler_metrics,)):
                merged.update(agg(result))
            return merged
        return result if isinstance(result, dict) else {}

    # ------------------------------------------------------------------ workers
    def init_workers(self) -> None:
        """Roles that share a resource pool are fused into one worker process per GPU (hybrid engine);
        other roles get their own groups. Then models, sampler servers, program pipeline, weight-sync
        route and the mode-specific set-up."""
        by_pool: dict[int, tuple] = {}
        for role, rw in self.role_worker_mapping.items():
            entry = by_pool.setdefault(id(rw.resource_pool), (rw.resource_pool, {}))
            entry[1][str(role)] = ClassWithInitArgs(rw.cls, **rw.init_kwargs)
        groups: dict[str, object] = {}
        rpc_timeout = cfg_get(self.config, "rpc_timeout_s", 3600.0)
        for pool, class_dict in by_pool.values():
            out = init_worker_group(class_dict, pool, backend=self.backend, rpc_timeout=rpc_timeout)
            groups.update(out)
            self._all_wgs.append(next(iter(out.values())))
        self.actor_wg = groups.get(str(Role.Actor))
        self.sampler_wg = groups.get(str(Role.Sampler))
        self.critic_wg = groups.get(str(Role.Critic))
        self.ref_policy_wg = groups.get(str(Role.RefPolicy))
        self.rm_wg = groups.get(str(Role.RewardModel))
        assert self.actor_wg is not None and self.sampler_wg is not None, "actor and sampler roles are required"
        # trainers first: a colocated sampler binds to the trainer's parameter buffer
        for wg in (self.actor_wg, self.critic_wg, self.ref_policy_wg, self.rm_wg, self.sampler_wg):
            if wg is not None:
                wg.init_model()
        self.training_client = TrainingClient(self.actor_wg, self.tokenizer)
        self._initialize_sampler_servers()
        comps = create_program_components(self.config, self.tokenizer, self.processor, self.server_addresses,
                                          self.sampler_servers, hybrid_engine=self.hybrid_engine)
        self.sampling_client, self.engine = comps.sampling_client, comps.engine
        self.program_processor, self.program_runner, self.tasks_loop = comps.program_processor, comps.program_runner, comps.tasks_loop
        if cfg_get(self.config, "kl_reward"):
            self.kl_ctrl = get_kl_controller(cfg_get(self.config, "kl_reward_args", {}))
        if cfg_get(self.config, "moe_replay", False) and cfg_get(self.config, "strategy", "fsdp") != "megatron":
            raise ValueError("moe_replay needs the megatron-style trainer (strategy=megatron)")
        if self.disaggregated:
            self._init_p2p_weight_sync()
        self._init_mode()

    def _initialize_sampler_servers(self) -> None:
        """In-process server objects when the workers live in this process (inline backend), HTTP
        addresses otherwise."""
        self.sampler_servers, self.server_addresses = [], []
        if self.backend == "inline":
            for w in self.sampler_wg.workers:
                obj = w.role_objects[str(Role.Sampler)] if hasattr(w, "role_objects") else w
                self.sampler_servers.append(obj.get_server())
            return
        addrs = self.sampler_wg.get_server_address()
        self.server_addresses = [a for a in addrs if a]
        assert self.server_addresses, "sampler workers did not report an HTTP address (set sampler.serve_http=true)"

    def _init_p2p_weight_sync(self) -> None:
        """Bridge process group over trainer + sampler ranks, both sides' parameter maps, and the
        routing table that says which trainer rank feeds which sampler shard."""
        from ..controller.worker_group import _free_port
        from ..utils.p2p.routing_table import RoutingTable
        n_train, n_samp = self.actor_wg.world_size, self.sampler_wg.world_size
        port = _free_port()
        kw = dict(master_addr="127.0.0.1", master_port=port, world_size=n_train + n_samp)
        self._nonblocking(self.sampler_wg, "connect_sampler_to_trainer", rank_offset=n_train, **kw)
        self.actor_wg.connect_trainer_to_sampler(rank_offset=0, **kw)
        self._join_nonblocking()
        actor_map = self.actor_wg.get_parameter_mapping()
        sampler_map = self.sampler_wg.get_parameter_mapping()
        self.routing_table = RoutingTable(actor_map, sampler_map)

    # non-blocking RPC helpers (the two sides of a P2P exchange must run at the same time)
    def _nonblocking(self, wg, method: str, *args, **kwargs) -> None:
        import threading
        err: list = []

        def run():
            try:
                getattr(wg, method)(*args, **kwargs)
            except BaseException as e:       # noqa: BLE001
                err.append(e)
        t = threading.Thread(target=run, daemon=True)
        t.start()
        self._pending_rpc = getattr(self, "_pending_rpc", []) + [(t, err)]

    def _join_nonblocking(self) -> None:
        for t, err in getattr(self, "_pending_rpc", []):
            t.join()
            if err:
                raise err[0]
        self._pending_rpc = []

    def _broadcast_weights(self) -> None:
        """Trainer -> sampler weight push: receivers are posted first (non-blocking), then the senders
        run. The routing table travels once; workers keep their compiled plans."""
        self._nonblocking(self.sampler_wg, "receive_trainer_to_sampler_weights", routing_table=self.routing_table)
        sent = self.actor_wg.send_trainer_to_sampler_weights(routing_table=self.routing_table)
        self._join_nonblocking()
        self.routing_table = None
        # what the last push did, per trainer rank: bytes, seconds, transport ("peer-store kernel" | "messages")
        self.last_weight_sync = sent if isinstance(sent, list) else [sent]

    def weight_sync_metrics(self) -> dict:
        """Scalars of the last trainer -> sampler push for the step log."""
        recs = [r for r in (getattr(self, "last_weight_sync", None) or []) if isinstance(r, dict)]
        if not recs:
            return {}
        out = {"sync/bytes": float(sum(r.get("bytes", 0) for r in recs)),
               "sync/seconds_max": float(max(r.get("seconds", 0.0) for r in recs)),
               "sync/peer_store_kernel": float(all(r.get("transport") == "peer-store kernel" for r in recs))}
        if all("kernel_ms" in r for r in recs):
            out["sync/kernel_ms_max"] = float(max(r["kernel_ms"] for r in recs))
        return out

    def _collect_world_sizes(self) -> list[int]:
        sizes = [wg.world_size for wg, on in ((self.critic_wg, self.use_critic), (self.ref_policy_wg, self.use_ref),
                                               (self.rm_wg, self.use_rm)) if on and wg is not None and wg.world_size]
        sizes.append(self.actor_wg.world_size)
        if self.disaggregated and self.sampler_wg is not None:
            sizes.append(self.sampler_wg.world_size)
        return sizes

    # ------------------------------------------------------------------ top-level loop
    def train_rl(self) -> None:
        try:
            if not self._eval_only:
                self._load_state()
                if self.disaggregated and not self._use_dummy_batch:
                    self._broadcast_weights()
            val_cfg = cfg_get(self.config, "validation")
            if val_cfg and self.val_dataloader is not None and (cfg_get(val_cfg, "before_train", False) or self._eval_only):
                self.tracking.log(self._validation_step(), step=self.global_steps)
            if self._eval_only:
                return
            if self._memory_stress_test:
                self._run_memory_stress_test()
                return
            self._run_training_loop()
            if self.val_dataloader is not None:
                self.tracking.log(self._validation_step(), step=self.global_steps)
        finally:
            self.tracking.finish()

    def _run_memory_stress_test(self) -> None:
        """Worst-case memory rehearsal: a full batch of maximum-length rows goes through sampler
        wake/sleep, the old-log-prob forward and one forward_backward + optim_step. If this passes the
        configuration fits."""
        from .components.advantage_component import compute_advantage_component
        from .driver_utils import balance_batch, pad_dataproto_to_world_size, update_trainer
        asyncio.run(self.sampling_client.wake_up())
        asyncio.run(self.sampling_client.sleep())
        batch = self.program_processor.create_dummy_batch(None, batch_size=self.train_batch_size,
                                                          n_samples=int(cfg_get(self.config, "decoding.n", 1)))
        metrics: dict = {}
        batch = compute_advantage_component(batch, self._adv_config(drop_zero=False), metrics)
        batch = pad_dataproto_to_world_size(batch, self._collect_world_sizes())
        batch = balance_batch(batch, self.actor_wg.world_size, metrics)
        batch.meta_info["temperature"] = float(cfg_get(self.config, "decoding.temperature", 1.0))
        old = self.actor_wg.forward(batch)
        batch.batch["old_log_probs"] = old.batch["log_probs"]
        metrics.update(update_trainer(batch, self.training_client, cfg_get(self.config, "loss", "ppo"), self._loss_args(),
                                      epochs=1, mini_batch_size=int(cfg_get(self.config, "mini_batch_size", 0) or 0),
                                      world_size=self.actor_wg.world_size))
        self.tracking.log({f"stress/{k}": v for k, v in metrics.items()}, step=0)

    def _adv_config(self, drop_zero: bool | None = None) -> dict:
        return {"advantage": cfg_get(self.config, "advantage", "grpo"),
                "advantage_args": dict(cfg_get(self.config, "advantage_args", {}) or {}),
                "drop_zero_advantage_samples": bool(cfg_get(self.config, "drop_zero_advantage_samples", False)) if drop_zero is None else drop_zero,
                "stepwise_advantage_mode": cfg_get(self.config, "stepwise_advantage_mode", "broadcast")}

    def _loss_args(self) -> dict:
        args = cfg_get(self.config, "loss_args", {}) or {}
        return args.to_dict() if hasattr(args, "to_dict") else dict(args)

    # ------------------------------------------------------------------ post-step
    def _post_step(self, metrics: dict, timing_raw: dict) -> None:
        vsteps = int(cfg_get(self.config, "validation.steps", -1) or -1)
        if vsteps > 0 and self.val_dataloader is not None and self.global_steps % vsteps == 0:
            t0 = time.time()
            metrics.update(self._validation_step())
            timing_raw["validation"] = time.time() - t0
        save_steps = int(cfg_get(self.config, "save_steps", -1) or -1)
        if save_steps > 0 and self.global_steps % save_steps == 0:
            t0 = time.time()
            self._save_state()
            timing_raw["save_state"] = time.time() - t0
        for key in ("validation", "save_state"):
            if key in timing_raw:
                metrics[f"timing_s/{key}"] = timing_raw[key]
        self.tracking.log(metrics, step=self.global_steps)
        self.temperature_scheduler.step()
        self.global_steps += 1

    def _compute_validation_metrics(self, programs, n_samples: int) -> dict:
        res = ValidationResult(n_samples=n_samples)
        for p in programs:
            res.add(p.reward, p.group_id, (p.metadata or {}).get("data_source", "unknown"))
        return res.compute_metrics()

    # ------------------------------------------------------------------ checkpoints
    def _save_state(self) -> None:
        folder = os.path.join(self.experiment_dir, "checkpoints", f"step_{self.global_steps}")
        os.makedirs(folder, exist_ok=True)
        kw = dict(max_ckpt_to_keep=cfg_get(self.config, "max_checkpoints_to_keep"),
                  save_mode=cfg_get(self.config, "checkpoint_format", "sharded"), async_save=bool(cfg_get(self.config, "async_save", False)))
        self.actor_wg.save_state(os.path.join(folder, str(Role.Actor)), self.global_steps, **kw)
        if self.use_critic:
            self.critic_wg.save_state(os.path.join(folder, str(Role.Critic)), self.global_steps, **kw)
        state = {"dataloader": self.train_dataloader.state_dict(), "global_steps": self.global_steps,
                 "temperature_step": self.temperature_scheduler.current_step,
                 "kl_ctrl": getattr(self.kl_ctrl, "__dict__", None) and dict(self.kl_ctrl.__dict__)}
        tmp = os.path.join(folder, "data.pt.tmp")
        torch.save(state, tmp)
        os.replace(tmp, os.path.join(folder, "data.pt"))

    def _load_state(self) -> None:
        if not cfg_get(self.config, "resume_from_checkpoint", False):
            return
        folder = find_latest_ckpt_path(os.path.join(self.experiment_dir, "checkpoints"))
        if folder is None:
            print(f"[load_state] no checkpoint under {self.experiment_dir}/checkpoints; starting from scratch", flush=True)
            return
        m = re.search(r"(\d+)$", os.path.basename(folder))
        mode = cfg_get(self.config, "checkpoint_format", "sharded")
        self.actor_wg.load_state(os.path.join(folder, str(Role.Actor)), save_mode=mode)
        if self.use_critic:
            self.critic_wg.load_state(os.path.join(folder, str(Role.Critic)), save_mode=mode)
        data_path = os.path.join(folder, "data.pt")
        if os.path.exists(data_path):
            state = torch.load(data_path, weights_only=False)
            if "dataloader" in state:
                self.train_dataloader.load_state_dict(state["dataloader"])
                self.temperature_scheduler.set_step(int(state.get("temperature_step", 0)))
                if self.kl_ctrl is not None and state.get("kl_ctrl"):
                    self.kl_ctrl.__dict__.update(state["kl_ctrl"])
            else:                        # bare dataloader state
                self.train_dataloader.load_state_dict(state)
        self.global_steps = (int(m.group(1)) if m else 0) + 1      # the saved step is complete
        print(f"[load_state] resumed from {folder}; next step {self.global_steps}", flush=True)

    # ------------------------------------------------------------------ shutdown
    def shutdown(self) -> None:
        try:
            if getattr(self, "program_runner", None) is not None:
                self.program_runner.shutdown()
            if getattr(self, "engine", None) is not None:
                try:
                    self.engine.run_in_engine_loop(self.engine.shutdown(), timeout=10)
                except Exception:
                    pass
            if self.sampler_wg is not None:
                try:
                    self.sampler_wg.shutdown_servers() if hasattr(self.sampler_wg, "shutdown_servers") else None
                except Exception:
                    pass
        finally:
            seen = set()
            for wg in self._all_wgs:
                root = getattr(wg, "_wg", wg)
                if id(root) not in seen:
                    seen.add(id(root))
                    root.shutdown()
