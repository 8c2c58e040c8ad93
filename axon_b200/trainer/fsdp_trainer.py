"""Data-parallel trainer worker (the reference's FSDP personality: axon/trainer/fsdp_trainer.py:107-869).

One worker per GPU. The model's parameters live in one flat bf16 buffer that every rank holds in
full; fp32 master weights and Adam moments are sharded 1/W per rank (ZeRO-1) and gradients are
reduced once per optimizer step — with 180 GB of HBM per GPU this trades memory the device has for
the per-layer all-gathers and reduce-scatters that parameter sharding would put on every
micro-batch. The worker exposes the reference's RPC surface: ``init_model``, ``forward``,
``forward_backward``, ``optim_step``, ``save_state`` / ``load_state``, ``load_model`` /
``offload_model`` and the profiler hooks. ``model`` selects the head: ``CausalLM`` (policy / reference
log-probs), ``ValueModel`` (critic) or ``RewardModel``.
"""
from __future__ import annotations

import datetime
import os
import time

import numpy as np
import torch
import torch.distributed as dist

from ..controller.decorator import Dispatch, make_nd_compute_dataproto_dispatch_fn, register
from ..core.worker import Worker
from ..protocol import DataProto
from ..utils.profiler import DistProfiler, DistProfilerExtension, FlopsCounter, ProfilerConfig
from .policy import OptimConfig, PolicyEngine


def _get(cfg, key, default=None):
    if cfg is None:
        return default
    cur = cfg
    for part in key.split("."):
        if isinstance(cur, dict) and part in cur:
            cur = cur[part]
        elif not isinstance(cur, dict) and hasattr(cur, part):
            cur = getattr(cur, part)
        else:
            return default
    return default if cur is None else cur


# --------------------------------------------------------------------------------------- model kinds
class CausalLM:
    """Policy / reference model: log-probs (and entropy) of the batch's own tokens."""
    value_head = False
    forward_keys = ("input_ids", "attention_mask", "position_ids", "response_mask")

    @staticmethod
    def forward(engine: PolicyEngine, data: DataProto, calculate_entropy: bool) -> DataProto:
        return engine.forward(data, want_entropy=calculate_entropy)

    @staticmethod
    def forward_backward(engine: PolicyEngine, data: DataProto, loss_fn: str, loss_fn_args: dict) -> dict:
        return engine.forward_backward(data, loss_fn=loss_fn, loss_args=loss_fn_args)


class ValueModel:
    """Critic: a scalar value per token from a value head."""
    value_head = True
    forward_keys = ("input_ids", "attention_mask", "position_ids", "response_mask")

    @staticmethod
    def forward(engine: PolicyEngine, data: DataProto, calculate_entropy: bool) -> DataProto:
        return engine.forward_values(data)

    @staticmethod
    def forward_backward(engine: PolicyEngine, data: DataProto, loss_fn: str, loss_fn_args: dict) -> dict:
        return engine.forward_backward_values(data, loss_fn=loss_fn or "value", loss_args=loss_fn_args)


class RewardModel:
    """Sequence-level reward from a value head on the last token."""
    value_head = True
    forward_keys = ("input_ids", "attention_mask", "position_ids")

    @staticmethod
    def forward(engine: PolicyEngine, data: DataProto, calculate_entropy: bool) -> DataProto:
        return engine.forward_rewards(data)

    @staticmethod
    def forward_backward(engine, data, loss_fn, loss_fn_args):
        raise RuntimeError("reward models are forward-only")


MODEL_KINDS = {"causal_lm": CausalLM, "value": ValueModel, "reward": RewardModel}


class TrainerWorker(Worker, DistProfilerExtension):
    def __init__(self, config, model=None, name: str = "trainer", **kwargs):
        Worker.__init__(self)
        self.config = config
        self.name = name
        self.model_kind = MODEL_KINDS[model] if isinstance(model, str) else (model or CausalLM)
        self._forward_only = bool(_get(config, "forward_only", False))
        use_cuda = torch.cuda.is_available() and not _get(config, "force_cpu", False)
        if use_cuda:
            torch.cuda.set_device(self.local_rank % torch.cuda.device_count())
            self.device = torch.device("cuda", torch.cuda.current_device())
        else:
            self.device = torch.device("cpu")
        self.pg = None
        if self.world_size > 1:
            if not dist.is_initialized():
                dist.init_process_group(backend="nccl" if use_cuda else "gloo", rank=self.rank, world_size=self.world_size,
                                        init_method=f"tcp://{self._master_addr}:{self._master_port}",
                                        timeout=datetime.timedelta(seconds=int(_get(config, "dist_timeout_s", 600))))
            self.pg = dist.group.WORLD
        sp = int(_get(config, "fsdp.ulysses_sequence_parallel_size", 1))
        assert self.world_size % sp == 0, f"world size {self.world_size} is not divisible by sequence-parallel size {sp}"
        self.ulysses_sequence_parallel_size = sp
        # ranks of one sequence-parallel group consume the same data shard; the group's rank 0 reports
        self._register_dispatch_collect_info("trainer", dp_rank=self.rank // sp, is_collect=self.rank % sp == 0)
        pcfg = ProfilerConfig.from_config(_get(config, "profiler", {}), _get(config, "global_profiler", None))
        DistProfilerExtension.__init__(self, DistProfiler(self.rank, pcfg))
        self._is_offload_param = bool(_get(config, "param_offload", False))
        self._is_offload_optimizer = not self._forward_only and bool(_get(config, "optimizer_offload", False))
        self.engine: PolicyEngine | None = None
        self.model = None
        self.tokenizer = None
        self.state_manager = None
        self.flops_counter = None
        self._fb_time_acc, self._fb_seqlens_acc = 0.0, []
        self._host_params: torch.Tensor | None = None

    # ------------------------------------------------------------------ set-up
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def init_model(self):
        from ..utils.hf_model import build_model
        from ..utils.state import FSDPStateManager
        from ..utils.tokenizer import hf_tokenizer
        cfg = self.config
        model_path = _get(cfg, "model_path")
        assert model_path, "config.model_path is required"
        dtype = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
                 "float16": torch.float16}[str(_get(cfg, "dtype", "bfloat16" if self.device.type == "cuda" else "float32"))]
        if self.device.type == "cpu" and dtype != torch.float32 and not _get(cfg, "allow_cpu_low_precision", False):
            dtype = torch.float32
        seed = int(_get(cfg, "seed", 42))
        torch.manual_seed(seed)
        self.model = self._build(model_path, dtype, seed)
        try:
            self.tokenizer = hf_tokenizer(model_path, trust_remote_code=bool(_get(cfg, "trust_remote_code", False)))
        except Exception:
            self.tokenizer = None
        betas = _get(cfg, "optimizer_args.betas", [0.9, 0.95])
        from .policy import schedule_from_config
        sched = schedule_from_config(_get(cfg, "lr_scheduler", None), _get(cfg, "lr_scheduler_args", None),
                                     float(_get(cfg, "optimizer_args.lr", 1e-6)))
        extra = dict(_get(cfg, "optimizer_args.override_optimizer_args", {}) or {})
        ocfg = OptimConfig(lr=float(_get(cfg, "optimizer_args.lr", 1e-6)), weight_decay=float(extra.get("weight_decay", _get(cfg, "optimizer_args.weight_decay", 0.1))),
                           beta1=float(betas[0]), beta2=float(betas[1]), eps=float(extra.get("eps", _get(cfg, "optimizer_args.eps", 1e-8))),
                           grad_clip=float(_get(cfg, "grad_clip", 1.0) or 0.0),
                           grad_norm_threshold=float(_get(cfg, "fsdp.grad_norm_threshold", 0.0) or 0.0), **sched)
        self.engine = PolicyEngine(self.model, ocfg, process_group=self.pg,
                                   max_token_len_per_gpu=int(_get(cfg, "max_token_len_per_gpu", 16384)) * self.ulysses_sequence_parallel_size,
                                   temperature=1.0, shard_size=int(_get(cfg, "fsdp.fsdp_size", -1) or -1))
        # multi-token prediction: on when the model has such a module and the factor is set (the reference
        # switches it with AXON_ENABLE_MTP and takes megatron's mtp_loss_scaling_factor)
        if os.environ.get("AXON_ENABLE_MTP", "1") not in ("0", "false", "False"):
            self.engine.mtp_loss_coef = float(_get(cfg, "mtp_loss_scaling_factor", _get(cfg, "megatron.mtp_loss_scaling_factor", 0.0)) or 0.0)
        if bool(_get(cfg, "fsdp.enable_activation_offload", False)) and not self._forward_only:
            from ..utils.activation_offload import ActivationOffloader
            target = getattr(self.model, "inner", self.model)
            target.offloader = ActivationOffloader(self.device)
        self.flops_counter = FlopsCounter(self.model.cfg, dtype)
        self.state_manager = self._make_state_manager()
        if self._is_offload_param:
            self.offload_model(include_model=True, include_optimizer=False)
        return {"num_params": int(self.model.params.numel), "device": str(self.device), "dtype": str(dtype)}

    def _make_state_manager(self):
        from ..utils.state import FSDPStateManager
        if hasattr(self.model, "full_named_tensors") and hasattr(self.model, "layer_offsets"):      # a family model cut layer by layer
            from ..utils.state.fsdp_state_manager import ShardedFamilyStateManager
            return ShardedFamilyStateManager(self.model, self.engine, group=self._mp_group, processing_class=self.tokenizer,
                                             rank=self.rank, world_size=self.world_size)
        if getattr(self.model, "shard", None) is not None:      # parameter shards: per-rank files + gathered HF export
            from ..utils.state.megatron_state_manager import MegatronStateManager
            return MegatronStateManager(self.model, self.engine, mp_group=self._mp_group, dp_rank=0, processing_class=self.tokenizer,
                                        rank=self.rank, world_size=self.world_size, process_group=self.pg)
        return FSDPStateManager(self.model, self.engine, processing_class=self.tokenizer, rank=self.rank,
                                world_size=self.world_size, process_group=self.pg)

    def _build(self, model_path, dtype, seed):
        from ..models.config import get_config
        from ..models.moe import build_model_for
        from ..utils.hf_model import has_hf_weights, load_hf_weights
        mcfg = get_config(model_path)
        if self.model_kind.value_head:
            mcfg.extra = {**mcfg.extra, "value_head": True}
        lora = _get(self.config, "lora", None)
        if lora is not None and int(_get(lora, "rank", 0) or 0) > 0:
            # adapters: the base stays frozen in the model, `model.params` (what the optimizer, its
            # shards and the checkpoints see) holds only the low-rank matrices
            from ..models.lora import LoRAConfig, LoRADenseModel
            assert mcfg.num_experts == 0 and not self.model_kind.value_head, "LoRA is available on dense causal-LM models"
            model = LoRADenseModel(mcfg, LoRAConfig.from_dict(lora), device=self.device, dtype=dtype)
            model.recompute = str(_get(self.config, "recompute", "selective"))
            if os.path.isdir(str(model_path)) and has_hf_weights(model_path):
                from ..utils.hf_model import iter_hf_weights
                model.base.load_hf_state_dict(dict(iter_hf_weights(model_path)))
            else:
                model.base.init_random(seed=seed)
            return model
        if bool(_get(self.config, "fsdp.param_sharding", False)) and self.world_size > 1:
            # ZeRO-3 / FSDP-style parameter shards over all ranks: the optimizer works on this rank's shards only
            # (a group of its own), replicated parameters are summed by the model's hook
            from ..models.families import FAMILY_TYPES
            from ..models.zero3_dense import Zero3DenseModel
            from ..parallel.zero3 import ShardContext
            family = mcfg.model_type in FAMILY_TYPES
            assert (family or mcfg.num_experts == 0) and not self.model_kind.value_head and self.ulysses_sequence_parallel_size == 1, \
                "parameter sharding is available on dense causal-LM models and on the family toolkit's models, without sequence parallelism"
            own = None
            for r in range(self.world_size):
                g = dist.new_group([r])
                if r == self.rank:
                    own = g
            world_group = self.pg
            self.pg = own
            self._mp_group = world_group
            if family:
                # one piece of every decoder layer per rank; a layer is gathered for its forward and again for its backward
                from ..models.sharded_family import ShardedFamilyModel
                model = ShardedFamilyModel(mcfg, ShardContext(world_group, self.device, fused=False), device=self.device, dtype=dtype)
                if os.path.isdir(str(model_path)) and has_hf_weights(model_path):
                    model.load_hf_checkpoint(model_path)
                else:
                    model.init_random(seed=seed)
                return model
            model = Zero3DenseModel(mcfg, ShardContext(world_group, self.device), device=self.device, dtype=dtype)
            model.recompute = str(_get(self.config, "recompute", "selective"))
            if os.path.isdir(str(model_path)) and has_hf_weights(model_path):
                from ..models.params import FlatParams
                from ..utils.hf_model import iter_hf_weights
                ref = FlatParams(mcfg, "cpu", dtype)
                ref.load_hf_state_dict(dict(iter_hf_weights(model_path)))
                model.load_full_state(ref.views)
            else:
                model.init_random(seed=seed)
            return model
        sp = self.ulysses_sequence_parallel_size
        if sp > 1:
            # Ulysses: consecutive ranks form a sequence-parallel group (same rows, T / sp tokens each); the
            # optimizer keeps sharding over ALL ranks, so its reduce-scatter also completes the partial
            # weight gradients of the group
            from ..models.ulysses import UlyssesDenseModel, UlyssesModelAdapter
            from ..parallel.ulysses import UlyssesContext
            assert mcfg.num_experts == 0 and not self.model_kind.value_head, "sequence parallelism is available on dense causal-LM models"
            sp_group = None
            for i in range(self.world_size // sp):
                ranks = list(range(i * sp, (i + 1) * sp))
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    sp_group = g
            cap = int(_get(self.config, "max_token_len_per_gpu", 16384))       # per-rank token cap; the group packs sp times that
            ctx = UlyssesContext(sp_group, self.device, max_rows_per_rank=(cap + 127) // 128 * 128 + 128, max_width=mcfg.qkv_size)
            inner = UlyssesDenseModel(mcfg, ctx, device=self.device, dtype=dtype)
            inner.recompute = str(_get(self.config, "recompute", "selective"))
            if os.path.isdir(str(model_path)) and has_hf_weights(model_path):
                load_hf_weights(inner, model_path)
            else:
                inner.params.init_random(seed=seed)
            return UlyssesModelAdapter(inner)
        model = build_model_for(mcfg, device=self.device, dtype=dtype)
        model.recompute = str(_get(self.config, "recompute", "selective"))
        if os.path.isdir(str(model_path)) and has_hf_weights(model_path):
            load_hf_weights(model, model_path, strict=not self.model_kind.value_head)
            if self.model_kind.value_head:
                torch.nn.init.normal_(model.params["v_head.weight"], std=0.02)
        else:
            model.params.init_random(seed=seed)     # same seed on every rank: identical replicas
        return model

    # ------------------------------------------------------------------ residency
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def load_model(self, include_model: bool = True, include_optimizer: bool = True):
        if include_model and self._host_params is not None:
            flat = self._host_params.to(self.device, non_blocking=True)
            self.model.params.rebind(flat)
            self._host_params = None
        if include_optimizer and self.engine is not None and not self._forward_only:
            self.engine.load_optimizer()

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def offload_model(self, include_model: bool = True, include_optimizer: bool = True):
        if include_optimizer and self.engine is not None and (self._is_offload_optimizer or include_optimizer == "force"):
            self.engine.offload_optimizer()
        if include_model and self._is_offload_param and self.device.type == "cuda" and self._host_params is None:
            flat = self.model.params.flat
            self._host_params = torch.empty(flat.shape, dtype=flat.dtype, pin_memory=True)
            self._host_params.copy_(flat, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            self.model.params.rebind(torch.empty(0, dtype=flat.dtype, device=self.device))
            torch.cuda.empty_cache()

    # ------------------------------------------------------------------ compute RPCs
    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn(mesh_name="trainer"))
    @DistProfiler.annotate(color="blue", role="forward")
    def forward(self, data: DataProto):
        assert "temperature" in data.meta_info, "temperature must be provided in meta_info"
        keys = [k for k in self.model_kind.forward_keys if data.batch is not None and k in data.batch]
        sel = data.select(batch_keys=keys, non_tensor_batch_keys=[])
        sel.meta_info = dict(data.meta_info)
        max_tok = data.meta_info.get("max_token_len", _get(self.config, "forward_max_token_len_per_gpu", None))
        prev = self.engine.max_tokens
        if max_tok:
            self.engine.max_tokens = int(max_tok) * self.ulysses_sequence_parallel_size
        try:
            out = self.model_kind.forward(self.engine, sel, calculate_entropy=not self._forward_only)
        finally:
            self.engine.max_tokens = prev
        return out.to("cpu")

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn(mesh_name="trainer"))
    @DistProfiler.annotate(color="red", role="forward_backward")
    def forward_backward(self, data: DataProto, loss_fn: str = "ppo", loss_fn_args: dict | None = None):
        if self._forward_only:
            raise RuntimeError("forward_backward must not be called on forward-only workers")
        t0 = time.monotonic()
        # padding rows stay in: every rank must see the same number of rows; their mask is zero
        raw = self.model_kind.forward_backward(self.engine, data, loss_fn, dict(loss_fn_args or {}))
        self._fb_time_acc += time.monotonic() - t0
        self._fb_seqlens_acc.extend(data.batch["attention_mask"].sum(-1).tolist())
        # additive terms (the loss is a partial sum against mini-batch-global denominators) add up over
        # micro-batches; everything else is averaged
        additive = ("loss", "pg_loss", "vf_loss", "entropy_loss", "kl_loss")
        metrics = {f"{self.name}/{k}": float(np.sum(v) if k in additive else np.mean(v)) for k, v in raw.items() if len(v)}
        return DataProto(meta_info={"metrics": metrics})

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn(mesh_name="trainer"))
    @DistProfiler.annotate(color="red", role="optim_step")
    def optim_step(self, step_lr: bool = False):
        """Reduce + clip + sharded AdamW + parameter gather. Optimizer state comes onto the device just
        in time when it is kept on the host between steps."""
        if self._forward_only:
            raise RuntimeError("optim_step must not be called on forward-only workers")
        t0 = time.monotonic()
        out = self.engine.optim_step(step_lr=step_lr)
        if self._is_offload_optimizer:
            self.engine.offload_optimizer()
        metrics = {f"{self.name}/grad_norm": out["grad_norm"], f"{self.name}/lr": out["lr"],
                   f"{self.name}/optim_step_skipped": out["skipped"], f"{self.name}/optim_step_time_s": time.monotonic() - t0}
        if self.device.type == "cuda":
            metrics[f"perf/{self.name}/max_memory_allocated_gb"] = torch.cuda.max_memory_allocated() / 2 ** 30
            metrics[f"perf/{self.name}/max_memory_reserved_gb"] = torch.cuda.max_memory_reserved() / 2 ** 30
            torch.cuda.reset_peak_memory_stats()
        if self._fb_time_acc > 0 and self._fb_seqlens_acc:
            achieved, peak = self.flops_counter.estimate_flops(self._fb_seqlens_acc, self._fb_time_acc)
            metrics[f"perf/{self.name}/mfu"] = achieved / peak if peak not in (0, float("inf")) else 0.0
            metrics[f"perf/{self.name}/tflops"] = achieved
        self._fb_time_acc, self._fb_seqlens_acc = 0.0, []
        return DataProto(meta_info={"metrics": metrics})

    # ------------------------------------------------------------------ checkpoints
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def save_state(self, path: str, global_step: int = 0, max_ckpt_to_keep=None, save_mode: str = "sharded",
                   async_save: bool = False):
        if hasattr(self.model, "save_adapter"):
            # adapter run: the sharded files hold adapters + optimizer state; the exportable artefact is
            # the PEFT-layout adapter directory (the frozen base is the model the run started from)
            save_mode = "sharded"
            if self.rank == 0:
                self.model.save_adapter(os.path.join(path, "lora_adapter"))
        self.state_manager.save_state(path, global_step=global_step, max_ckpt_to_keep=max_ckpt_to_keep,
                                      save_mode=save_mode, async_save=async_save)
        if self._is_offload_optimizer:
            self.engine.offload_optimizer()

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def load_state(self, path: str, save_mode: str = "sharded"):
        self.state_manager.load_state(path, save_mode=save_mode)
        if self._is_offload_optimizer:
            self.engine.offload_optimizer()

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def wait_for_save(self):
        self.state_manager.wait()

    # ------------------------------------------------------------------ misc RPCs
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def start_profile(self, **kw):
        DistProfilerExtension.start_profile(self, role=self.name, **kw)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def stop_profile(self):
        DistProfilerExtension.stop_profile(self)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def get_model_info(self) -> dict:
        c = self.model.cfg
        return {"num_params": int(self.model.params.numel), "hidden_size": c.hidden_size, "num_layers": c.num_hidden_layers,
                "vocab_size": c.vocab_size, "world_size": self.world_size}

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def param_sums(self) -> dict:
        """name -> (fp64 sum, shape, position-weighted fp64 sum) of every parameter tensor this rank holds (weight-sync
        checks compare them; the weighted sum also notices rows that arrived in the wrong place)."""
        from ..utils.state.utils import tensor_digest
        return {n: tensor_digest(v) for n, v in self.model.params.views.items()}

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def full_param_sums(self) -> dict:
        """``param_sums`` of the WHOLE tensors: a trainer with parameter shards or a model-parallel layout gathers them
        (a collective over its ranks), so that the result compares with a sampler that holds whole tensors."""
        from ..utils.state.utils import tensor_digest
        gathered = getattr(self.model, "full_named_tensors", None)
        if gathered is None and getattr(getattr(self, "state_manager", None), "mp_group", None) is not None:
            gathered = self.state_manager.full_named_tensors
        items = gathered() if gathered is not None else self.model.params.views.items()
        return {n: tensor_digest(t) for n, t in items}

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def params_checksum(self) -> float:
        """Sum of all parameters in fp64 — replicas must agree; used by resume and sync tests."""
        return float(self.model.params.flat.double().sum().item())
