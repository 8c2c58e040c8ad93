"""Policy training engine: the compute core behind the trainer workers.

Takes padded ``DataProto`` batches (schema: right-padded ``input_ids`` / ``attention_mask`` /
``response_mask`` ... ``[B, T]``), packs them into padding-free micro-batches under a token budget,
runs the model's explicit forward/backward, evaluates the registered loss on the padded view and
steps a sharded fused AdamW.

Data parallelism is ZeRO-1 on purpose: with 180 GB of HBM per GPU an 8B-30B model keeps a full bf16
working copy (shared with the colocated sampler) and a full fp32 main-gradient buffer on every rank,
so the only collectives of a step are ONE gradient reduce-scatter and ONE parameter all-gather per
optimizer step instead of two all-gathers and one reduce-scatter per layer per micro-batch
(the reference's FSDP path: axon/trainer/fsdp_trainer.py:362-422,587-771).

Log-prob convention: ``log_probs[b, t] = log softmax(logits[b, t-1] / temperature)[input_ids[b, t]]``
and 0 at t = 0 (axon/utils/fsdp/forward_utils.py:109-183).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

from ..models.dense import DenseModel, PackedBatch
from ..ops import optim as OPT
from ..protocol import DataProto
from ..utils.seqlen_balancing import prepare_dynamic_batch
from .algos.loss import agg_loss, compute_loss_fn


@dataclass
class OptimConfig:
    lr: float = 1e-6
    weight_decay: float = 0.1
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    grad_clip: float = 1.0
    grad_norm_threshold: float = 0.0      # > 0: skip the step when the norm exceeds it
    warmup_steps: int = 0
    total_steps: int = 0                  # > 0 enables decay to the floor (cosine / wsd)
    min_lr_ratio: float = 0.0
    schedule: str = "constant"            # constant | cosine | wsd
    min_lr: float = 0.0                   # absolute floor; the larger of min_lr and min_lr_ratio * lr applies
    warmup_init: float = 0.0              # learning rate the warm-up starts from
    num_cycles: float = 0.5               # cosine: half waves over the decay span
    decay_steps: int = 0                  # > 0: the decay ends here instead of at total_steps
    wsd_decay_steps: int = 0              # wsd: length of the final decay (the stable phase fills the rest)
    wsd_decay_style: str = "exponential"  # wsd: exponential | linear | cosine


def lr_at(cfg: OptimConfig, step: int) -> float:
    """Learning rate for 1-based optimizer step ``step``: linear warm-up from ``warmup_init``, then constant,
    cosine decay, or warm-up / stable / decay (``wsd``: constant until the last ``wsd_decay_steps`` steps, which
    fall to the floor with the chosen shape). Schedules of the reference: axon/utils/scheduler_utils.py:27-140
    and the megatron scheduler arguments of axon/config/trainer/trainer.yaml:36-57."""
    floor = max(cfg.min_lr, cfg.min_lr_ratio * cfg.lr)
    if cfg.warmup_steps > 0 and step <= cfg.warmup_steps:
        return cfg.warmup_init + (cfg.lr - cfg.warmup_init) * step / cfg.warmup_steps
    end = cfg.decay_steps if cfg.decay_steps > 0 else cfg.total_steps
    if cfg.schedule == "cosine" and end > cfg.warmup_steps:
        p = min(1.0, (step - cfg.warmup_steps) / (end - cfg.warmup_steps))
        return floor + (cfg.lr - floor) * 0.5 * (1 + math.cos(math.pi * 2 * cfg.num_cycles * p))
    if cfg.schedule == "wsd" and end > cfg.warmup_steps and cfg.wsd_decay_steps > 0:
        start = max(cfg.warmup_steps, end - cfg.wsd_decay_steps)
        if step <= start:
            return cfg.lr
        p = min(1.0, (step - start) / max(1, end - start))
        if cfg.wsd_decay_style == "linear":
            f = 1.0 - p
        elif cfg.wsd_decay_style == "cosine":
            f = 0.5 * (1 + math.cos(math.pi * p))
        else:                                   # exponential: 2^-p scaled to reach zero at p = 1
            f = (0.5 ** p - 0.5) * 2.0
        return floor + (cfg.lr - floor) * f
    return cfg.lr


def schedule_from_config(lr_scheduler, lr_scheduler_args, lr: float, fallback_total: int = 0) -> dict:
    """OptimConfig fields from a role's ``lr_scheduler`` / ``lr_scheduler_args`` blocks. ``lr_scheduler`` is the
    schedule's name (the reference's form) or a mapping ``{type, warmup_steps, warmup_ratio, min_lr_ratio,
    total_steps}``."""
    def g(d, k, default=None):
        if d is None:
            return default
        v = d.get(k, default) if isinstance(d, dict) else getattr(d, k, default)
        return default if v is None else v
    if isinstance(lr_scheduler, str) or lr_scheduler is None:
        a = lr_scheduler_args or {}
        total = int(g(a, "total_training_steps", -1))
        total = total if total > 0 else int(fallback_total or 0)
        warm = int(g(a, "lr_warmup_steps", -1))
        if warm < 0:
            warm = int(float(g(a, "lr_warmup_steps_ratio", 0.0)) * total) if total > 0 else 0
        return dict(schedule=str(lr_scheduler or "constant"), warmup_steps=warm, total_steps=total,
                    min_lr_ratio=float(g(a, "min_lr_ratio", 0.0)), min_lr=float(g(a, "min_lr", 0.0)),
                    warmup_init=float(g(a, "lr_warmup_init", 0.0)), num_cycles=float(g(a, "num_cycles", 0.5)),
                    decay_steps=int(g(a, "lr_decay_steps", 0)), wsd_decay_steps=int(g(a, "lr_wsd_decay_steps", 0)),
                    wsd_decay_style=str(g(a, "lr_wsd_decay_style", "exponential")))
    total = int(g(lr_scheduler, "total_steps", 0) or fallback_total or 0)
    warm = int(g(lr_scheduler, "warmup_steps", 0))
    if not warm and g(lr_scheduler, "warmup_ratio", 0.0) and total:
        warm = int(float(g(lr_scheduler, "warmup_ratio")) * total)
    return dict(schedule=str(g(lr_scheduler, "type", "constant")), warmup_steps=warm, total_steps=total,
                min_lr_ratio=float(g(lr_scheduler, "min_lr_ratio", 0.0)))


class _Packing:
    """Index maps between the padded [B,T] view and one packed micro-batch."""

    def __init__(self, input_ids: torch.Tensor, attention_mask: torch.Tensor, device, data: DataProto | None = None):
        lens = attention_mask.sum(1).to(torch.long).cpu().numpy()
        B, T = input_ids.shape
        rows = np.repeat(np.arange(B), lens)
        cols = np.concatenate([np.arange(n) for n in lens]) if B else np.zeros(0, dtype=np.int64)
        self.lens = lens
        self._rows, self._cols = rows, cols
        self.total = int(lens.sum())
        flat = torch.from_numpy(rows * T + cols).to(device)
        ids = input_ids.to(device).reshape(-1)[flat].to(torch.int32)
        starts = np.concatenate([[0], np.cumsum(lens)])
        labels = torch.full((self.total,), -100, dtype=torch.int32, device=device)
        if self.total > 1:
            labels[:-1] = ids[1:]
        last = torch.from_numpy(starts[1:] - 1).to(device)
        labels[last[torch.from_numpy(lens > 0).to(device)]] = -100
        self.batch = PackedBatch(ids, torch.from_numpy(cols.astype(np.int32)).to(device),
                                 torch.from_numpy(starts.astype(np.int32)).to(device), labels,
                                 int(lens.max()) if B else 0)
        # packed position p scores the token at padded index flat[p] + 1 (same row) unless p is a row's last token
        keep = np.ones(self.total, dtype=bool)
        keep[starts[1:][lens > 0] - 1] = False
        self.src = torch.from_numpy(np.nonzero(keep)[0]).to(device)
        self.dst = flat[self.src] + 1
        self.shape = (B, T)
        if data is not None:
            self.batch.multimodal = self._multimodal(data, device)

    def _multimodal(self, data: DataProto, device) -> dict | None:
        """Vision inputs of the rows in packed order: every row's ``multi_modal_inputs`` entry (pixel_values,
        image_grid_thw; videos likewise) concatenated, and the three rotary rows of ``position_ids`` ([B, 3, T], or
        [B, 4, T] with a leading text row) gathered at the packed tokens."""
        mm = data.non_tensor_batch.get("multi_modal_inputs") if data.non_tensor_batch else None
        if mm is None or not any(isinstance(m, dict) and len(m) for m in mm):
            return None
        pix, grids = [], []
        for b, n in enumerate(self.lens):
            m = mm[b] if isinstance(mm[b], dict) else {}
            if n == 0:
                continue
            for pk, gk in (("pixel_values", "image_grid_thw"), ("pixel_values_videos", "video_grid_thw")):
                if m.get(pk) is not None and len(m[pk]):
                    pix.append(torch.as_tensor(m[pk]))
                    grids.append(torch.as_tensor(m[gk]).reshape(-1, 3))
        out = {"pixel_values": torch.cat(pix).to(device) if pix else None,
               "image_grid_thw": torch.cat(grids) if grids else None, "mrope_positions": None}
        pos = data.batch.get("position_ids") if hasattr(data.batch, "get") else None
        if pos is not None and pos.dim() == 3:
            p3 = pos[:, -3:, :]                                  # [B, 3, T]
            out["mrope_positions"] = p3[torch.from_numpy(self._rows), :, torch.from_numpy(self._cols)].t().contiguous().to(device)
        return out

    def to_padded(self, packed: torch.Tensor) -> torch.Tensor:
        out = torch.zeros(self.shape[0] * self.shape[1], dtype=packed.dtype, device=packed.device)
        out = out.index_put((self.dst,), packed[self.src])     # differentiable scatter
        return out.view(self.shape)


class PolicyEngine:
    def __init__(self, model: DenseModel, optim: OptimConfig | None = None, process_group=None,
                 max_token_len_per_gpu: int = 8192, temperature: float = 1.0, fused_zero1: bool | None = None,
                 shard_size: int = -1):
        """``shard_size``: number of ranks the optimizer state (and the reduced gradient) is sharded over.
        -1 or the group size: every data-parallel rank holds 1 / world of it. A divisor S of the group size gives
        hybrid sharding (the reference's ``fsdp.fsdp_size``, axon/utils/fsdp/utils.py:550-573): consecutive ranks
        form shard groups of S, ranks with the same place in their groups are replicas; gradients are
        reduce-scattered inside a shard group and all-reduced across replicas, parameters are gathered inside
        the shard group only, so the wide collectives stay within S ranks."""
        self.model = model
        self.cfg = optim or OptimConfig()
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if (process_group is not None or dist.is_initialized()) else 1
        self.rank = dist.get_rank(process_group) if self.world > 1 else 0
        self.opt_group, self.rep_group = process_group, None
        self.opt_world, self.opt_rank = self.world, self.rank
        if shard_size is not None and 0 < int(shard_size) < self.world:
            S = int(shard_size)
            assert self.world % S == 0, f"shard size {S} must divide the data-parallel size {self.world}"
            ranks = dist.get_process_group_ranks(process_group if process_group is not None else dist.group.WORLD)
            for g in range(self.world // S):                      # every rank creates every group, in the same order
                grp = dist.new_group([ranks[g * S + i] for i in range(S)])
                if g == self.rank // S:
                    self.opt_group = grp
            for i in range(S):
                grp = dist.new_group([ranks[g * S + i] for g in range(self.world // S)])
                if i == self.rank % S:
                    self.rep_group = grp
            self.opt_world, self.opt_rank = S, self.rank % S
            fused_zero1 = False                                   # the peer-memory step reduces over one flat group
        self.max_tokens = max_token_len_per_gpu
        self.mtp_loss_coef = 0.0      # weight of the multi-token-prediction loss (models with such a module)
        self.temperature = temperature
        self.device = model.device
        n = model.params.numel
        per = (n + self.opt_world - 1) // self.opt_world
        per = (per + 127) // 128 * 128
        self.shard = (min(n, self.opt_rank * per), min(n, (self.opt_rank + 1) * per))
        self.shard_size = per
        self.master = self.exp_avg = self.exp_avg_sq = None
        self.opt_step = 0                     # optimizer updates so far (Adam bias correction)
        self.sched_step = 0                   # learning-rate schedule position (advances once per RL step)
        self.state = torch.zeros(4, dtype=torch.float32, device=self.device)
        self._host_state: dict | None = None
        self.fused = None
        mp = self._model_parallel()
        ep = getattr(model, "ep", None) or getattr(model, "shard", None)      # ranks with different data that meet in collectives layer by layer
        self.micro_group = ep.group if (ep is not None and ep.world > 1) else None      # ranks that must run equal micro-batch counts
        if fused_zero1 is None:
            # the fused step computes the clipping norm over the data-parallel group only; a model-parallel
            # group adds terms to the norm, so those runs take the NCCL path with the corrected norm
            fused_zero1 = (mp is None or mp.world == 1) and self.world > 1 and self.device.type == "cuda" and n % (self.world * 128) == 0 and \
                dist.get_backend(process_group) == "nccl"
        if fused_zero1:
            self._enable_fused_zero1()

    def _model_parallel(self):
        """The context of the model's parallel group of any kind (tensor, expert, pipeline, parameter shards)."""
        for attr in ("mp_ctx", "tp", "ep", "pp", "shard"):
            ctx = getattr(self.model, attr, None)
            if ctx is not None:
                return ctx
        return None

    def _enable_fused_zero1(self) -> None:
        """Move the parameters and the main-gradient buffer into symmetric memory and route the
        optimizer step through the peer-memory kernels (reduce via peer loads, AdamW whose epilogue
        stores the new bf16 values into every rank's parameters). Falls back to NCCL collectives when
        symmetric memory cannot be set up."""
        from ..parallel.zero1 import FusedZero1
        p = self.model.params
        try:
            fz = FusedZero1(p.flat.numel(), group=self.pg, device=self.device)
        except Exception as e:          # noqa: BLE001 - no peer access / unsupported driver
            import warnings
            warnings.warn(f"fused ZeRO-1 unavailable ({type(e).__name__}: {e}); using NCCL collectives", stacklevel=2)
            return
        fz.params.tensor.copy_(p.flat)
        p.rebind(fz.params.tensor)
        p.grad_flat, p.grads = None, {}
        p.alloc_grads(grad_flat=fz.grads.tensor)
        p.grads_persistent = True       # symmetric memory is mapped once; rollouts must not free it
        self.fused = fz
        lo, hi = self.shard
        assert (fz.lo, fz.lo + fz.n) == (lo, hi), "shard boundaries of the fused path and the engine differ"

    # ------------------------------------------------------------------ optimizer state
    def init_optimizer(self) -> None:
        lo, hi = self.shard
        self.master = self.model.params.flat[lo:hi].float().clone()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)

    def prepare_offload_buffers(self) -> None:
        """Allocate the pinned host buffers of ``offload_optimizer`` ahead of time."""
        if self._host_state is None and self.master is not None and self.device.type == "cuda":
            self._host_state = {k: torch.empty(v.shape, dtype=v.dtype, pin_memory=True)
                                for k, v in (("master", self.master), ("m", self.exp_avg), ("v", self.exp_avg_sq))}

    def offload_optimizer(self) -> None:
        """Move master / moments to pinned host memory (frees HBM for the KV pool during rollout)."""
        if self.master is None or self.device.type != "cuda":
            return
        if self._host_state is None:
            self._host_state = {k: torch.empty(v.shape, dtype=v.dtype, pin_memory=True)
                                for k, v in (("master", self.master), ("m", self.exp_avg), ("v", self.exp_avg_sq))}
        for k, v in (("master", self.master), ("m", self.exp_avg), ("v", self.exp_avg_sq)):
            self._host_state[k].copy_(v, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.master = self.exp_avg = self.exp_avg_sq = None

    def load_optimizer(self) -> None:
        if self.master is not None or self._host_state is None:
            return
        self.master = self._host_state["master"].to(self.device, non_blocking=True)
        self.exp_avg = self._host_state["m"].to(self.device, non_blocking=True)
        self.exp_avg_sq = self._host_state["v"].to(self.device, non_blocking=True)

    # ------------------------------------------------------------------ forward only
    @torch.no_grad()
    def forward(self, data: DataProto, temperature: float | None = None, want_entropy: bool = True) -> DataProto:
        """Returns a DataProto with ``log_probs`` (and ``entropy``) [B,T] for the rows of ``data``."""
        temp = temperature if temperature is not None else data.meta_info.get("temperature", self.temperature)
        mbs, idx = prepare_dynamic_batch(data, self.max_tokens, dp_group=self.micro_group, strict_equal=self.micro_group is not None)
        lps, ents = [], []
        packs = [_Packing(mb.batch["input_ids"], mb.batch["attention_mask"], self.device, mb) for mb in mbs]
        if hasattr(self.model, "forward_many"):      # pipeline stages: micro-batches stream through the stages
            results = self.model.forward_many([pk.batch for pk in packs], temp)
        else:
            results = (self.model.forward(pk.batch, temp) for pk in packs)
        for pk, (lp, ent) in zip(packs, results):
            lps.append(pk.to_padded(lp))
            ents.append(pk.to_padded(ent))
        order = torch.tensor([i for p in idx for i in p], dtype=torch.long, device=self.device)
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=self.device)
        out = {"log_probs": torch.cat(lps)[inv]}
        if want_entropy:
            out["entropy"] = torch.cat(ents)[inv]
        return DataProto.from_dict(out)

    # ------------------------------------------------------------------ forward + backward
    def forward_backward(self, data: DataProto, loss_fn: str = "ppo", loss_args: dict | None = None) -> dict:
        """Accumulates gradients of the registered loss over token-capped micro-batches. The loss's
        mini-batch-global denominators (``valid_token_count`` ...) must already be on the batch for exact
        multi-micro-batch / multi-rank scaling; gradients are SUMMED across ranks in ``optim_step``."""
        args = dict(loss_args or {})
        temp = data.meta_info.get("temperature", self.temperature)
        ent_coef = float(args.get("entropy_coef", 0.0) or 0.0)
        kl_coef = float(args.get("kl_coef", 0.0) or 0.0)
        self.model.params.alloc_grads()
        # expert-parallel ranks hold different data but exchange tokens layer by layer: equal micro-batch counts
        mbs, _ = prepare_dynamic_batch(data, self.max_tokens, dp_group=self.micro_group, strict_equal=self.micro_group is not None)
        metrics: dict[str, list] = {}

        def loss_step(mb, pk, lp_packed, ent_packed):
            """Loss of one micro-batch from its packed log-probs / entropies: returns their gradients."""
            lp_leaf = lp_packed.detach().requires_grad_(True)
            ent_leaf = ent_packed.detach().requires_grad_(ent_coef != 0.0)
            mb.batch["log_probs"] = pk.to_padded(lp_leaf)
            mb.batch["entropy"] = pk.to_padded(ent_leaf)
            if "old_log_probs" not in mb.batch:      # on-policy: the detached current log-probs
                mb.batch["old_log_probs"] = mb.batch["log_probs"].detach()
            loss, m = compute_loss_fn(mb, loss_fn, args)
            total = loss
            counts = {k: mb.batch.get(k, None) for k in ("valid_token_count", "valid_batch_size",
                                                         "valid_program_count", "per_row_token_count")}
            agg = dict(token_reduce=args.get("token_reduce", "sum"), batch_reduce=args.get("batch_reduce", "token-mean"),
                       num_program_tokens=mb.batch.get("num_program_tokens", None),
                       num_program_steps=mb.batch.get("num_program_steps", None), **counts)
            if ent_coef != 0.0:
                ent_loss = agg_loss(mb.batch["entropy"], mb.batch["response_mask"], **agg)
                total = total - ent_coef * ent_loss
                m["entropy_loss"] = ent_loss.detach().item()
            if kl_coef != 0.0 and "ref_log_probs" in mb.batch:
                from ..utils.rl.kl import kl_penalty
                kld = kl_penalty(mb.batch["log_probs"], mb.batch["ref_log_probs"], args.get("kl_type", "low_var_kl"))
                kl_loss = agg_loss(kld, mb.batch["response_mask"], **agg)
                total = total + kl_coef * kl_loss
                m["kl_loss"] = kl_loss.detach().item()
            total.backward()
            m["loss"] = total.detach().item()
            with torch.no_grad():
                rm = mb.batch["response_mask"]
                m["entropy"] = ((mb.batch["entropy"].detach() * rm).sum() / rm.sum().clamp_min(1)).item()
            for k, v in m.items():
                metrics.setdefault(k, []).append(v)
            return lp_leaf.grad, ent_leaf.grad if ent_coef != 0.0 else None

        mbs = [mb.to(self.device) for mb in mbs]
        mtp = self.mtp_loss_coef > 0 and getattr(self.model.cfg, "num_nextn_predict_layers", 0) > 0 and hasattr(self.model, "mtp_scale")
        if mtp:
            # token-mean over the whole mini-batch (all ranks, all micro-batches): a sequence of n tokens has n - 2 targets
            cnt = sum((mb.batch["attention_mask"].sum(1) - 2).clamp_min(0).sum() for mb in mbs).float().reshape(1)
            if self.world > 1:
                dist.all_reduce(cnt, group=self.pg)
            peers = getattr(self.model, "sum_over_row_peers", None)
            if peers is not None:
                peers(cnt)          # ranks outside the optimizer's group that bring rows of their own (expert-parallel, parameter-sharding peers)
            cnt = cnt / float(getattr(self.model, "same_rows_ranks", 1))     # sequence- / context-parallel peers counted the same rows
            self.model.mtp_scale = self.mtp_loss_coef / max(float(cnt), 1.0)
        packs = [_Packing(mb.batch["input_ids"], mb.batch["attention_mask"], self.device, mb) for mb in mbs]
        if hasattr(self.model, "train_many"):
            # pipeline stages: the model orders forwards and backwards of the micro-batches (1F1B) and calls
            # the loss on the last stage only; its metrics are then handed to the other stages
            self.model.train_many([pk.batch for pk in packs], temp, lambda i, lp, ent: loss_step(mbs[i], packs[i], lp, ent))
            if mtp:
                for nll, n in getattr(self.model, "mtp_records", []):           # filled on the stage that holds the module
                    metrics.setdefault("mtp_loss", []).append(float(nll) / max(float(n), 1.0))
                self.model.mtp_records = []
                self.model.mtp_scale = 0.0
            return self.model.share_from_last(metrics)
        for mb, pk in zip(mbs, packs):
            lp_packed, ent_packed = self.model.forward(pk.batch, temp, save_for_backward=True)
            g_lp, g_ent = loss_step(mb, pk, lp_packed, ent_packed)
            last = self.model.mtp_last if mtp else None        # read once: an adapter sums it over its group
            if last is not None:
                nll, n = last
                metrics.setdefault("mtp_loss", []).append(float(nll) / max(float(n), 1.0))
            self.model.backward(g_lp, g_ent)
        if mtp:
            self.model.mtp_scale = 0.0
        return metrics

    # ------------------------------------------------------------------ value head (critic / reward model)
    @torch.no_grad()
    def forward_values(self, data: DataProto) -> DataProto:
        """``values[b, t]`` = value head on the hidden state BEFORE token t (0 at t = 0), masked by
        ``response_mask`` when present (reference: axon/models/fsdp_models.py:299-372)."""
        mbs, idx = prepare_dynamic_batch(data, self.max_tokens, dp_group=None)
        outs = []
        for mb in mbs:
            pk = _Packing(mb.batch["input_ids"], mb.batch["attention_mask"], self.device)
            outs.append(pk.to_padded(self.model.forward_values(pk.batch)))
        order = torch.tensor([i for p in idx for i in p], dtype=torch.long, device=self.device)
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=self.device)
        values = torch.cat(outs)[inv]
        if "response_mask" in data.batch:
            values = values * data.batch["response_mask"].to(values.device)
        return DataProto.from_dict({"values": values})

    @torch.no_grad()
    def forward_rewards(self, data: DataProto) -> DataProto:
        """Sequence reward = value head on the LAST real token's hidden state, placed at that token."""
        mbs, idx = prepare_dynamic_batch(data, self.max_tokens, dp_group=None)
        outs = []
        for mb in mbs:
            am = mb.batch["attention_mask"].to(self.device)
            pk = _Packing(mb.batch["input_ids"], am, self.device)
            v = self.model.forward_values(pk.batch)
            last_packed = torch.from_numpy(np.cumsum(pk.lens) - 1).to(self.device)
            scores = torch.zeros(am.shape, dtype=torch.float32, device=self.device)
            rows = torch.nonzero(torch.from_numpy(pk.lens > 0).to(self.device)).flatten()
            scores[rows, (am.sum(1) - 1)[rows]] = v[last_packed[rows]]
            outs.append(scores)
        order = torch.tensor([i for p in idx for i in p], dtype=torch.long, device=self.device)
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=self.device)
        return DataProto.from_dict({"rm_scores": torch.cat(outs)[inv]})

    def forward_backward_values(self, data: DataProto, loss_fn: str = "value", loss_args: dict | None = None) -> dict:
        """Critic update: value-head predictions against ``returns`` with the registered value loss."""
        args = dict(loss_args or {})
        self.model.params.alloc_grads()
        mbs, _ = prepare_dynamic_batch(data, self.max_tokens, dp_group=None)
        metrics: dict[str, list] = {}
        for mb in mbs:
            mb = mb.to(self.device)
            pk = _Packing(mb.batch["input_ids"], mb.batch["attention_mask"], self.device)
            v_packed = self.model.forward_values(pk.batch, save_for_backward=True)
            leaf = v_packed.detach().requires_grad_(True)
            mb.batch["vpreds"] = pk.to_padded(leaf) * mb.batch["response_mask"]
            loss, m = compute_loss_fn(mb, loss_fn, args)
            loss.backward()
            self.model.backward_values(leaf.grad if leaf.grad is not None else torch.zeros_like(leaf))
            for k, v in m.items():
                metrics.setdefault(k, []).append(v)
        return metrics

    # ------------------------------------------------------------------ optimizer step
    def optim_step(self, step_lr: bool = True) -> dict:
        """Reduce gradients over the data-parallel group, clip by global norm, fused AdamW on the local
        shard, gather the updated bf16 parameters. Skips the update when the norm is not finite."""
        p = self.model.params
        assert p.grad_flat is not None, "no gradients accumulated"
        for hook in ("sync_replicated_grads", "finalize_grads"):      # model-parallel sums, adapter masks
            if hasattr(self.model, hook):
                getattr(self.model, hook)()
        if self.master is None:
            self.load_optimizer()
            if self.master is None:
                self.init_optimizer()
        lo, hi = self.shard
        if self.fused is not None:
            self.opt_step += 1
            lr = lr_at(self.cfg, self.sched_step + 1)
            if step_lr:
                self.sched_step += 1
            state = self.fused.step(self.master, self.exp_avg, self.exp_avg_sq, lr, self.cfg.beta1, self.cfg.beta2,
                                    self.cfg.eps, self.cfg.weight_decay, self.opt_step, self.cfg.grad_clip,
                                    self.cfg.grad_norm_threshold)
            p.zero_grads()
            st = state.tolist()
            return {"grad_norm": st[1], "lr": lr, "skipped": st[3]}
        if self.world > 1:
            grad_shard = self._reduce_scatter_grads()
        else:
            grad_shard = p.grad_flat[lo:hi]
        if hasattr(self.model, "sync_replicated_grads") and self.world == 1:
            pass        # single data-parallel rank: replicated gradients were summed before the reduce below
        OPT.sumsq(grad_shard, self.state)
        if self.opt_world > 1:
            dist.all_reduce(self.state[:1], group=self.opt_group)
        self._tensor_parallel_norm(grad_shard, lo)
        OPT.clip_coef(self.state, self.cfg.grad_clip, self.cfg.grad_norm_threshold)
        self.opt_step += 1
        lr = lr_at(self.cfg, self.sched_step + 1)
        if step_lr:
            self.sched_step += 1
        OPT.adamw_step(self.master, p.flat[lo:hi], grad_shard, self.exp_avg, self.exp_avg_sq, lr, self.cfg.beta1,
                       self.cfg.beta2, self.cfg.eps, self.cfg.weight_decay, self.opt_step, self.state)
        if self.world > 1:
            self._all_gather_params()
        if hasattr(self.model, "after_optim_step"):      # sharded parameters: tell the peers the new values are in place
            self.model.after_optim_step()
        p.zero_grads()
        st = self.state.tolist()
        return {"grad_norm": st[1], "lr": lr, "skipped": st[3]}

    def _tensor_parallel_norm(self, grad_shard: torch.Tensor, lo: int) -> None:
        """With a tensor-, expert- or pipeline-parallel model the squared norm is the sum over the TP ranks of their sharded
        parameters plus the replicated parameters ONCE: sum_r S_r - (W - 1) * rep, where S_r is rank r's
        full-buffer value and rep the replicated part (equal on every rank)."""
        tp = self._model_parallel()
        if tp is None or tp.world == 1:
            return
        rep = torch.zeros(1, dtype=torch.float32, device=self.device)
        for a, b in self.model.replicated_ranges():
            a2, b2 = max(a, lo) - lo, min(b, lo + grad_shard.numel()) - lo
            if b2 > a2:
                rep += grad_shard[a2:b2].float().pow(2).sum()
        if self.opt_world > 1:
            dist.all_reduce(rep, group=self.opt_group)
        tot = self.state[:1].clone()
        tp.all_reduce_(tot)
        # every replicated parameter appears R times in the sum over the group (R = the group size, or the tensor-parallel
        # size when the group also spans pipeline stages, whose replicated parts differ): keep one of the R
        R = int(getattr(tp, "replication", tp.world))
        rep_all = tp.all_reduce_(rep.clone())
        self.state[:1] = tot - rep_all * ((R - 1) / R)
        if hasattr(self.model, "duplicate_ranges"):       # parameters held by some ranks of the group only (tied embedding on pipeline ends)
            dup = torch.zeros(1, dtype=torch.float32, device=self.device)
            for a, b in self.model.duplicate_ranges():
                a2, b2 = max(a, lo) - lo, min(b, lo + grad_shard.numel()) - lo
                if b2 > a2:
                    dup += grad_shard[a2:b2].float().pow(2).sum()
            if self.opt_world > 1:
                dist.all_reduce(dup, group=self.opt_group)
            tp.all_reduce_(dup)
            self.state[:1] -= dup

    def _padded_flat(self, t: torch.Tensor) -> torch.Tensor:
        need = self.shard_size * self.opt_world
        if t.numel() == need:
            return t
        out = torch.zeros(need, dtype=t.dtype, device=t.device)
        out[: t.numel()] = t
        return out

    def _reduce_scatter_grads(self) -> torch.Tensor:
        g = self._padded_flat(self.model.params.grad_flat)
        out = torch.empty(self.shard_size, dtype=g.dtype, device=g.device)
        if self.opt_world == 1:
            out.copy_(g[: self.shard_size])
        elif dist.get_backend(self.pg) == "gloo":
            dist.all_reduce(g, group=self.opt_group)
            out.copy_(g[self.opt_rank * self.shard_size:(self.opt_rank + 1) * self.shard_size])
        else:
            dist.reduce_scatter_tensor(out, g, group=self.opt_group)
        if self.rep_group is not None:                  # hybrid sharding: sum the shard over the replicas
            dist.all_reduce(out, group=self.rep_group)
        lo, hi = self.shard
        return out[: hi - lo]

    def _all_gather_params(self) -> None:
        p = self.model.params
        lo, hi = self.shard
        if self.opt_world == 1:
            return
        if self.shard_size * self.opt_world == p.flat.numel() and dist.get_backend(self.pg) != "gloo":
            dist.all_gather_into_tensor(p.flat, p.flat[lo:hi], group=self.opt_group)   # in place
            return
        mine = torch.zeros(self.shard_size, dtype=p.flat.dtype, device=p.flat.device)
        mine[: hi - lo] = p.flat[lo:hi]
        full = torch.empty(self.shard_size * self.opt_world, dtype=p.flat.dtype, device=p.flat.device)
        if dist.get_backend(self.pg) == "gloo":
            parts = [torch.empty_like(mine) for _ in range(self.opt_world)]
            dist.all_gather(parts, mine, group=self.opt_group)
            full = torch.cat(parts)
        else:
            dist.all_gather_into_tensor(full, mine, group=self.opt_group)
        p.flat.copy_(full[: p.flat.numel()])
