"""Checkpoints of a model-parallel trainer (reference: ``MegatronStateManager``,
axon/utils/state/megatron_state_manager.py:177-473 - sharded state through megatron's dist_checkpointing,
HF export through the bridge's ``save_weights``).

Sharded state goes to ``<path>/dist_ckpt/`` in the layout-independent array store of ``dist_checkpoint.py``:
every parameter is one array in full-model coordinates to which each tensor- / expert- / pipeline-parallel rank
contributes its boxes, so the parameters load under ANY other (tp, ep, pp, dp) layout; the fp32 master weights
and Adam moments are flat per model-parallel rank and load under any data-parallel size of the same
model-parallel layout (under another one the masters are rebuilt from the parameters and the moments start at
zero, with a warning). ``model_parallel_config.json`` names the layout the checkpoint was written under.
Checkpoints in the older per-rank layout (``model_world_size_W_rank_R.pt``) are still read.

HF export: tensor- and expert-parallel shards are gathered over the model-parallel group and re-assembled
with the same row / column boxes the weight-sync planner uses (``utils/p2p/param_mapper.shard_rows``), then
written once in the HuggingFace layout - the checkpoint a sampler, another framework or a differently
sharded run can load.
"""
from __future__ import annotations

import json
import os
import warnings

import torch
import torch.distributed as dist

from ..p2p.param_mapper import shard_rows
from .dist_checkpoint import AsyncSaveRequest, ShardedObject, ShardedTensor, load_sharded, read_metadata, save_sharded
from .fsdp_state_manager import FSDPStateManager, _barrier
from .utils import delete_oldest_checkpoints


def view2d(name: str, shape) -> tuple[int, int]:
    """The two-dimensional view in which a parameter's shards are boxes. Stacked down projections of the experts
    ``[E, H, F]`` are seen as ``[E H, F]`` - whole experts AND column slices of every expert (expert tensor parallelism)
    are then single boxes; everything else as ``[dim 0, the rest]``."""
    if name.endswith("w2_weight") and len(shape) == 3:
        return int(shape[0]) * int(shape[1]), int(shape[2])
    return int(shape[0]), int(torch.Size(shape[1:]).numel()) if len(shape) > 1 else 1


def expert_boxes(name: str, shape, ep: int, ep_rank: int, etp: int, etp_rank: int) -> list:
    """Boxes ((row, column), (rows, columns)) in ``view2d`` coordinates of the part of a stacked expert tensor held by
    one rank: experts ``[e0, e1)`` of the expert-parallel split, and of each of them the slice ``[f0, f1)`` of the
    expert's intermediate units (rows of gate and of up in ``w13``, columns of ``w2``)."""
    E = int(shape[0])
    e0, e1 = ep_rank * E // ep, (ep_rank + 1) * E // ep
    if name.endswith("w2_weight"):
        H, F = int(shape[1]), int(shape[2])
        f0, f1 = etp_rank * F // etp, (etp_rank + 1) * F // etp
        return [((e0 * H, f0), ((e1 - e0) * H, f1 - f0))]
    F2, H = int(shape[1]), int(shape[2])
    if etp == 1:
        return [((e0, 0), (e1 - e0, F2 * H))]
    F = F2 // 2
    f0, f1 = etp_rank * F // etp, (etp_rank + 1) * F // etp
    return [b for e in range(e0, e1) for b in (((e, f0 * H), (1, (f1 - f0) * H)), ((e, (F + f0) * H), (1, (f1 - f0) * H)))]


def gather_full_params(model, group, tp: int = 1, tp_rank: int = 0, ep: int = 1, ep_rank: int = 0, replicated_names=()):
    """Full (unsharded) tensors of every parameter on every rank of ``group`` (CPU, model dtype).
    ``model`` holds this rank's shards in ``model.params`` under the full model's names."""
    from ...models.params import param_layout
    cfg, local = model.cfg, model.params
    world = dist.get_world_size(group) if group is not None else 1
    full_layout = param_layout(cfg)
    out = {}
    rep = set(replicated_names)
    for name, full_shape in full_layout.items():
        mine = local[name].detach()
        if world == 1 or tuple(mine.shape) == tuple(full_shape):
            out[name] = mine.cpu().clone()
            continue
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine.contiguous(), group=group)
        full = torch.empty(full_shape, dtype=mine.dtype)
        flat2d = full.reshape(full_shape[0], -1) if len(full_shape) > 1 else full.reshape(-1, 1)
        for r, part in enumerate(parts):
            boxes = shard_rows(cfg, name, tp, r if tp > 1 else 0, ep, r if ep > 1 else 0, rep)
            p2 = part.cpu().reshape(-1, boxes[0][3] - boxes[0][2])
            row = 0
            for (r0, r1, c0, c1) in boxes:
                flat2d[r0:r1, c0:c1] = p2[row:row + (r1 - r0)]
                row += r1 - r0
        out[name] = full
    return out


class MegatronStateManager(FSDPStateManager):
    def __init__(self, model, optimizer, mp_group=None, tp: int = 1, ep: int = 1, pp: int = 1, dp_rank: int = 0,
                 tp_rank: int | None = None, etp: int = 1, **kw):
        """``tp_rank``: this rank's place in its tensor-parallel group when that differs from its place in ``mp_group``
        (tensor parallelism inside pipeline stages, where ``mp_group`` is the whole tensor x pipeline block)."""
        super().__init__(model, optimizer, **kw)
        self.mp_group, self.tp, self.ep, self.pp, self.dp_rank = mp_group, tp, ep, pp, dp_rank
        self.etp = int(etp)           # ranks over which every expert's intermediate units are divided (the tensor-parallel group)
        self.tp_rank = tp_rank
        self._request: AsyncSaveRequest | None = None

    def _mp_rank(self) -> int:
        return dist.get_rank(self.mp_group) if self.mp_group is not None else 0

    def wait(self) -> None:
        super().wait()
        if self._request is not None:
            req, self._request = self._request, None
            req.finalize()

    # ------------------------------------------------------------------ sharded arrays
    def _inner(self):
        return getattr(self.model, "inner", self.model)

    def _layout_tag(self) -> str:
        v = int(getattr(self._inner(), "vpp", 1) or 1)        # interleaved chunks change which layers a pipeline rank holds
        return f"tp{self.tp}_ep{self.ep}{f'_etp{self.etp}' if self.etp > 1 else ''}_pp{self.pp}{f'v{v}' if v > 1 else ''}_mp{self._mp_rank()}"

    def _param_entries(self) -> dict:
        """key -> ShardedTensor for the parameters this rank holds, in full-model coordinates."""
        from ...models.params import param_layout
        inner = self._inner()
        cfg = inner.cfg
        full = param_layout(cfg)
        rep = set(inner.replicated_names()) if hasattr(inner, "replicated_names") else set()
        r = self.tp_rank if self.tp_rank is not None else self._mp_rank()
        out = {}
        for name, mine in inner.params.views.items():
            shape = full[name]
            g2 = view2d(name, shape)
            zshard = getattr(self.model, "shard", None)
            if name.endswith(("w13_weight", "w2_weight")) and len(shape) == 3:       # stacked experts: whole ones and / or slices of each
                boxes = expert_boxes(name, shape, self.ep, r if self.ep > 1 else 0, self.etp, r if self.etp > 1 else 0)
                writer = self.dp_rank == 0 and (self.ep > 1 or self.etp > 1 or ((self.pp > 1 and self.tp == 1) or r == 0))
            elif tuple(mine.shape) == tuple(shape):          # whole tensor on this rank (a stage's own, or replicated in its group)
                boxes = [((0, 0), g2)]
                one_of_group = (self.pp > 1 and self.tp == 1) or (r == 0 and (zshard is None or zshard.rank == 0))
                writer = self.dp_rank == 0 and one_of_group
            elif zshard is not None and self.tp == 1 and self.ep == 1:    # row shards of the parameter-sharded data-parallel model
                boxes = [((zshard.rank * int(mine.shape[0]), 0), (int(mine.shape[0]), g2[1]))]
                writer = True
            else:
                rows = shard_rows(cfg, name, self.tp, r if self.tp > 1 else 0, self.ep, r if self.ep > 1 else 0, rep)
                boxes = [((r0, c0), (r1 - r0, c1 - c0)) for (r0, r1, c0, c1) in rows]
                writer = self.dp_rank == 0
            out["model/" + name] = ShardedTensor("model/" + name, mine.detach(), g2, boxes, 0 if writer else 1)
        return out

    def full_named_tensors(self):
        """(name, whole tensor) of every parameter of the model, on EVERY rank of the model-parallel group, one tensor
        at a time - for a colocated sampler that does not share the trainer's layout (the reference materialises every
        parameter out of its sharded trainer the same way, axon/sampler/mixins/sync_mixin.py:86-168). Which rank holds
        which box of which tensor is exchanged once; then every box travels in one broadcast from the rank that would
        write it into a checkpoint. A collective: every rank of the group iterates it to the end."""
        from ...models.params import param_layout
        inner = self._inner()
        full_layout = param_layout(inner.cfg)
        mine = self._param_entries()
        group = self.mp_group
        world = dist.get_world_size(group) if group is not None else 1
        if world == 1:
            for name in full_layout:
                yield name, inner.params[name].detach()
            return
        if getattr(self, "_gather_table", None) is None:
            note = {k: (tuple(e.global_shape), [tuple(map(tuple, b)) for b in e.boxes], e.replica_id == 0) for k, e in mine.items()}
            table = [None] * world
            dist.all_gather_object(table, note, group=group)
            self._gather_table = table
        ranks = dist.get_process_group_ranks(group)
        me = dist.get_rank(group)
        dev, dtype = inner.params.flat.device, inner.params.flat.dtype
        for name, shape in full_layout.items():
            key = "model/" + name
            full2d = None
            for r, note in enumerate(self._gather_table):
                ent = note.get(key)
                if ent is None or not ent[2]:
                    continue
                g2, boxes, _ = ent
                if full2d is None:
                    full2d = torch.empty(g2, dtype=dtype, device=dev)
                local = mine[key].data.detach().reshape(-1) if r == me else None
                at = 0
                for (r0, c0), (nr, nc) in boxes:
                    piece = local[at:at + nr * nc].reshape(nr, nc).contiguous() if r == me else torch.empty(nr, nc, dtype=dtype, device=dev)
                    dist.broadcast(piece, src=ranks[r], group=group)
                    full2d[r0:r0 + nr, c0:c0 + nc] = piece
                    at += nr * nc
            assert full2d is not None, f"no rank of the group writes '{name}'"
            yield name, full2d.reshape(shape)

    def _optim_entries(self) -> dict:
        eng = self.optimizer
        lo, hi = eng.shard
        n = int(self.model.params.flat.numel())
        tag = self._layout_tag()
        out = {}
        for part in ("master", "exp_avg", "exp_avg_sq"):
            t = getattr(eng, part)
            if t is not None:
                key = f"optimizer/{tag}/{part}"
                out[key] = ShardedTensor.slice_1d(key, t, n, lo)
        return out

    def save_state(self, local_path: str, global_step: int = 0, max_ckpt_to_keep: int | None = None,
                   save_mode: str | None = None, async_save: bool | None = None):
        if local_path is None:
            return
        self.wait()
        want_hf = save_mode in ("hf", "both")
        os.makedirs(local_path, exist_ok=True)
        _barrier(None)
        eng = self.optimizer
        eng.load_optimizer()
        state = {}
        state.update(self._param_entries())
        state.update(self._optim_entries())
        state["extra/common"] = ShardedObject("extra/common", {"opt_step": eng.opt_step, "sched_step": getattr(eng, "sched_step", eng.opt_step),
                                                               "global_step": global_step}, replica_id=self.rank)
        state[f"extra/rng_rank{self.rank}"] = ShardedObject(f"extra/rng_rank{self.rank}", self.get_rng_state())
        # manifests and barriers span ALL ranks of the job (the optimizer's group is one data-parallel replica set only)
        req = save_sharded(state, os.path.join(local_path, "dist_ckpt"), group=None, async_save=bool(async_save))
        if self.rank == 0:
            with open(os.path.join(local_path, "model_parallel_config.json"), "w") as f:
                json.dump({"tensor_model_parallel_size": self.tp, "expert_model_parallel_size": self.ep,
                           "pipeline_model_parallel_size": self.pp, "world_size": self.world_size, "layout": "dist_ckpt",
                           "param_shards": getattr(getattr(self.model, "shard", None), "world", 1)}, f, indent=1)
            hf_dir = os.path.join(local_path, "huggingface")
            os.makedirs(hf_dir, exist_ok=True)
            if not want_hf:
                self._inner().cfg.save_pretrained(hf_dir)
        if async_save:
            self._request = req            # finalized by wait(): before the next save, a load, or shutdown
        elif max_ckpt_to_keep and max_ckpt_to_keep > 0 and self.rank == 0:
            delete_oldest_checkpoints(os.path.dirname(os.path.dirname(os.path.abspath(local_path))), max_ckpt_to_keep)
        if want_hf and ((self.tp > 1 and self.pp > 1) or self.etp > 1):
            # shards of two kinds: assemble the export from the array store just written (any layout reads back whole)
            req.finalize()
            self._request = None
            if self.rank == 0:
                from ...models.params import FlatParams
                from ..hf_model import save_hf_model
                inner = self._inner()
                host = FlatParams(inner.cfg, "cpu", inner.params.flat.dtype)
                load_sharded({"model/" + n: ShardedTensor("model/" + n, v, view2d(n, v.shape), [((0, 0), view2d(n, v.shape))])
                              for n, v in host.views.items()}, os.path.join(local_path, "dist_ckpt"), group=False)
                save_hf_model(host, os.path.join(local_path, "huggingface"), cfg=inner.cfg, tokenizer=self.processing_class)
            _barrier(None)
            return
        if want_hf and self.dp_rank == 0:
            inner = getattr(self.model, "inner", self.model)
            rep = inner.replicated_names() if hasattr(inner, "replicated_names") else ()
            r = self._mp_rank()
            if hasattr(inner, "gather_full"):      # the model knows how its shards make up the full tensors
                full = inner.gather_full()
            elif self.pp > 1:          # stages hold disjoint parameters: collect them by name
                stages = [None] * self.pp
                dist.all_gather_object(stages, {n: v.detach().cpu() for n, v in inner.params.views.items()}, group=self.mp_group)
                full = {n: v for d in stages for n, v in d.items()}
            else:
                full = gather_full_params(inner, self.mp_group, self.tp, r if self.tp > 1 else 0, self.ep, r if self.ep > 1 else 0, rep)
            if r == 0:
                from ...models.params import FlatParams
                from ..hf_model import save_hf_model
                host = FlatParams(inner.cfg, "cpu", inner.params.flat.dtype)
                for name, v in host.views.items():
                    v.copy_(full[name])
                save_hf_model(host, os.path.join(local_path, "huggingface"), cfg=inner.cfg, tokenizer=self.processing_class)

    def load_state(self, local_path: str, save_mode: str | None = None):
        if local_path is None:
            return
        self.wait()
        dist_dir = os.path.join(local_path, "dist_ckpt")
        if not os.path.exists(os.path.join(dist_dir, "metadata.json")):
            return self._load_per_rank_files(local_path)
        meta = read_metadata(dist_dir)
        eng = self.optimizer
        eng.load_optimizer()
        template = dict(self._param_entries())
        optim = self._optim_entries()
        same_mp = all(k in meta["tensors"] and tuple(meta["tensors"][k]["global_shape"]) == tuple(v.global_shape) for k, v in optim.items())
        if same_mp:
            template.update(optim)
        template["extra/common"] = ShardedObject("extra/common", None)
        rng_key = f"extra/rng_rank{self.rank}"
        if rng_key in meta["objects"]:
            template[rng_key] = ShardedObject(rng_key, None)
        objs = load_sharded(template, dist_dir, group=None)
        if not same_mp:
            warnings.warn(f"{local_path}: optimizer state was written under another model-parallel layout than {self._layout_tag()}; "
                          "master weights are rebuilt from the parameters and the Adam moments start at zero", stacklevel=2)
            lo, hi = eng.shard
            eng.master.copy_(self.model.params.flat[lo:hi].float())
            eng.exp_avg.zero_()
            eng.exp_avg_sq.zero_()
        common = objs.get("extra/common") or {}
        eng.opt_step = int(common.get("opt_step", eng.opt_step))
        if hasattr(eng, "sched_step"):
            eng.sched_step = int(common.get("sched_step", eng.opt_step))
        if rng_key in objs:
            self.load_rng_state(objs[rng_key])
        _barrier(None)

    def _load_per_rank_files(self, local_path: str):
        cfg_file = os.path.join(local_path or "", "model_parallel_config.json")
        if local_path and os.path.exists(cfg_file):
            with open(cfg_file) as f:
                c = json.load(f)
            assert (c["tensor_model_parallel_size"], c["expert_model_parallel_size"], c.get("pipeline_model_parallel_size", 1),
                    c["world_size"]) == (self.tp, self.ep, self.pp, self.world_size), \
                f"checkpoint was written with layout {c}, this run has tp={self.tp} ep={self.ep} pp={self.pp} world={self.world_size}; " \
                f"load its huggingface/ export instead"
        return super().load_state(local_path, "sharded")
