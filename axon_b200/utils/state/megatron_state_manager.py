"""Checkpoints of a model-parallel trainer (reference: ``MegatronStateManager``,
axon/utils/state/megatron_state_manager.py:177-473 - sharded state through megatron's dist_checkpointing,
HF export through the bridge's ``save_weights``).

Sharded files: every rank writes its slice of ITS OWN flat parameter buffer and its optimizer shard
(``model_world_size_W_rank_R.pt`` ... as the data-parallel manager does), plus ``model_parallel_config.json``
naming the (tp, ep) layout the files were written under; resuming needs the same layout.

HF export: tensor- and expert-parallel shards are gathered over the model-parallel group and re-assembled
with the same row / column boxes the weight-sync planner uses (``utils/p2p/param_mapper.shard_rows``), then
written once in the HuggingFace layout - the checkpoint a sampler, another framework or a differently
sharded run can load.
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

from ..p2p.param_mapper import shard_rows
from .fsdp_state_manager import FSDPStateManager


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
    def __init__(self, model, optimizer, mp_group=None, tp: int = 1, ep: int = 1, pp: int = 1, dp_rank: int = 0, **kw):
        super().__init__(model, optimizer, **kw)
        self.mp_group, self.tp, self.ep, self.pp, self.dp_rank = mp_group, tp, ep, pp, dp_rank

    def _mp_rank(self) -> int:
        return dist.get_rank(self.mp_group) if self.mp_group is not None else 0

    def save_state(self, local_path: str, global_step: int = 0, max_ckpt_to_keep: int | None = None,
                   save_mode: str | None = None, async_save: bool | None = None):
        if local_path is None:
            return
        want_hf = save_mode in ("hf", "both")
        # the sharded part (and rotation, async writing) is the data-parallel manager's; HF export is done here
        super().save_state(local_path, global_step, max_ckpt_to_keep, "sharded", async_save)
        if self.rank == 0:
            with open(os.path.join(local_path, "model_parallel_config.json"), "w") as f:
                json.dump({"tensor_model_parallel_size": self.tp, "expert_model_parallel_size": self.ep,
                           "pipeline_model_parallel_size": self.pp, "world_size": self.world_size,
                           "param_shards": getattr(getattr(self.model, "shard", None), "world", 1)}, f, indent=1)
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
        cfg_file = os.path.join(local_path or "", "model_parallel_config.json")
        if local_path and os.path.exists(cfg_file):
            with open(cfg_file) as f:
                c = json.load(f)
            assert (c["tensor_model_parallel_size"], c["expert_model_parallel_size"], c.get("pipeline_model_parallel_size", 1),
                    c["world_size"]) == (self.tp, self.ep, self.pp, self.world_size), \
                f"checkpoint was written with layout {c}, this run has tp={self.tp} ep={self.ep} pp={self.pp} world={self.world_size}; " \
                f"load its huggingface/ export instead"
        return super().load_state(local_path, "sharded")
