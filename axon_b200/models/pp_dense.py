"""Pipeline-parallel dense decoder (reference: ``pipeline_model_parallel_size`` of the Megatron trainer,
schedules of ``megatron_forward_backward``, axon/utils/megatron/ - send / recv over NCCL p2p).

The layers are cut into ``P`` contiguous stages; stage 0 also owns the embedding, the last stage the final
norm and the vocabulary head (tied embeddings would need the embedding on both ends and are refused).
Each stage holds only its own parameters, optimizer shards and activations. One micro-batch runs as

    forward :  recv (x, delta) <- prev   ->  local layers  ->  send (x, delta) -> next      last: head -> logprob / entropy
    backward:  recv d(stream)  <- next   ->  local layers  ->  send d(stream)  -> prev      first: embedding gradient

with ``torch.distributed`` point-to-point calls on the stage group (NCCL p2p on GPUs, gloo on CPU), and the
per-token log-probs of the last stage are broadcast to the group, so the loss code runs unchanged on
every stage and hands each one the same upstream gradient (only the last stage consumes it).

Schedule: the policy engine processes micro-batches one after another (forward, loss, backward), so
stages take turns within a micro-batch - this partitions memory P ways but does not overlap stages
across micro-batches; an interleaved (1F1B) schedule needs the engine to keep several micro-batches in
flight and is not built yet.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import lm_head as LM
from ..ops import norm as N
from .config import ModelConfig
from .dense import DenseModel, PackedBatch
from .params import FlatParams, param_layout


def stage_layers(num_layers: int, stages: int, stage: int) -> range:
    """Contiguous layer range of ``stage``; earlier stages take the remainder layers."""
    base, rem = divmod(num_layers, stages)
    lo = stage * base + min(stage, rem)
    return range(lo, lo + base + (1 if stage < rem else 0))


def stage_layout(cfg: ModelConfig, stages: int, stage: int):
    lay = param_layout(cfg)
    keep = {f"model.layers.{l}." for l in stage_layers(cfg.num_hidden_layers, stages, stage)}
    out = type(lay)()
    for name, shape in lay.items():
        if name.startswith("model.layers."):
            if any(name.startswith(p) for p in keep):
                out[name] = shape
        elif name == "model.embed_tokens.weight":
            if stage == 0:
                out[name] = shape
        elif stage == stages - 1:          # final norm, head, value head
            out[name] = shape
    return out


class PipelineContext:
    def __init__(self, group, device):
        live = dist.is_initialized() and group is not None
        self.group, self.device = group, torch.device(device)
        self.world = dist.get_world_size(group) if live else 1
        self.rank = dist.get_rank(group) if live else 0
        self.ranks = dist.get_process_group_ranks(group) if live else [0]

    def send(self, t: torch.Tensor, to_stage: int) -> None:
        dist.send(t.contiguous(), dst=self.ranks[to_stage], group=self.group)

    def recv(self, shape, dtype, from_stage: int) -> torch.Tensor:
        t = torch.empty(shape, dtype=dtype, device=self.device)
        dist.recv(t, src=self.ranks[from_stage], group=self.group)
        return t

    def broadcast_from_last(self, t: torch.Tensor) -> torch.Tensor:
        dist.broadcast(t, src=self.ranks[-1], group=self.group)
        return t

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t


class PPDenseModel(DenseModel):
    def __init__(self, cfg: ModelConfig, pp: PipelineContext, device="cuda", dtype=torch.bfloat16):
        assert cfg.num_experts == 0, "pipeline stages are built for dense models"
        assert not cfg.tie_word_embeddings or pp.world == 1, "tied embeddings cannot be split over pipeline stages"
        assert pp.world <= cfg.num_hidden_layers
        self.pp = pp
        self.stage, self.stages = pp.rank, pp.world
        params = FlatParams(cfg, torch.device(device), dtype, layout=stage_layout(cfg, self.stages, self.stage))
        super().__init__(cfg, device, dtype, params=params)
        self.layers = stage_layers(cfg.num_hidden_layers, self.stages, self.stage)

    @property
    def first(self) -> bool:
        return self.stage == 0

    @property
    def last(self) -> bool:
        return self.stage == self.stages - 1

    def load_full_state(self, full_views: dict) -> None:
        for name, dst in self.params.views.items():
            dst.copy_(full_views[name].to(dst.device).to(dst.dtype))

    def replicated_names(self) -> list[str]:
        return []

    def replicated_ranges(self):
        return []

    # ------------------------------------------------------------------ one micro-batch
    def _stage_fwd(self, batch: PackedBatch, save: bool):
        from ..ops import activation as A
        c = self.cfg
        T, H = batch.input_ids.numel(), c.hidden_size
        tables = self._tables(int(batch.max_seqlen) if batch.max_seqlen else c.max_position_embeddings)
        if self.first:
            x, delta = A.embedding_fwd(batch.input_ids, self.weights["model.embed_tokens.weight"]), None
        else:
            x = self.pp.recv((T, H), self.dtype, self.stage - 1)
            delta = self.pp.recv((T, H), self.dtype, self.stage - 1)
        kept = []
        for l in self.layers:
            x, delta, saved = self.layer_fwd(l, x, delta, batch, tables, keep=save)
            if save:
                kept.append(saved)
        if not self.last:
            self.pp.send(x, self.stage + 1)
            self.pp.send(delta, self.stage + 1)
        return x, delta, dict(batch=batch, tables=tables, layer_inputs=kept)

    def forward(self, batch: PackedBatch, temperature: float = 1.0, save_for_backward: bool = False):
        x, delta, state = self._stage_fwd(batch, save_for_backward)
        T = batch.input_ids.numel()
        if self.last:
            hf, rstd_f, xf = N.rmsnorm_fwd(x, self.weights["model.norm.weight"], self.cfg.rms_norm_eps, delta=delta)
            lp, ent, lse = LM.lmhead_fwd(hf, self.head_weight(), batch.labels, temperature)
            state.update(hf=hf, rstd_f=rstd_f, xf=xf, lse=lse, ent=ent, temperature=temperature)
            both = torch.stack([lp.float(), ent.float()])
        else:
            both = torch.empty(2, T, dtype=torch.float32, device=self.device)
        self.pp.broadcast_from_last(both)
        if save_for_backward:
            state["kind"] = "lm"
            self._saved = state
        return both[0], both[1]

    def backward(self, g_logprob, g_entropy=None) -> None:
        s = self._saved
        assert s is not None and s.get("kind") == "lm", "call forward(save_for_backward=True) first"
        self._saved = None
        self.params.alloc_grads()
        batch, tables = s["batch"], s["tables"]
        T, H = batch.input_ids.numel(), self.cfg.hidden_size
        if self.last:
            g_lp = None if g_logprob is None else g_logprob.float().contiguous()
            g_ent = None if g_entropy is None else g_entropy.float().contiguous()
            dhf = LM.lmhead_bwd(s["hf"], self.head_weight(), batch.labels, s["lse"], s["ent"], g_lp, g_ent,
                                s["temperature"], dweight=self.head_grad())
            dx = N.rmsnorm_bwd(dhf, s["xf"], self.weights["model.norm.weight"], s["rstd_f"], self._wgrad("model.norm.weight"))
        else:
            dx = self.pp.recv((T, H), self.dtype, self.stage + 1)
        kept = s["layer_inputs"]
        for l in reversed(self.layers):
            dx = self.layer_bwd(l, kept.pop(), dx, batch, tables)
        if self.first:
            self._embed_bwd(batch, dx)
        else:
            self.pp.send(dx, self.stage - 1)

    def flops_per_token(self, seqlen: int) -> float:
        return DenseModel.flops_per_token(self, seqlen) / self.stages
