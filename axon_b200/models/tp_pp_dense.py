"""Tensor parallelism INSIDE pipeline stages: ``world = dp x pp x tp`` (reference: the Megatron trainer initialises
tensor-, pipeline- and data-parallel sizes together, axon/trainer/megatron_trainer.py:164-173; its quick-start recipe
runs TP 4 x PP 2).

A stage holds the tensor-parallel shards of its own layers (``tp_dense.TPDenseModel`` restricted by
``pp_dense.stage_keeps``); the residual stream that travels between stages is the sequence-parallel local part
[T / tp, H], so every tensor-parallel rank talks to the same rank of the neighbouring stage and the point-to-point
volume per rank drops by tp. The schedules (one micro-batch, streamed forward, one-forward-one-backward) are those of
``pp_dense.PipelineSchedule``. The last stage's per-token results are gathered over its tensor-parallel group, so the
loss code sees whole micro-batches, and the incoming gradients are cut back to the local rows.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import activation as A
from ..ops import lm_head as LM
from ..ops import norm as N
from ..ops import rope as R
from ..parallel.tp import TPContext
from .config import ModelConfig
from .dense import DenseModel, PackedBatch
from .pp_dense import PipelineContext, PipelineSchedule, chunk_layers, stage_keeps
from .tp_dense import TPDenseModel, pad_packed_batch


class BlockContext:
    """The model-parallel block (all tensor-parallel ranks of all stages of one replica) as the policy engine sees it:
    gradient-norm pieces are summed over ``group``; parameters replicated inside a tensor-parallel group appear
    ``replication`` times in that sum."""

    def __init__(self, group, world: int, replication: int):
        self.group, self.world, self.replication = group, world, replication

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t


class TPPPDenseModel(PipelineSchedule, TPDenseModel):
    def __init__(self, cfg: ModelConfig, tp: TPContext, pp: PipelineContext, block_group=None, device="cuda", dtype=torch.bfloat16,
                 virtual: int = 1):
        """``virtual``: model chunks per pipeline rank (interleaved stages, as in ``pp_dense.PPDenseModel``)."""
        assert pp.world * virtual <= cfg.num_hidden_layers, "every (virtual) stage needs at least one layer"
        assert virtual == 1 or pp.world > 1
        if (cfg.tie_word_embeddings or cfg.num_nextn_predict_layers > 0) and pp.world > 2 and pp.rank in (0, pp.world - 1):
            assert pp.ends_group is not None, "an embedding held by the first and the last of more than two stages needs the group of the two"
        self.pp = pp
        self.mtp_records: list = []       # (sum of negative log-probs, targets) of the prediction module per micro-batch, last stage
        self.stage, self.stages, self.vpp = pp.rank, pp.world, int(virtual)
        TPDenseModel.__init__(self, cfg, tp, device=device, dtype=dtype, vocab_parallel_head=False,
                              holds=stage_keeps(cfg, self.stages, self.stage, self.vpp))
        self.chunks = chunk_layers(cfg.num_hidden_layers, self.stages, self.stage, self.vpp)
        self.layers = self.chunks[0]
        self.mp_ctx = BlockContext(block_group, tp.world * pp.world, tp.world)
        self.recompute = "full"

    # ------------------------------------------------------------------ parameters shared between ranks
    def _shares_embedding(self) -> bool:
        c = self.cfg             # tied head, or a multi-token-prediction module: both read the table on the last stage
        return (c.tie_word_embeddings or c.num_nextn_predict_layers > 0) and self.stages > 1 and (self.first or self.last)

    def sync_replicated_grads(self) -> None:
        TPDenseModel.sync_replicated_grads(self)            # norms / embedding / head: partial per tensor-parallel rank
        if self._shares_embedding() and self.params.grad_flat is not None:
            group = self.pp.ends_group if self.stages > 2 else self.pp.group
            dist.all_reduce(self.params.grads["model.embed_tokens.weight"], group=group)

    def replicated_ranges(self) -> list[tuple[int, int]]:
        keep = set(self.replicated_names())
        return [(o, o + n) for name, (o, n) in self.params.offsets.items() if name in keep]

    def duplicate_ranges(self) -> list[tuple[int, int]]:
        # the tied table also lives on the first stage: counted once more by ONE rank of the last stage
        if self._shares_embedding() and self.last and self.tp.rank == 0:
            o, n = self.params.offsets["model.embed_tokens.weight"]
            return [(o, o + n)]
        return []

    # ------------------------------------------------------------------ the pieces of one micro-batch
    def _padded_len(self, batch: PackedBatch) -> int:
        m = 128 * self.tp.world
        return (batch.input_ids.numel() + m - 1) // m * m

    def _stream_shape(self, batch: PackedBatch):
        return (self._padded_len(batch) // self.tp.world, self.cfg.hidden_size)

    def _layers_fwd(self, batch: PackedBatch, inp, save: bool, chunk: int = 0):
        c = self.cfg
        self.tp.begin_pass()
        very_first, very_last = self.first and chunk == 0, self.last and chunk == self.vpp - 1
        padded, t_real = pad_packed_batch(batch, 128 * self.tp.world)
        T = padded.input_ids.numel()
        sl = self.local_slice(T)
        tables = R.rope_tables(max(int(padded.max_seqlen) or c.max_position_embeddings, 8), c.head_dim, c.rope_theta, self.device, c.rotary_dim)
        if very_first:
            x, delta = A.embedding_fwd(padded.input_ids[sl].contiguous(), self.params["model.embed_tokens.weight"]), None
        else:
            x, delta = inp
        inputs = []
        for l in self.chunks[chunk]:
            x, delta, xin = self.layer_fwd(l, x, delta, padded, tables)
            if save:
                inputs.append(xin)
        return x, delta, dict(batch=padded, tables=tables, inputs=inputs, sl=sl, T=T, T_real=t_real, layers=self.chunks[chunk],
                              very_first=very_first, very_last=very_last)

    def _head_fwd(self, x, delta, batch: PackedBatch, temperature: float, state: dict):
        hf, rstd_f, xf = N.rmsnorm_fwd(x, self.params["model.norm.weight"], self.cfg.rms_norm_eps, delta=delta)
        labels = state["batch"].labels[state["sl"]].contiguous()
        lp, ent, lse = LM.lmhead_fwd(hf, self.head_weight(), labels, temperature)
        state.update(hf=hf, rstd_f=rstd_f, xf=xf, lse=lse, ent=ent, labels=labels, temperature=temperature)
        if self.cfg.num_nextn_predict_layers > 0 and self.mtp_scale:       # the engine sets the scale for training passes only
            self.mtp_last = self._mtp_fwd(state)
            self.mtp_records.append(self.mtp_last)
        n = state["T_real"]
        return self.tp.all_gather_rows(lp.contiguous())[:n], self.tp.all_gather_rows(ent.contiguous())[:n]

    def _cut(self, g, s):
        if g is None:
            return None
        full = torch.zeros(s["T"], dtype=torch.float32, device=self.device)
        full[: s["T_real"]] = g.float()
        return full[s["sl"]].contiguous()

    def _state_bwd(self, s: dict, upstream):
        self.tp.begin_pass()
        batch, tables = s["batch"], s["tables"]
        if s["very_last"]:
            g_lp, g_ent = self._cut(upstream[0], s), self._cut(upstream[1], s)
            dhf = LM.lmhead_bwd(s["hf"], self.head_weight(), s["labels"], s["lse"], s["ent"], g_lp, g_ent, s["temperature"],
                                dweight=self.head_grad())
            extra = self._mtp_bwd(s, float(self.mtp_scale)) if "mtp" in s else None
            dx = N.rmsnorm_bwd(dhf, s["xf"], self.params["model.norm.weight"], s["rstd_f"], self.params.grads["model.norm.weight"],
                               dres=extra)
        else:
            dx = upstream
        kept = s["inputs"]
        for l in reversed(s["layers"]):
            dx = self.layer_bwd(l, kept.pop(), dx, batch, tables)
        if s["very_first"]:
            A.embedding_bwd(batch.input_ids[s["sl"]].contiguous(), dx, self.params.grads["model.embed_tokens.weight"])
            return None
        return dx

    def flops_per_token(self, seqlen: int) -> float:
        from .moe import MoEModel
        return (MoEModel if self.cfg.num_experts > 0 else DenseModel).flops_per_token(self, seqlen) / (self.stages * self.tp.world)


class TPPPMoEModel(TPPPDenseModel):
    """Sparse decoder with tensor + expert parallelism over one group INSIDE pipeline stages (``world = dp x pp x tp``,
    ``ep == tp``): the stage model above with the MLP of ``tp_moe.TPMoEModel`` - every rank routes its own T / tp rows of
    the stream through the expert-parallel dispatch of its stage's group. The expert choice of a micro-batch is kept
    with its saved state, because several micro-batches are in flight between a forward and its backward.
    (reference: the Qwen3-30B-A3B recipe trains with pipeline 2 x tensor 4 x expert 4,
    recipes/math/train_polaris_qwen_30b_a3b.sh.)"""
    SPARSE = True

    def __init__(self, cfg: ModelConfig, tp: TPContext, ep, pp: PipelineContext, block_group=None, device="cuda", dtype=torch.bfloat16,
                 virtual: int = 1):
        """``ep``: an ``EPContext`` over the stage's tensor-parallel ranks, or None for expert TENSOR parallelism (every rank
        of the stage keeps a slice of every expert of the stage's layers)."""
        if ep is not None:
            assert ep.world == tp.world and ep.rank == tp.rank, "experts are divided over the tensor-parallel group's own ranks"
            assert cfg.num_experts % tp.world == 0, f"{cfg.num_experts} experts do not divide over {tp.world} ranks"
            self.ep = ep if ep.world > 1 else None
            self.ep_world = ep.world
        else:
            assert cfg.moe_intermediate_size % tp.world == 0, f"expert width {cfg.moe_intermediate_size} does not divide over {tp.world} ranks"
            self.ep = None
            self.etp_world = tp.world
        super().__init__(cfg, tp, pp, block_group, device=device, dtype=dtype, virtual=virtual)
        self.params.expert_offset = tp.rank * (cfg.num_experts // tp.world) if self.ep_world > 1 else 0
        self.capture_routing, self.last_routing = False, None
        self._ids: dict = {}

    def _layers_fwd(self, batch: PackedBatch, inp, save: bool, chunk: int = 0):
        self._ids = {}
        x, delta, state = super()._layers_fwd(batch, inp, save, chunk)
        if save:
            state["moe_ids"] = self._ids
        return x, delta, state

    def _state_bwd(self, s: dict, upstream):
        self._ids = s["moe_ids"]
        return super()._state_bwd(s, upstream)


def _borrow_sparse_mlp() -> None:
    from .tp_moe import TPMoEModel
    for name in ("_route", "_experts", "_combine", "_moe_rebuild", "_moe_bwd", "_replay_local", "_mlp_fwd", "_mlp_bwd",
                 "_etp_experts", "_etp_fwd", "_etp_bwd"):
        setattr(TPPPMoEModel, name, getattr(TPMoEModel, name))


_borrow_sparse_mlp()
