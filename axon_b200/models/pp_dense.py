"""Pipeline-parallel dense decoder (reference: ``pipeline_model_parallel_size`` of the Megatron trainer,
schedules of ``megatron_forward_backward``, axon/utils/megatron/ - send / recv over NCCL p2p).

The layers are cut into ``P`` contiguous stages; stage 0 also owns the embedding, the last stage the final
norm and the vocabulary head (with tied embeddings both ends hold the table and sum its gradient before the optimizer).
Each stage holds only its own parameters, optimizer shards and activations. One micro-batch runs as

    forward :  recv (x, delta) <- prev   ->  local layers  ->  send (x, delta) -> next      last: head -> logprob / entropy
    backward:  recv d(stream)  <- next   ->  local layers  ->  send d(stream)  -> prev      first: embedding gradient

with ``torch.distributed`` point-to-point calls on the stage group (NCCL p2p on GPUs, gloo on CPU), and the
per-token log-probs of the last stage are broadcast to the group, so the loss code runs unchanged on
every stage and hands each one the same upstream gradient (only the last stage consumes it).

Schedules. ``train_many`` runs the micro-batches of a mini-batch one-forward-one-backward: stages overlap
across micro-batches, the loss runs on the last stage only and neighbouring stages swap activation and
gradient in one batched point-to-point step. ``forward_many`` streams forward-only micro-batches.
``forward`` / ``backward`` keep the one-micro-batch interface of the dense model (stages take turns, the
log-probs of the last stage are broadcast so the caller's loss code runs everywhere).
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


def stage_keeps(cfg: ModelConfig, stages: int, stage: int):
    """Predicate over parameter names: does ``stage`` hold this parameter?"""
    keep = tuple(f"model.layers.{l}." for l in stage_layers(cfg.num_hidden_layers, stages, stage))

    def holds(name: str) -> bool:
        if name.startswith("model.layers."):
            return name.startswith(keep) if keep else False
        if name == "model.embed_tokens.weight":
            return stage == 0 or (cfg.tie_word_embeddings and stage == stages - 1)      # tied: the last stage's head reads it too
        return stage == stages - 1         # final norm, head, value head
    return holds


def stage_layout(cfg: ModelConfig, stages: int, stage: int):
    lay = param_layout(cfg)
    holds = stage_keeps(cfg, stages, stage)
    out = type(lay)()
    for name, shape in lay.items():
        if holds(name):
            out[name] = shape
    return out


class PipelineContext:
    def __init__(self, group, device, ends_group=None):
        """``ends_group``: the first and the last stage of this pipeline (they share the tied embedding); with two
        stages that is the pipeline group itself."""
        live = dist.is_initialized() and group is not None
        self.group, self.device = group, torch.device(device)
        self.ends_group = ends_group
        self.world = dist.get_world_size(group) if live else 1
        self.rank = dist.get_rank(group) if live else 0
        self.ranks = dist.get_process_group_ranks(group) if live else [0]

    def send(self, t: torch.Tensor, to_stage: int) -> None:
        dist.send(t.contiguous(), dst=self.ranks[to_stage], group=self.group)

    def recv(self, shape, dtype, from_stage: int) -> torch.Tensor:
        t = torch.empty(shape, dtype=dtype, device=self.device)
        dist.recv(t, src=self.ranks[from_stage], group=self.group)
        return t

    def exchange(self, sends: list, recvs: list) -> list[torch.Tensor]:
        """One batch of point-to-point transfers: ``sends`` = [(tensor, stage)], ``recvs`` = [(shape, dtype,
        stage)]; returns the received tensors. Sends and receives of a batch progress together, so two
        neighbours may each send to the other in the same step without waiting on each other."""
        ops, out = [], []
        for t, to in sends:
            ops.append(dist.P2POp(dist.isend, t.contiguous(), self.ranks[to], self.group))
        for shape, dtype, frm in recvs:
            t = torch.empty(shape, dtype=dtype, device=self.device)
            out.append(t)
            ops.append(dist.P2POp(dist.irecv, t, self.ranks[frm], self.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return out

    def share_object_from_last(self, obj):
        if self.world == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=self.ranks[-1], group=self.group)
        return box[0]

    def broadcast_from_last(self, t: torch.Tensor) -> torch.Tensor:
        dist.broadcast(t, src=self.ranks[-1], group=self.group)
        return t

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t


class PipelineSchedule:
    """The stage-to-stage protocol and the schedules, for any model that provides the pieces of one micro-batch on its
    stage: ``_layers_fwd(batch, inp, save) -> (x, delta, state)``, ``_head_fwd(x, delta, batch, temperature, state) ->
    (logprob, entropy)`` over the whole micro-batch (last stage), ``_state_bwd(state, upstream) -> d(stream) | None`` and
    ``_stream_shape(batch)``; plus ``pp`` (PipelineContext), ``stage``, ``stages``, ``params``, ``device``, ``dtype``."""

    @property
    def first(self) -> bool:
        return self.stage == 0

    @property
    def last(self) -> bool:
        return self.stage == self.stages - 1

    def _recv_fwd(self, batch: PackedBatch):
        if self.first:
            return None
        sh = self._stream_shape(batch)
        return tuple(self.pp.exchange([], [(sh, self.dtype, self.stage - 1)] * 2))

    def _send_fwd(self, x, delta) -> None:
        if not self.last:
            self.pp.exchange([(x, self.stage + 1), (delta, self.stage + 1)], [])

    # ------------------------------------------------------------------ one micro-batch (stages take turns)
    def forward(self, batch: PackedBatch, temperature: float = 1.0, save_for_backward: bool = False):
        x, delta, state = self._layers_fwd(batch, self._recv_fwd(batch), save_for_backward)
        T = batch.input_ids.numel()
        if self.last:
            lp, ent = self._head_fwd(x, delta, batch, temperature, state)
            both = torch.stack([lp.float(), ent.float()])
        else:
            self._send_fwd(x, delta)
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
        if self.last:
            dx = self._state_bwd(s, (g_logprob, g_entropy))
        else:
            dx = self._state_bwd(s, self.pp.exchange([], [(self._stream_shape(s["batch"]), self.dtype, self.stage + 1)])[0])
        if not self.first:
            self.pp.exchange([(dx, self.stage - 1)], [])

    # ------------------------------------------------------------------ many micro-batches (stages overlap)
    @torch.no_grad()
    def forward_many(self, batches: list[PackedBatch], temperature: float = 1.0):
        """Forward only: micro-batches stream through the stages (stage s works on micro-batch i while
        stage s + 1 works on i - 1); the last stage's per-token results reach every stage in one broadcast."""
        outs = []
        for b in batches:
            x, delta, state = self._layers_fwd(b, self._recv_fwd(b), save=False)
            if self.last:
                lp, ent = self._head_fwd(x, delta, b, temperature, state)
                outs.append(torch.stack([lp.float(), ent.float()]))
            else:
                self._send_fwd(x, delta)
        sizes = [b.input_ids.numel() for b in batches]
        both = torch.cat(outs, dim=1) if self.last else torch.empty(2, sum(sizes), dtype=torch.float32, device=self.device)
        self.pp.broadcast_from_last(both)
        return [(part[0], part[1]) for part in both.split(sizes, dim=1)]

    def train_many(self, batches: list[PackedBatch], temperature: float, loss_cb) -> None:
        """One-forward-one-backward schedule over the micro-batches (reference: the non-interleaved
        pipeline schedule behind ``megatron_forward_backward``). Stage s first runs ``P - 1 - s`` forwards,
        then alternates forward / backward - activations of at most ``P - s`` micro-batches are alive - and
        drains the remaining backwards. ``loss_cb(i, logprob, entropy) -> (g_logprob, g_entropy)`` runs on
        the last stage only, right after the forward of micro-batch i."""
        from collections import deque
        self.params.alloc_grads()
        P, s, M = self.stages, self.stage, len(batches)
        warm = min(P - 1 - s, M)
        rest = M - warm
        alive: deque = deque()
        nxt, prv = s + 1, s - 1

        def run_fwd(i, inp):
            x, delta, st = self._layers_fwd(batches[i], inp, save=True)
            if self.last:
                lp, ent = self._head_fwd(x, delta, batches[i], temperature, st)
                st["upstream"] = loss_cb(i, lp, ent)
            alive.append(st)
            return x, delta

        def run_bwd(upstream):
            st = alive.popleft()
            return self._state_bwd(st, st.pop("upstream") if self.last else upstream)

        def grad_recv(i):
            return [] if self.last else [(self._stream_shape(batches[i]), self.dtype, nxt)]

        def act_recv(i):
            return [] if self.first else [(self._stream_shape(batches[i]), self.dtype, prv)] * 2

        for i in range(warm):
            self._send_fwd(*run_fwd(i, self._recv_fwd(batches[i])))
        inp = self._recv_fwd(batches[warm]) if rest > 0 else None
        for j in range(rest):
            i = warm + j
            x, delta = run_fwd(i, inp)
            got = self.pp.exchange([] if self.last else [(x, nxt), (delta, nxt)], grad_recv(j))     # forward out, gradient in
            dx = run_bwd(got[0] if got else None)
            more = j + 1 < rest
            got = self.pp.exchange([] if self.first else [(dx, prv)], act_recv(i + 1) if more else [])   # gradient out, next input in
            inp = tuple(got) if got else None
        for j in range(rest, M):
            got = self.pp.exchange([], grad_recv(j))
            dx = run_bwd(got[0] if got else None)
            if not self.first:
                self.pp.exchange([(dx, prv)], [])
        assert not alive

    def share_from_last(self, obj):
        """Hand a (picklable) result of the last stage to every stage."""
        return self.pp.share_object_from_last(obj)


class PPDenseModel(PipelineSchedule, DenseModel):
    def __init__(self, cfg: ModelConfig, pp: PipelineContext, device="cuda", dtype=torch.bfloat16):
        assert cfg.num_experts == 0, "pipeline stages are built for dense models"
        if cfg.tie_word_embeddings and pp.world > 2 and pp.rank in (0, pp.world - 1):
            assert pp.ends_group is not None, "tied embeddings over more than two stages need the group of the first and the last stage"
        assert pp.world <= cfg.num_hidden_layers
        self.pp = pp
        self.stage, self.stages = pp.rank, pp.world
        params = FlatParams(cfg, torch.device(device), dtype, layout=stage_layout(cfg, self.stages, self.stage))
        super().__init__(cfg, device, dtype, params=params)
        self.layers = stage_layers(cfg.num_hidden_layers, self.stages, self.stage)

    def load_full_state(self, full_views: dict) -> None:
        for name, dst in self.params.views.items():
            dst.copy_(full_views[name].to(dst.device).to(dst.dtype))

    def replicated_names(self) -> list[str]:
        return []

    def replicated_ranges(self):
        return []

    # Tied embeddings: the table lives on the first stage (lookup) and on the last (output head). Both copies start
    # equal, their gradients are summed over the two stages before the optimizer, so they stay equal.
    def _shares_embedding(self) -> bool:
        return self.cfg.tie_word_embeddings and self.stages > 1 and (self.first or self.last)

    def sync_replicated_grads(self) -> None:
        if self._shares_embedding() and self.params.grad_flat is not None:
            group = self.pp.ends_group if self.stages > 2 else self.pp.group
            dist.all_reduce(self.params.grads["model.embed_tokens.weight"], group=group)

    def duplicate_ranges(self) -> list[tuple[int, int]]:
        """Ranges of the flat gradient that another stage holds as well (counted once in the global norm):
        reported by the last stage only."""
        if self._shares_embedding() and self.last:
            o, n = self.params.offsets["model.embed_tokens.weight"]
            return [(o, o + n)]
        return []

    # ------------------------------------------------------------------ the pieces of one micro-batch
    def _layers_fwd(self, batch: PackedBatch, inp, save: bool):
        """``inp`` = (x, delta) from the previous stage, None on the first. Returns (x, delta, state)."""
        from ..ops import activation as A
        c = self.cfg
        tables = self._tables(int(batch.max_seqlen) if batch.max_seqlen else c.max_position_embeddings)
        if self.first:
            x, delta = A.embedding_fwd(batch.input_ids, self.weights["model.embed_tokens.weight"]), None
        else:
            x, delta = inp
        kept = []
        for l in self.layers:
            x, delta, saved = self.layer_fwd(l, x, delta, batch, tables, keep=save)
            if save:
                kept.append(saved)
        return x, delta, dict(batch=batch, tables=tables, layer_inputs=kept)

    def _head_fwd(self, x, delta, batch: PackedBatch, temperature: float, state: dict):
        hf, rstd_f, xf = N.rmsnorm_fwd(x, self.weights["model.norm.weight"], self.cfg.rms_norm_eps, delta=delta)
        lp, ent, lse = LM.lmhead_fwd(hf, self.head_weight(), batch.labels, temperature)
        state.update(hf=hf, rstd_f=rstd_f, xf=xf, lse=lse, ent=ent, temperature=temperature)
        return lp, ent

    def _state_bwd(self, s: dict, upstream):
        """``upstream``: (g_logprob, g_entropy) on the last stage, d(stream) from the next stage otherwise.
        Returns d(stream) for the previous stage (None on the first, which ends in the embedding)."""
        batch, tables = s["batch"], s["tables"]
        if self.last:
            g_logprob, g_entropy = upstream
            g_lp = None if g_logprob is None else g_logprob.float().contiguous()
            g_ent = None if g_entropy is None else g_entropy.float().contiguous()
            dhf = LM.lmhead_bwd(s["hf"], self.head_weight(), batch.labels, s["lse"], s["ent"], g_lp, g_ent,
                                s["temperature"], dweight=self.head_grad())
            dx = N.rmsnorm_bwd(dhf, s["xf"], self.weights["model.norm.weight"], s["rstd_f"], self._wgrad("model.norm.weight"))
        else:
            dx = upstream
        kept = s["layer_inputs"]
        for l in reversed(self.layers):
            dx = self.layer_bwd(l, kept.pop(), dx, batch, tables)
        if self.first:
            self._embed_bwd(batch, dx)
            return None
        return dx

    def _stream_shape(self, batch: PackedBatch):
        return (batch.input_ids.numel(), self.cfg.hidden_size)

    def flops_per_token(self, seqlen: int) -> float:
        return DenseModel.flops_per_token(self, seqlen) / self.stages
