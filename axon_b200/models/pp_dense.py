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


def chunk_layers(num_layers: int, stages: int, stage: int, virtual: int = 1) -> list[range]:
    """Layer ranges of the ``virtual`` model chunks of ``stage``: chunk c is virtual stage ``c * stages + stage`` of
    a pipeline of ``stages * virtual`` virtual stages (interleaved assignment)."""
    return [stage_layers(num_layers, stages * virtual, c * stages + stage) for c in range(virtual)]


def virtual_schedule(stages: int, virtual: int, micro: int, train: bool = True, backward_only: bool = False) -> list[list[tuple]]:
    """The interleaved one-forward-one-backward schedule of every rank as lock-step ticks.

    Forwards visit the micro-batches in groups of ``stages`` and, inside a group, chunk after chunk; backwards visit the
    chunks in reverse (reference: the interleaved schedule behind ``virtual_pipeline_model_parallel_size``,
    axon/utils/megatron/pipeline_parallel.py). A rank prefers a backward whose upstream gradient has arrived; else it
    runs its next forward whose input has arrived, as long as it holds the activations of fewer than
    ``2 (stages - 1 - rank) + (virtual - 1) stages + 1`` forwards (``stages - rank`` with one chunk) - the warm-up depth
    of that schedule, which bounds activation memory. "Arrived" means produced in an EARLIER tick: everything produced
    in a tick is exchanged at the end of that tick, so the send of one rank and the receive of its neighbour always sit
    in the same batch of point-to-point operations. If the bound ever blocks every rank (micro-batch counts that are
    not a multiple of ``stages``), it is lifted for that tick.

    Returns ``ticks[t][rank] = (kind, micro-batch, chunk) | None``; every rank computes the same table."""
    P, v, M = stages, virtual, micro
    K = P * v
    fwd = [(m, c) for g0 in range(0, M, P) for c in range(v) for m in range(g0, min(g0 + P, M))]
    bwd = [(m, c) for g0 in range(0, M, P) for c in reversed(range(v)) for m in range(g0, min(g0 + P, M))]
    want_f = not backward_only
    want_b = train or backward_only
    done_f = set() if want_f else {(m, k) for m in range(M) for k in range(K)}
    done_b: set = set()
    todo_f = [list(fwd) if want_f else [] for _ in range(P)]
    todo_b = [list(bwd) if want_b else [] for _ in range(P)]
    held = [0] * P
    cap = [((P - r - 1) * 2 + (v - 1) * P if v > 1 else P - 1 - r) + 1 for r in range(P)]
    ticks = []

    def pick(r, bounded):
        for m, c in todo_b[r]:
            k = c * P + r
            if (m, k) in done_f and (k == K - 1 or (m, k + 1) in done_b):
                return ("B", m, c)
        if todo_f[r] and (not bounded or not want_b or held[r] < cap[r]):
            m, c = todo_f[r][0]                  # forwards strictly in order: the receiver's inputs arrive in order too
            k = c * P + r
            if k == 0 or (m, k - 1) in done_f:
                return ("F", m, c)
        return None

    while any(todo_f[r] or todo_b[r] for r in range(P)):
        step = [pick(r, True) for r in range(P)]
        if not any(step):
            step = [pick(r, False) for r in range(P)]
        assert any(step), f"pipeline schedule stalls (stages={P}, virtual={v}, micro-batches={M})"
        for r, op in enumerate(step):
            if op is None:
                continue
            kind, m, c = op
            if kind == "F":
                done_f.add((m, c * P + r))
                todo_f[r].remove((m, c))
                held[r] += 1
            else:
                done_b.add((m, c * P + r))
                todo_b[r].remove((m, c))
                held[r] -= 1
        ticks.append(step)
    return ticks


def stage_keeps(cfg: ModelConfig, stages: int, stage: int, virtual: int = 1):
    """Predicate over parameter names: does ``stage`` hold this parameter?"""
    keep = tuple(f"model.layers.{l}." for rng in chunk_layers(cfg.num_hidden_layers, stages, stage, virtual) for l in rng)
    L = cfg.num_hidden_layers
    after = tuple(f"model.layers.{l}." for l in range(L, L + cfg.num_nextn_predict_layers))      # multi-token-prediction modules

    def holds(name: str) -> bool:
        if name.startswith("model.layers."):
            if after and name.startswith(after):
                return stage == stages - 1         # they read the stream that enters the final norm
            return name.startswith(keep) if keep else False
        if name == "model.embed_tokens.weight":
            # tied: the last stage's head reads it too; so does a prediction module, which embeds the next token
            return stage == 0 or ((cfg.tie_word_embeddings or bool(after)) and stage == stages - 1)
        return stage == stages - 1         # final norm, head, value head
    return holds


def stage_layout(cfg: ModelConfig, stages: int, stage: int, virtual: int = 1):
    lay = param_layout(cfg)
    holds = stage_keeps(cfg, stages, stage, virtual)
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

    vpp = 1          # model chunks per rank (interleaved / virtual pipeline stages); > 1 runs the tick engine below

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

    # ------------------------------------------------------------------ interleaved (virtual) stages
    def _run_ticks(self, batches, ticks, temperature: float, loss_cb=None, save: bool = True, states: dict | None = None,
                   collect: dict | None = None) -> dict:
        """Execute this rank's column of a ``virtual_schedule`` table. A forward of virtual stage k hands (x, delta) to
        the rank after this one (the last rank wraps around to the first, whose next chunk continues), a backward hands
        d(stream) to the rank before; both travel in the ONE batch of point-to-point operations that ends the tick, in
        which the receiving rank has posted the matching receive. ``states``: (micro-batch, chunk) -> saved forward
        state; ``collect``: micro-batch -> (log-prob, entropy) on the rank that holds the head."""
        P, r, v = self.stages, self.stage, self.vpp
        K = P * v
        inbox: dict = {}
        states = {} if states is None else states
        for step in ticks:
            sends, op = [], step[r]
            if op is not None:
                kind, m, c = op
                k = c * P + r
                if kind == "F":
                    x, delta, st = self._layers_fwd(batches[m], None if k == 0 else inbox.pop(("F", m, k)), save, chunk=c)
                    if k == K - 1:
                        lp, ent = self._head_fwd(x, delta, batches[m], temperature, st)
                        if loss_cb is not None:
                            st["upstream"] = loss_cb(m, lp, ent)
                        if collect is not None:
                            collect[m] = (lp, ent)
                    else:
                        sends += [(x, (r + 1) % P), (delta, (r + 1) % P)]
                    if save:
                        states[(m, c)] = st
                else:
                    st = states.pop((m, c))
                    dx = self._state_bwd(st, st.pop("upstream") if k == K - 1 else inbox.pop(("B", m, k)))
                    if k > 0:
                        sends.append((dx, (r - 1) % P))
            recvs, keys = [], []
            for q, oq in enumerate(step):              # what the other ranks produced for this one in this tick
                if oq is None or q == r:
                    continue
                kind, m, c = oq
                k = c * P + q
                shape = self._stream_shape(batches[m])
                if kind == "F" and k < K - 1 and (q + 1) % P == r:
                    recvs += [(shape, self.dtype, q)] * 2
                    keys.append(("F", m, k + 1, 2))
                elif kind == "B" and k > 0 and (q - 1) % P == r:
                    recvs.append((shape, self.dtype, q))
                    keys.append(("B", m, k - 1, 1))
            got = self.pp.exchange(sends, recvs) if (sends or recvs) else []
            at = 0
            for kind, m, k, n in keys:
                inbox[(kind, m, k)] = tuple(got[at:at + n]) if n == 2 else got[at]
                at += n
        assert not inbox, "activations or gradients were left undelivered"
        return states

    # ------------------------------------------------------------------ one micro-batch (stages take turns)
    def forward(self, batch: PackedBatch, temperature: float = 1.0, save_for_backward: bool = False):
        if self.vpp > 1:
            T, got = batch.input_ids.numel(), {}
            states = self._run_ticks([batch], virtual_schedule(self.stages, self.vpp, 1, train=False), temperature,
                                     save=save_for_backward, collect=got)
            both = torch.stack([got[0][0].float(), got[0][1].float()]) if self.last else torch.empty(2, T, dtype=torch.float32, device=self.device)
            self.pp.broadcast_from_last(both)
            if save_for_backward:
                self._saved = {"kind": "lm", "states": states, "batch": batch}
            return both[0], both[1]
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
        if self.vpp > 1:
            if self.last:
                s["states"][(0, self.vpp - 1)]["upstream"] = (g_logprob, g_entropy)
            self._run_ticks([s["batch"]], virtual_schedule(self.stages, self.vpp, 1, backward_only=True), 1.0, states=s["states"])
            return
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
        if self.vpp > 1:
            got: dict = {}
            self._run_ticks(batches, virtual_schedule(self.stages, self.vpp, len(batches), train=False), temperature, save=False, collect=got)
            sizes = [b.input_ids.numel() for b in batches]
            both = torch.cat([torch.stack([got[i][0].float(), got[i][1].float()]) for i in range(len(batches))], dim=1) if self.last \
                else torch.empty(2, sum(sizes), dtype=torch.float32, device=self.device)
            self.pp.broadcast_from_last(both)
            return [(part[0], part[1]) for part in both.split(sizes, dim=1)]
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
        if self.vpp > 1:
            left = self._run_ticks(batches, virtual_schedule(self.stages, self.vpp, len(batches)), temperature, loss_cb=loss_cb)
            assert not left
            return
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
    serves_sampler = False       # a stage holds a slice of the layers: a colocated sampler keeps weights of its own

    def __init__(self, cfg: ModelConfig, pp: PipelineContext, device="cuda", dtype=torch.bfloat16, virtual: int = 1):
        """``virtual``: model chunks per rank. With v > 1 rank r holds the layers of virtual stages r, P + r, 2 P + r, ...
        of a pipeline of P v virtual stages and the schedule interleaves them (a smaller pipeline bubble for the same
        number of micro-batches, more point-to-point traffic)."""
        assert cfg.num_experts == 0, "pipeline stages are built for dense models"
        assert virtual == 1 or pp.world > 1, "virtual stages need at least two pipeline ranks"
        if (cfg.tie_word_embeddings or cfg.num_nextn_predict_layers > 0) and pp.world > 2 and pp.rank in (0, pp.world - 1):
            assert pp.ends_group is not None, "an embedding held by the first and the last of more than two stages needs the group of the two"
        assert pp.world * virtual <= cfg.num_hidden_layers, "every (virtual) stage needs at least one layer"
        self.pp = pp
        self.mtp_records: list = []       # (sum of negative log-probs, targets) of the prediction module per micro-batch, last stage
        self.stage, self.stages, self.vpp = pp.rank, pp.world, int(virtual)
        params = FlatParams(cfg, torch.device(device), dtype, layout=stage_layout(cfg, self.stages, self.stage, self.vpp))
        super().__init__(cfg, device, dtype, params=params)
        self.chunks = chunk_layers(cfg.num_hidden_layers, self.stages, self.stage, self.vpp)
        self.layers = self.chunks[0]

    def load_full_state(self, full_views: dict) -> None:
        for name, dst in self.params.views.items():
            dst.copy_(full_views[name].to(dst.device).to(dst.dtype))

    def replicated_names(self) -> list[str]:
        return []

    def replicated_ranges(self):
        return []

    # Tied embeddings: the table lives on the first stage (lookup) and on the last (output head). Both copies start
    # equal, their gradients are summed over the two stages before the optimizer, so they stay equal. A multi-token-
    # prediction module (on the last stage) looks the next token up in the same table, tied or not.
    def _shares_embedding(self) -> bool:
        c = self.cfg
        return (c.tie_word_embeddings or c.num_nextn_predict_layers > 0) and self.stages > 1 and (self.first or self.last)

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
    def _layers_fwd(self, batch: PackedBatch, inp, save: bool, chunk: int = 0):
        """``inp`` = (x, delta) from the previous (virtual) stage, None on the very first. Returns (x, delta, state)."""
        from ..ops import activation as A
        c = self.cfg
        tables = self._tables(int(batch.max_seqlen) if batch.max_seqlen else c.max_position_embeddings)
        very_first, very_last = self.first and chunk == 0, self.last and chunk == self.vpp - 1
        if very_first:
            x, delta = A.embedding_fwd(batch.input_ids, self.weights["model.embed_tokens.weight"]), None
        else:
            x, delta = inp
        kept = []
        for l in self.chunks[chunk]:
            x, delta, saved = self.layer_fwd(l, x, delta, batch, tables, keep=save)
            if save:
                kept.append(saved)
        return x, delta, dict(batch=batch, tables=tables, layer_inputs=kept, layers=self.chunks[chunk], very_first=very_first,
                              very_last=very_last)

    def _head_fwd(self, x, delta, batch: PackedBatch, temperature: float, state: dict):
        hf, rstd_f, xf = N.rmsnorm_fwd(x, self.weights["model.norm.weight"], self.cfg.rms_norm_eps, delta=delta)
        lp, ent, lse = LM.lmhead_fwd(hf, self.head_weight(), batch.labels, temperature)
        state.update(hf=hf, rstd_f=rstd_f, xf=xf, lse=lse, ent=ent, temperature=temperature)
        if self.cfg.num_nextn_predict_layers > 0 and self.mtp_scale:       # the engine sets the scale for training passes only
            from .mtp import mtp_fwd
            self.mtp_last = mtp_fwd(self, state)
            self.mtp_records.append(self.mtp_last)
        return lp, ent

    def _state_bwd(self, s: dict, upstream):
        """``upstream``: (g_logprob, g_entropy) on the last stage, d(stream) from the next stage otherwise.
        Returns d(stream) for the previous stage (None on the first, which ends in the embedding)."""
        batch, tables = s["batch"], s["tables"]
        if s["very_last"]:
            g_logprob, g_entropy = upstream
            g_lp = None if g_logprob is None else g_logprob.float().contiguous()
            g_ent = None if g_entropy is None else g_entropy.float().contiguous()
            dhf = LM.lmhead_bwd(s["hf"], self.head_weight(), batch.labels, s["lse"], s["ent"], g_lp, g_ent,
                                s["temperature"], dweight=self.head_grad())
            extra = None
            if "mtp" in s:
                from .mtp import mtp_bwd
                extra = mtp_bwd(self, s, float(self.mtp_scale))
            dx = N.rmsnorm_bwd(dhf, s["xf"], self.weights["model.norm.weight"], s["rstd_f"], self._wgrad("model.norm.weight"), dres=extra)
        else:
            dx = upstream
        kept = s["layer_inputs"]
        for l in reversed(s["layers"]):
            dx = self.layer_bwd(l, kept.pop(), dx, batch, tables)
        if s["very_first"]:
            self._embed_bwd(batch, dx)
            return None
        return dx

    def _stream_shape(self, batch: PackedBatch):
        return (batch.input_ids.numel(), self.cfg.hidden_size)

    def flops_per_token(self, seqlen: int) -> float:
        return DenseModel.flops_per_token(self, seqlen) / self.stages
