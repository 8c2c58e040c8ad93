"""Tensor-parallel dense decoder with sequence-parallel activations (Megatron-style layout).

Each of the W ranks of a tensor-parallel group holds, per layer, the rows of the fused QKV and
gate/up projections for its share of the heads / FFN units (column-parallel) and the matching
columns of the attention-output and down projections (row-parallel). Norm weights, the embedding and
the vocabulary head are replicated. The residual stream is sharded along the token dimension: every
rank owns T/W packed tokens, norms and the vocabulary head run on those rows only, and full-length
activations exist only between an all-gather -> GEMM and the following GEMM -> reduce-scatter
(``parallel/tp.TPContext``: both fused with the GEMM over NVLink peer memory on CUDA).

Backward recomputes a layer from its saved local input; there the gathered activations are needed
twice (input gradient and weight gradient), so they are gathered once explicitly. Gradients of the
replicated parameters are partial per rank (local tokens) and are summed over the group by
``sync_replicated_grads`` before the optimizer step.

(reference: axon/trainer/megatron_trainer.py:164-173 with Megatron-Core column/row-parallel linears
and ``sequence_parallel: true``; parameter sharding as in axon/utils/p2p/param_mapper.py.)
"""
from __future__ import annotations

from collections import OrderedDict

import torch

from ..ops import activation as A
from ..ops import attention as AT
from ..ops import gemm as G
from ..ops import lm_head as LM
from ..ops import norm as N
from ..ops import rope as R
from ..parallel.tp import TPContext
from ..utils.p2p.param_mapper import shard_rows, split_kind
from .config import ModelConfig
from .dense import PackedBatch
from .params import FlatParams, param_layout

REPLICATED_KINDS = ("replicated", "vocab")
_SHARD_HEAD = False      # set per model: the untied output head split by vocabulary rows


def _replicated(name: str, shard_head: bool) -> bool:
    if shard_head and name == "lm_head.weight":
        return False
    return split_kind(name) in REPLICATED_KINDS


def tp_param_layout(cfg: ModelConfig, tp: int, tp_rank: int, shard_head: bool = False, ep: int = 1, etp: int = 1) -> "OrderedDict[str, tuple[int, ...]]":
    """Parameter shapes of one rank, in the full model's parameter order. ``ep``: the stacked expert tensors keep
    ``num_experts / ep`` whole experts (which ones does not change the shape); ``etp``: every expert keeps 1 / etp of its
    intermediate units (gate and up rows of ``w13``, columns of ``w2``)."""
    out: OrderedDict[str, tuple[int, ...]] = OrderedDict()
    for name, full in param_layout(cfg).items():
        if split_kind(name) == "expert":
            if name.endswith("w13_weight"):
                out[name] = (full[0] // ep, full[1] // etp, full[2])
            else:
                out[name] = (full[0] // ep, full[1], full[2] // etp)
            continue
        if _replicated(name, shard_head) or tp == 1:
            out[name] = tuple(full)
            continue
        boxes = shard_rows(cfg, name, tp, tp_rank)
        rows = sum(b[1] - b[0] for b in boxes)
        out[name] = (rows, boxes[0][3] - boxes[0][2]) if len(full) > 1 else (rows,)
    return out


def slice_full_param(cfg: ModelConfig, name: str, full: torch.Tensor, tp: int, tp_rank: int, shard_head: bool = False,
                     ep: int = 1, ep_rank: int = 0, etp: int = 1, etp_rank: int = 0) -> torch.Tensor:
    if split_kind(name) == "expert":
        n = full.shape[0] // ep
        part = full[ep_rank * n:(ep_rank + 1) * n]
        if etp > 1 and name.endswith("w13_weight"):
            F = part.shape[1] // 2
            f0, f1 = etp_rank * F // etp, (etp_rank + 1) * F // etp
            part = torch.cat([part[:, f0:f1], part[:, F + f0:F + f1]], dim=1)
        elif etp > 1:
            F = part.shape[2]
            part = part[:, :, etp_rank * F // etp:(etp_rank + 1) * F // etp]
        return part
    if _replicated(name, shard_head) or tp == 1:
        return full
    if full.dim() == 1:
        return torch.cat([full[a:b] for a, b, _, _ in shard_rows(cfg, name, tp, tp_rank)], 0)
    return torch.cat([full[a:b, c:d] for a, b, c, d in shard_rows(cfg, name, tp, tp_rank)], 0)


def pad_packed_batch(batch: PackedBatch, multiple: int) -> tuple[PackedBatch, int]:
    """Append a dummy sequence so that the token count is a multiple of ``multiple`` (labels -100)."""
    T = batch.input_ids.numel()
    pad = (-T) % multiple
    if pad == 0:
        return batch, T
    dev = batch.input_ids.device
    z = lambda n, v, dt: torch.full((n,), v, dtype=dt, device=dev)      # noqa: E731
    rm = getattr(batch, "routermap", None)
    if rm is not None:                       # padding rows replay nothing
        rm = torch.cat([rm, torch.full((pad, *rm.shape[1:]), -1, dtype=rm.dtype, device=rm.device)])
    out = PackedBatch(torch.cat([batch.input_ids, z(pad, 0, batch.input_ids.dtype)]),
                      torch.cat([batch.position_ids, torch.arange(pad, dtype=batch.position_ids.dtype, device=dev)]),
                      torch.cat([batch.cu_seqlens, torch.tensor([T + pad], dtype=batch.cu_seqlens.dtype, device=dev)]),
                      torch.cat([batch.labels, z(pad, -100, batch.labels.dtype)]),
                      max(batch.max_seqlen, pad), routermap=rm)
    pre = getattr(batch, "mtp_inputs", None)         # shifted ids / labels that an outer adapter cut for this rank
    if pre is not None:
        out.mtp_inputs = (torch.cat([pre[0], z(pad, 0, pre[0].dtype)]), torch.cat([pre[1], z(pad, -100, pre[1].dtype)]))
    return out, T


class TPDenseModel:
    SPARSE = False           # the sparse subclass (tp_moe.TPMoEModel) replaces the MLP hooks
    ep_world = 1
    etp_world = 1
    MTP_OK = True

    def __init__(self, cfg: ModelConfig, tp: TPContext, device="cuda", dtype=torch.bfloat16, vocab_parallel_head: bool = False,
                 holds=None):
        """``holds``: optional predicate over parameter names; only those parameters are allocated (pipeline stages)."""
        assert (cfg.num_experts > 0) == self.SPARSE, "dense configurations use TPDenseModel, sparse ones TPMoEModel"
        assert cfg.num_key_value_heads % tp.world == 0 and (self.SPARSE or cfg.intermediate_size % tp.world == 0)
        assert not cfg.sandwich_norm, "sandwich-norm families (GLM-4) run under data / sequence / context / pipeline parallelism; the tensor-parallel layer code does not carry the extra norms yet"
        assert cfg.num_nextn_predict_layers == 0 or self.MTP_OK, \
            "the multi-token-prediction module is not built for context-parallel ranks"
        self.cfg, self.tp = cfg, tp
        self.device, self.dtype = torch.device(device), dtype
        self.shard_head = bool(vocab_parallel_head) and not cfg.tie_word_embeddings and tp.world > 1
        layout = tp_param_layout(cfg, tp.world, tp.rank, self.shard_head, ep=self.ep_world, etp=self.etp_world)
        if holds is not None:
            layout = OrderedDict((n, sh) for n, sh in layout.items() if holds(n))
        self.params = FlatParams(cfg, self.device, dtype, layout=layout)
        self.vp_head = None
        if self.shard_head:
            from ..parallel.vocab_parallel import VocabParallelHead
            self.vp_head = VocabParallelHead(tp, cfg.vocab_size)
        self.hq, self.hkv = cfg.num_attention_heads // tp.world, cfg.num_key_value_heads // tp.world
        self._saved = None
        self.mtp_scale = 0.0          # weight of sum_t(-logprob) of the multi-token-prediction module in backward (0 = module idle)
        self.mtp_last = None          # (sum of negative log-probs, positions) of the latest micro-batch, over the whole group

    # ------------------------------------------------------------------ parameters
    def load_full_state(self, full_views: dict) -> None:
        for name, dst in self.params.views.items():
            dst.copy_(slice_full_param(self.cfg, name, full_views[name], self.tp.world, self.tp.rank, self.shard_head,
                                       ep=self.ep_world, ep_rank=self.tp.rank if self.ep_world > 1 else 0,
                                       etp=self.etp_world, etp_rank=self.tp.rank if self.etp_world > 1 else 0).to(dst.device).to(dst.dtype))

    def init_random(self, std: float = 0.02, seed: int = 0) -> None:
        """Same values as ``FlatParams.init_random`` of the unsharded model with this seed."""
        ref = FlatParams(self.cfg, self.device, self.dtype)
        ref.init_random(std=std, seed=seed)
        self.load_full_state(ref.views)

    def replicated_names(self) -> list[str]:
        return [n for n in self.params.layout if _replicated(n, self.shard_head)]

    def sync_replicated_grads(self) -> None:
        """Sum the partial gradients of replicated parameters over the tensor-parallel group."""
        if self.tp.world == 1 or self.params.grad_flat is None:
            return
        names = self.replicated_names()
        flat = torch.cat([self.params.grads[n].reshape(-1) for n in names])
        self.tp.all_reduce_(flat)
        off = 0
        for n in names:
            g = self.params.grads[n]
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()

    def grad_sumsq(self) -> torch.Tensor:
        """This rank's contribution to the global squared gradient norm: sharded parameters in full,
        replicated ones (identical on every rank after ``sync_replicated_grads``) divided by W."""
        g = self.params.grad_flat
        total = g.double().pow(2).sum()
        if self.tp.world > 1:
            rep = sum(self.params.grads[n].double().pow(2).sum() for n in self.replicated_names())
            total = total - rep * (1.0 - 1.0 / self.tp.world)
        return total

    def _p(self, l, name):
        return self.params[f"model.layers.{l}.{name}"]

    def _g(self, l, name):
        return self.params.grads[f"model.layers.{l}.{name}"]

    def head_weight(self):
        return self.params["model.embed_tokens.weight" if self.cfg.tie_word_embeddings else "lm_head.weight"]

    def head_grad(self):
        return self.params.grads["model.embed_tokens.weight" if self.cfg.tie_word_embeddings else "lm_head.weight"]

    # ------------------------------------------------------------------ one layer
    def _attn(self, l, qkv, batch, tables, need_lse):
        c = self.cfg
        qw = self._p(l, "self_attn.q_norm.weight") if c.qk_norm else None
        kw = self._p(l, "self_attn.k_norm.weight") if c.qk_norm else None
        qkv_r = R.qknorm_rope_fwd(qkv, batch.position_ids, tables[0], tables[1], self.hq, self.hkv, c.head_dim, qw, kw, c.rms_norm_eps)
        o, lse = self._attn_kernel(qkv_r, batch, need_lse)
        return qkv_r, o, lse

    def _attn_kernel(self, qkv_r, batch, need_lse):
        return AT.attn_fwd(qkv_r, batch.cu_seqlens, self.hq, self.hkv, self.cfg.head_dim, need_lse=need_lse)

    def _attn_bwd(self, do, qkv_r, o, lse, batch):
        """Gradient of the attention kernel call of ``_attn`` w.r.t. the rotated q | k | v of this rank's heads."""
        return AT.attn_bwd(do, qkv_r, o, lse, batch.cu_seqlens, self.hq, self.hkv, self.cfg.head_dim)

    def layer_fwd(self, l, x, delta, batch, tables):
        """x (+ delta): local rows [T/W, H] of the stream entering the layer -> (x1, mlp_out, xin), all local rows."""
        c, tp = self.cfg, self.tp
        h, _, xin = N.rmsnorm_fwd(x, self._p(l, "input_layernorm.weight"), c.rms_norm_eps, delta=delta)
        qkv = tp.allgather_gemm(h, self._p(l, "self_attn.qkv_proj.weight"))
        if c.attention_bias:
            qkv += self._p(l, "self_attn.qkv_proj.bias")          # this rank's heads: the bias splits like the rows
        _, o, _ = self._attn(l, qkv, batch, tables, need_lse=False)
        ao = tp.gemm_reduce_scatter(o, self._p(l, "self_attn.o_proj.weight"))
        h2, _, x1 = N.rmsnorm_fwd(xin, self._p(l, "post_attention_layernorm.weight"), c.rms_norm_eps, delta=ao)
        return x1, self._mlp_fwd(l, h2, batch), xin

    def _mlp_fwd(self, l, h2, batch):
        """MLP on this rank's rows h2 [T/W, H] -> [T/W, H]: column-parallel gate / up over all rows, row-parallel down."""
        tp = self.tp
        gu = tp.allgather_gemm(h2, self._p(l, "mlp.gate_up_proj.weight"))
        return tp.gemm_reduce_scatter(A.swiglu_fwd(gu), self._p(l, "mlp.down_proj.weight"))

    def _mlp_bwd(self, l, h2, dx_out, batch):
        """Gradient w.r.t. h2 (local rows) from the gradient of the MLP output (local rows); recomputes the MLP's
        activations and accumulates its weight gradients."""
        tp = self.tp
        h2_full = tp.all_gather_rows(h2)
        gu = G.gemm_nt(h2_full, self._p(l, "mlp.gate_up_proj.weight"))
        a = A.swiglu_fwd(gu)
        dy_full = tp.all_gather_rows(dx_out)                                   # grad of the row-parallel output, all rows
        da = G.gemm_nn(dy_full, self._p(l, "mlp.down_proj.weight"))
        G.gemm_tn(dy_full, a, out=self._g(l, "mlp.down_proj.weight"), accumulate=True)
        dgu = A.swiglu_bwd(da, gu)
        del da, a, gu
        G.gemm_tn(dgu, h2_full, out=self._g(l, "mlp.gate_up_proj.weight"), accumulate=True)
        return tp.gemm_reduce_scatter(dgu, self._p(l, "mlp.gate_up_proj.weight"), w_is_kn=True)

    def layer_bwd(self, l, xin, dx_out, batch, tables):
        c, tp = self.cfg, self.tp
        qw = self._p(l, "self_attn.q_norm.weight") if c.qk_norm else None
        kw = self._p(l, "self_attn.k_norm.weight") if c.qk_norm else None
        # ---- recompute with explicit gathers (the gathered tensors feed both dgrad and wgrad)
        h, rstd1, _ = N.rmsnorm_fwd(xin, self._p(l, "input_layernorm.weight"), c.rms_norm_eps)
        h_full = tp.all_gather_rows(h)
        qkv = G.gemm_nt(h_full, self._p(l, "self_attn.qkv_proj.weight"))
        if c.attention_bias:
            qkv += self._p(l, "self_attn.qkv_proj.bias")
        qkv_r, o, lse = self._attn(l, qkv, batch, tables, need_lse=True)
        ao = tp.gemm_reduce_scatter(o, self._p(l, "self_attn.o_proj.weight"))
        h2, rstd2, x1 = N.rmsnorm_fwd(xin, self._p(l, "post_attention_layernorm.weight"), c.rms_norm_eps, delta=ao)
        # ---- MLP backward
        dh2 = self._mlp_bwd(l, h2, dx_out, batch)
        dx1 = N.rmsnorm_bwd(dh2, x1, self._p(l, "post_attention_layernorm.weight"), rstd2,
                            self._g(l, "post_attention_layernorm.weight"), dres=dx_out)
        # ---- attention backward
        dao_full = tp.all_gather_rows(dx1)
        do = G.gemm_nn(dao_full, self._p(l, "self_attn.o_proj.weight"))
        G.gemm_tn(dao_full, o, out=self._g(l, "self_attn.o_proj.weight"), accumulate=True)
        dqkv_r = self._attn_bwd(do, qkv_r, o, lse, batch)
        dqkv = R.qknorm_rope_bwd(dqkv_r, qkv, batch.position_ids, tables[0], tables[1], self.hq, self.hkv, c.head_dim, qw, kw,
                                 self._g(l, "self_attn.q_norm.weight") if c.qk_norm else None,
                                 self._g(l, "self_attn.k_norm.weight") if c.qk_norm else None, c.rms_norm_eps)
        G.gemm_tn(dqkv, h_full, out=self._g(l, "self_attn.qkv_proj.weight"), accumulate=True)
        if c.attention_bias:
            self._g(l, "self_attn.qkv_proj.bias").add_(dqkv.float().sum(0))      # all rows, own columns: complete on this rank
        dh = tp.gemm_reduce_scatter(dqkv, self._p(l, "self_attn.qkv_proj.weight"), w_is_kn=True)
        return N.rmsnorm_bwd(dh, xin, self._p(l, "input_layernorm.weight"), rstd1, self._g(l, "input_layernorm.weight"), dres=dx1)

    # ------------------------------------------------------------------ whole model
    def local_slice(self, T: int) -> slice:
        n = T // self.tp.world
        return slice(self.tp.rank * n, (self.tp.rank + 1) * n)

    def _trunk_fwd(self, batch: PackedBatch, save: bool):
        """Embedding, layers and final norm on THIS rank's rows -> (hf [T/W, H], state)."""
        c = self.cfg
        self.tp.begin_pass()
        T = batch.input_ids.numel()
        assert T % (128 * self.tp.world) == 0, "pad the batch with pad_packed_batch(batch, 128 * tp)"
        sl = self.local_slice(T)
        tables = R.rope_tables(max(int(batch.max_seqlen) or c.max_position_embeddings, 8), c.head_dim, c.rope_theta, self.device, c.rotary_dim)
        x = A.embedding_fwd(batch.input_ids[sl].contiguous(), self.params["model.embed_tokens.weight"])
        delta, inputs = None, []
        for l in range(c.num_hidden_layers):
            x, delta, xin = self.layer_fwd(l, x, delta, batch, tables)
            if save:
                inputs.append(xin)
        hf, rstd_f, xf = N.rmsnorm_fwd(x, self.params["model.norm.weight"], c.rms_norm_eps, delta=delta)
        return hf, dict(batch=batch, tables=tables, inputs=inputs, xf=xf, hf=hf, rstd_f=rstd_f, sl=sl)

    def _trunk_bwd(self, s: dict, dhf, extra_dx=None) -> None:
        """``extra_dx``: a second gradient w.r.t. the stream before the final norm (the multi-token-prediction module's)."""
        c = self.cfg
        dx = N.rmsnorm_bwd(dhf, s["xf"], self.params["model.norm.weight"], s["rstd_f"], self.params.grads["model.norm.weight"],
                           dres=extra_dx)
        for l in reversed(range(c.num_hidden_layers)):
            dx = self.layer_bwd(l, s["inputs"].pop(), dx, s["batch"], s["tables"])
        A.embedding_bwd(s["batch"].input_ids[s["sl"]].contiguous(), dx, self.params.grads["model.embed_tokens.weight"])

    def forward(self, batch: PackedBatch, temperature: float = 1.0, save_for_backward: bool = False):
        """``batch`` is the full packed batch, its length a multiple of 128 * W (``pad_packed_batch``).
        Returns (log-prob, entropy) of THIS rank's tokens [T/W]."""
        hf, state = self._trunk_fwd(batch, save_for_backward)
        # the parameter gradient of a qk-norm weight is partial per rank (local heads); norms over the
        # hidden size see local tokens only — both are summed by sync_replicated_grads
        labels = batch.labels[state["sl"]].contiguous()
        if self.vp_head is not None:
            lp, ent, head_ctx = self.vp_head.forward(hf, self.head_weight(), batch.labels, temperature)
            lse = None
        else:
            lp, ent, lse = LM.lmhead_fwd(hf, self.head_weight(), labels, temperature)
            head_ctx = None
        if save_for_backward:
            state.update(kind="lm", lse=lse, ent=ent, labels=labels, temperature=temperature, head_ctx=head_ctx)
            if self.cfg.num_nextn_predict_layers > 0 and self.mtp_scale:
                self.mtp_last = self._mtp_fwd(state)
            self._saved = state
        return lp, ent

    # ---- multi-token prediction (depth 1) on this rank's rows; the module's own layer is tensor-parallel like the others,
    # its projection and norms are whole on every rank (``models/mtp.py`` is the data-parallel form and documents the math)
    def _mtp_fwd(self, s: dict):
        from .mtp import shifted_inputs
        assert self.vp_head is None, "the multi-token-prediction module uses the whole output head"
        c, batch, L, sl = self.cfg, s["batch"], self.cfg.num_hidden_layers, s["sl"]
        p, w = f"model.layers.{L}.", self.params
        pre = getattr(batch, "mtp_inputs", None)         # context-parallel ranks: shifted within whole sequences before the cut
        nxt, lab2 = pre if pre is not None else shifted_inputs(batch)
        nxt, lab2 = nxt[sl].contiguous(), lab2[sl].contiguous()
        e = A.embedding_fwd(nxt, w["model.embed_tokens.weight"])
        en, rstd_e, _ = N.rmsnorm_fwd(e, w[p + "enorm.weight"], c.rms_norm_eps)
        hn, rstd_h, _ = N.rmsnorm_fwd(s["xf"], w[p + "hnorm.weight"], c.rms_norm_eps)
        cat = torch.cat([en, hn], dim=1)
        z = G.gemm_nt(cat, w[p + "eh_proj.weight"])
        x2, delta2, xin2 = self.layer_fwd(L, z, None, batch, s["tables"])
        hf2, rstd2, xf2 = N.rmsnorm_fwd(x2, w[p + "shared_head.norm.weight"], c.rms_norm_eps, delta=delta2)
        lp2, ent2, lse2 = LM.lmhead_fwd(hf2, self.head_weight(), lab2, 1.0)
        valid = lab2 >= 0
        s["mtp"] = dict(nxt=nxt, lab2=lab2, e=e, rstd_e=rstd_e, rstd_h=rstd_h, cat=cat, xin2=xin2, hf2=hf2, rstd2=rstd2, xf2=xf2,
                        lse2=lse2, ent2=ent2, valid=valid)
        both = torch.stack([-(lp2.float() * valid).sum(), valid.sum().float()])
        self.tp.all_reduce_(both)                      # every rank reports the group's totals
        return both[0], both[1]

    def _mtp_bwd(self, s: dict, scale: float):
        c, batch, L = self.cfg, s["batch"], self.cfg.num_hidden_layers
        p, w, g, m = f"model.layers.{L}.", self.params, self.params.grads, s.pop("mtp")
        H = c.hidden_size
        dhf2 = LM.lmhead_bwd(m["hf2"], self.head_weight(), m["lab2"], m["lse2"], m["ent2"], (-scale) * m["valid"].float(), None, 1.0,
                             dweight=self.head_grad())
        dx2 = N.rmsnorm_bwd(dhf2, m["xf2"], w[p + "shared_head.norm.weight"], m["rstd2"], g[p + "shared_head.norm.weight"])
        dz = self.layer_bwd(L, m["xin2"], dx2, batch, s["tables"])
        dcat = G.gemm_nn(dz, w[p + "eh_proj.weight"])
        G.gemm_tn(dz, m["cat"], out=g[p + "eh_proj.weight"], accumulate=True)
        den, dhn = dcat[:, :H].contiguous(), dcat[:, H:].contiguous()
        de = N.rmsnorm_bwd(den, m["e"], w[p + "enorm.weight"], m["rstd_e"], g[p + "enorm.weight"])
        A.embedding_bwd(m["nxt"], de, g["model.embed_tokens.weight"])
        return N.rmsnorm_bwd(dhn, s["xf"], w[p + "hnorm.weight"], m["rstd_h"], g[p + "hnorm.weight"])

    def backward(self, g_logprob, g_entropy=None) -> None:
        s = self._saved
        assert s is not None and s.get("kind") == "lm"
        self._saved = None
        self.tp.begin_pass()
        self.params.alloc_grads()
        g_lp = None if g_logprob is None else g_logprob.float().contiguous()
        g_ent = None if g_entropy is None else g_entropy.float().contiguous()
        if s["head_ctx"] is not None:
            dhf = self.vp_head.backward(s["head_ctx"], g_lp, g_ent, dweight=self.head_grad())
        else:
            dhf = LM.lmhead_bwd(s["hf"], self.head_weight(), s["labels"], s["lse"], s["ent"], g_lp, g_ent, s["temperature"],
                                dweight=self.head_grad())
        self._trunk_bwd(s, dhf, self._mtp_bwd(s, float(self.mtp_scale)) if "mtp" in s else None)

    def forward_values(self, batch: PackedBatch, save_for_backward: bool = False) -> torch.Tensor:
        """Scalar value of THIS rank's tokens [T/W] from the value head (``value_head`` in the configuration: the head is
        whole on every rank and its gradient, like a norm's, is partial over the rank's tokens)."""
        hf, state = self._trunk_fwd(batch, save_for_backward)
        values = (hf.float() @ self.params["v_head.weight"].float().t()).squeeze(-1)
        if save_for_backward:
            state["kind"] = "values"
            self._saved = state
        return values

    def backward_values(self, g_values: torch.Tensor) -> None:
        s = self._saved
        assert s is not None and s.get("kind") == "values", "call forward_values(save_for_backward=True) first"
        self._saved = None
        self.tp.begin_pass()
        self.params.alloc_grads()
        g = g_values.float().contiguous()
        w = self.params["v_head.weight"]
        self.params.grads["v_head.weight"].add_(g[None, :] @ s["hf"].float())
        self._trunk_bwd(s, (g[:, None] * w.float()).to(s["hf"].dtype))


class TPModelAdapter:
    """Gives a tensor-parallel model the interface of ``DenseModel`` (full-batch log-probs in, full-batch
    gradients out), so the policy engine and the loss code run unchanged on every TP rank: local
    log-probs are all-gathered over the group, incoming gradients are cut back to the local rows."""

    def __init__(self, model: TPDenseModel):
        self.inner, self.tp = model, model.tp
        self.cfg, self.params, self.device, self.dtype = model.cfg, model.params, model.device, model.dtype
        self.recompute = "full"
        self._T = self._T_real = 0

    def forward(self, batch: PackedBatch, temperature: float = 1.0, save_for_backward: bool = False):
        padded, self._T_real = pad_packed_batch(batch, 128 * self.tp.world)
        self._T = padded.input_ids.numel()
        lp, ent = self.inner.forward(padded, temperature, save_for_backward)
        lp_full = self.tp.all_gather_rows(lp.contiguous())[: self._T_real]
        ent_full = self.tp.all_gather_rows(ent.contiguous())[: self._T_real]
        return lp_full, ent_full

    def backward(self, g_logprob, g_entropy=None) -> None:
        sl = self.inner.local_slice(self._T)

        def cut(g):
            if g is None:
                return None
            full = torch.zeros(self._T, dtype=torch.float32, device=g.device)
            full[: self._T_real] = g.float()
            return full[sl].contiguous()
        self.inner.backward(cut(g_logprob), cut(g_entropy))

    @property
    def mtp_scale(self) -> float:
        return self.inner.mtp_scale

    @mtp_scale.setter
    def mtp_scale(self, v: float) -> None:
        self.inner.mtp_scale = v

    @property
    def mtp_last(self):
        return self.inner.mtp_last

    def forward_values(self, batch: PackedBatch, save_for_backward: bool = False) -> torch.Tensor:
        padded, self._T_real = pad_packed_batch(batch, 128 * self.tp.world)
        self._T = padded.input_ids.numel()
        v = self.inner.forward_values(padded, save_for_backward)
        return self.tp.all_gather_rows(v.contiguous())[: self._T_real]

    def backward_values(self, g_values: torch.Tensor) -> None:
        full = torch.zeros(self._T, dtype=torch.float32, device=g_values.device)
        full[: self._T_real] = g_values.float()
        self.inner.backward_values(full[self.inner.local_slice(self._T)].contiguous())

    def sync_replicated_grads(self) -> None:
        self.inner.sync_replicated_grads()

    def replicated_ranges(self) -> list[tuple[int, int]]:
        return [(o, o + n) for name, (o, n) in self.params.offsets.items() if name in set(self.inner.replicated_names())]

    def flops_per_token(self, seqlen: int) -> float:
        from .dense import DenseModel
        from .moe import MoEModel
        return (MoEModel if self.cfg.num_experts > 0 else DenseModel).flops_per_token(self, seqlen) / self.tp.world
