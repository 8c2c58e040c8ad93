"""Sparse mixture-of-experts decoder (Qwen3-MoE family: softmax router, top-k, optional weight
renormalisation, SwiGLU experts, no shared expert).

Attention, norms, embedding and the vocabulary head are the dense model's; only the MLP differs:

    logits = h2 @ gate^T                     (fp32)
    ids, w = route(logits)                   top-k of softmax; with routing replay the ids come from
                                             the sampler's record and only the weights are recomputed
    xs     = gather(h2)                      expert-sorted, 128-row padded
    ys     = W2_e . swiglu(W13_e . xs)       two grouped tcgen05 GEMMs
    out    = sum_j w_j * ys[row(t, j)]       weights applied AFTER the second projection, as the
                                             sampler does, so trainer and sampler agree bit-for-bit
                                             on the order of operations

Backward recomputes the expert activations from what forward kept (``recompute`` as in the dense
model; "none" also keeps the gate/up output). Router gradients flow through the softmax weights of
the selected experts; the selection itself is not differentiated. Replaces the reference's fused-MoE
autograd functions (axon/utils/kernel/fused_moe.py:66-352), the Megatron MoE layer with its routing
replay and probability-placement patches (axon/monkey_patches/megatron/moe_replay.py,
moe_prob_placement.py) and the HF fused block (axon/models/transformers/qwen3_moe.py).
"""
from __future__ import annotations

import torch

from ..ops import activation as A
from ..ops import gemm as G
from ..ops import moe as M
from .config import ModelConfig
from .dense import DenseModel, PackedBatch


class MoEModel(DenseModel):
    def __init__(self, cfg: ModelConfig, device="cuda", dtype=torch.bfloat16, params=None, ep=None):
        """``ep``: an ``EPContext`` — every rank then holds only its E/W experts (``w13`` / ``w2`` have a
        leading dimension of E/W) and tokens reach their experts through peer memory."""
        assert cfg.num_experts > 0 and cfg.num_experts_per_tok > 0, "MoEModel needs num_experts / num_experts_per_tok"
        self.ep = ep if (ep is not None and ep.world > 1) else None
        if self.ep is not None and params is None:
            from .params import FlatParams, param_layout
            lay = param_layout(cfg)
            for n, shp in list(lay.items()):
                if n.endswith("w13_weight") or n.endswith("w2_weight"):
                    lay[n] = (shp[0] // self.ep.world, *shp[1:])
            params = FlatParams(cfg, torch.device(device), dtype, layout=lay)
        super().__init__(cfg, device, dtype, params)
        self.last_routing: list | None = None       # per layer ids of the latest sampler forward (routed-experts capture)
        self.capture_routing = False

    def load_full_state(self, full_views: dict) -> None:
        """Copy from an unsharded model's views, keeping only this rank's experts."""
        for name, dst in self.params.views.items():
            src = full_views[name]
            if self.ep is not None and (name.endswith("w13_weight") or name.endswith("w2_weight")):
                src = src[self.ep.local_experts()]
            dst.copy_(src.to(dst.device).to(dst.dtype))

    def replicated_names(self) -> list[str]:
        """Parameters every expert-parallel rank holds in full (everything but the experts): their
        gradients are partial per rank (local tokens) and are summed over the group before the step."""
        return [n for n in self.params.layout if not (n.endswith("w13_weight") or n.endswith("w2_weight"))]

    def replicated_ranges(self) -> list[tuple[int, int]]:
        """Contiguous [a, b) ranges of the flat buffers that hold replicated parameters (merged)."""
        if self.ep is None:
            return []
        keep = set(self.replicated_names())
        spans = sorted((o, o + n) for name, (o, n) in self.params.offsets.items() if name in keep)
        out: list[list[int]] = []
        for a, b in spans:
            if out and out[-1][1] == a:
                out[-1][1] = b
            else:
                out.append([a, b])
        return [(a, b) for a, b in out]

    def sum_over_row_peers(self, t: torch.Tensor) -> torch.Tensor:
        """The ranks of an expert-parallel group train on different rows (unlike tensor-parallel peers) and are not in the
        optimizer's group: a count over the rows of a mini-batch is completed here."""
        return self.ep.all_reduce_(t) if self.ep is not None else t

    def sync_replicated_grads(self) -> None:
        """Sum the gradients of the replicated parameters over the expert-parallel group (each rank saw
        only its own tokens); expert gradients are already complete for the group, since every token
        routed to an expert was computed on the expert's owner."""
        if self.ep is None or self.params.grad_flat is None:
            return
        for a, b in self.replicated_ranges():
            self.ep.all_reduce_(self.params.grad_flat[a:b])

    # ------------------------------------------------------------------ routing
    def _route(self, l: int, h2, replay):
        c = self.cfg
        logits = G.gemm_nt(h2, self._p(l, "mlp.gate.weight"), out_dtype=torch.float32)
        ids, w = M.route(logits, c.num_experts_per_tok, c.norm_topk_prob, replay)
        return logits, ids, w

    def _experts(self, l: int, h2, ids, w, keep_gu: bool):
        c = self.cfg
        if self.ep is not None:
            lay = self.ep.align(ids)
            xs = self.ep.dispatch(h2, lay)
            gu = M.grouped_fwd(xs, self._p(l, "mlp.experts.w13_weight"), lay.owner)
            a = A.swiglu_fwd(gu)
            ys = M.grouped_fwd(a, self._p(l, "mlp.experts.w2_weight"), lay.owner)
            return lay, xs, gu, a, ys
        lay = M.align(ids, c.num_experts)
        xs = M.gather(h2, lay)
        gu = M.grouped_fwd(xs, self._p(l, "mlp.experts.w13_weight"), lay)
        a = A.swiglu_fwd(gu)
        ys = M.grouped_fwd(a, self._p(l, "mlp.experts.w2_weight"), lay)
        return lay, xs, gu, a, ys

    def _combine(self, ys, w, lay):
        return self.ep.combine(ys, w, lay) if self.ep is not None else M.combine(ys, w, lay)

    def _replay_for(self, l: int, batch):
        rm = getattr(batch, "routermap", None) if batch is not None else None
        if rm is None or l >= rm.shape[1]:          # the record covers the decoder layers, not a prediction module behind them
            return None
        return rm[:, l, :].contiguous()

    # ------------------------------------------------------------------ hooks
    def mlp_fwd(self, l: int, h2, batch: PackedBatch, want=()):
        logits, ids, w = self._route(l, h2, self._replay_for(l, batch))
        lay, xs, gu, a, ys = self._experts(l, h2, ids, w, "gu" in want)
        out = self._combine(ys, w, lay)
        if self.capture_routing:
            if self.last_routing is None:
                self.last_routing = []
            self.last_routing.append(ids)
        saved = {"moe_ids": ids} if want else {}
        if "gu" in want and self.ep is None:       # with expert parallelism the buffers are shared workspaces: recompute
            saved.update(moe_gu=gu, moe_lay=lay, moe_xs=xs)
        return out, saved

    def mlp_infer(self, l: int, h2):
        return self.mlp_fwd(l, h2, None, ())[0]

    def mlp_rebuild(self, l: int, k: dict, batch: PackedBatch) -> None:
        c = self.cfg
        h2 = k["h2"]
        logits = G.gemm_nt(h2, self._p(l, "mlp.gate.weight"), out_dtype=torch.float32)
        ids = k["moe_ids"]
        k["moe_logits"] = logits
        k["moe_w"] = M.route_weights_from_probs(logits, ids, c.norm_topk_prob)
        if "moe_gu" in k:
            lay, xs, gu = k["moe_lay"], k["moe_xs"], k["moe_gu"]
            a = A.swiglu_fwd(gu)
            ys = M.grouped_fwd(a, self._p(l, "mlp.experts.w2_weight"), lay)
        else:
            lay, xs, gu, a, ys = self._experts(l, h2, ids, None, False)
            if self.ep is not None:
                xs = xs.clone()            # the dispatch buffer is reused before the weight gradient needs it
        k.update(moe_lay=lay, moe_xs=xs, moe_gu=gu, moe_a=a, moe_ys=ys)

    def mlp_bwd(self, l: int, k: dict, dx_out):
        c = self.cfg
        lay, xs, gu, a, ys = k["moe_lay"], k["moe_xs"], k["moe_gu"], k["moe_a"], k["moe_ys"]
        w = k["moe_w"]
        if self.ep is not None:
            dys, dw = self.ep.combine_bwd(dx_out, ys, w.detach(), lay)
            glay = lay.owner
        else:
            dys, dw = M.combine_bwd(dx_out, ys, w.detach(), lay)
            glay = lay
        M.grouped_wgrad(dys, a, self._g(l, "mlp.experts.w2_weight"), glay, accumulate=True)
        da = M.grouped_dgrad(dys, self._p(l, "mlp.experts.w2_weight"), glay)
        dgu = A.swiglu_bwd(da, gu)
        del da, dys
        M.grouped_wgrad(dgu, xs, self._g(l, "mlp.experts.w13_weight"), glay, accumulate=True)
        dxs = M.grouped_dgrad(dgu, self._p(l, "mlp.experts.w13_weight"), glay)
        del dgu
        dh2 = self.ep.collect(dxs, lay) if self.ep is not None else M.scatter_sum(dxs, lay)
        # router: d logits from d weights (softmax over all experts, renormalised over the chosen k)
        logits = k["moe_logits"].detach().requires_grad_(True)
        with torch.enable_grad():
            wt = M.route_weights_from_probs(logits, k["moe_ids"], c.norm_topk_prob)
            (wt * dw).sum().backward()
        dlog = logits.grad.to(k["h2"].dtype)
        G.gemm_tn(dlog, k["h2"], out=self._g(l, "mlp.gate.weight"), accumulate=True)
        dh2 = dh2 + G.gemm_nn(dlog, self._p(l, "mlp.gate.weight"))
        return dh2

    # ------------------------------------------------------------------ FLOPs
    def flops_per_token(self, seqlen: int) -> float:
        c = self.cfg
        moe = 3 * c.hidden_size * c.moe_intermediate_size * c.num_experts_per_tok + c.hidden_size * c.num_experts
        dense = c.num_hidden_layers * (c.qkv_size * c.hidden_size + c.hidden_size * c.q_size + moe) + c.vocab_size * c.hidden_size
        return 6 * dense + 12 * c.num_hidden_layers * c.q_size * seqlen / 2


def build_model_for(cfg: ModelConfig, device="cuda", dtype=torch.bfloat16):
    """Dense or sparse in-house model, or one of the families of ``models/families.py``, by configuration."""
    from .families import FAMILY_TYPES, FamilyModel
    if cfg.model_type in FAMILY_TYPES:
        return FamilyModel(cfg, device=device, dtype=dtype)
    return (MoEModel if cfg.num_experts > 0 else DenseModel)(cfg, device=device, dtype=dtype)
