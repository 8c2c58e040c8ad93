"""Sparse decoder under tensor parallelism AND expert parallelism over the same group of W ranks.

Attention is the tensor-parallel layer of ``tp_dense.TPDenseModel``: heads divided over the group, the
residual stream sharded along the token dimension (every rank owns T/W packed tokens), all-gather ->
GEMM and GEMM -> reduce-scatter fused over NVLink peer memory. The MLP needs none of those
collectives: the router (replicated) scores the rank's own T/W tokens, the expert-parallel context
sends each token to the ranks that own its experts (``parallel/ep.EPContext``: dispatch and combine
through peer memory, fused with the grouped GEMMs' layouts) and brings the weighted outputs back, so
a rank leaves the layer with its own T/W rows again. Each rank holds ``num_experts / W`` whole experts.

Gradients: expert weights are complete on their owner (every token routed to an expert is computed
there); router, norms, embedding and head are partial per rank (own tokens) and are summed over the
group by ``sync_replicated_grads``; attention weights as in the dense model. Backward re-runs the
MLP from the layer's recomputed input with the expert choice that forward recorded.

Expert TENSOR parallelism is the other way to divide the experts over the group (``ep=None``): every rank
keeps a slice of the intermediate units of every expert; the rows of the group are gathered, every rank
routes all of them, runs the grouped GEMMs on its slices and the partial outputs are reduce-scattered
back to the rows' owners - the dense tensor-parallel MLP with a router in front.

(reference: the quick-start recipe trains Qwen3-30B-A3B with ``tensor_model_parallel_size=4
expert_model_parallel_size=4`` on four GPUs - Megatron-Core's MoE layer with the all-to-all token
dispatcher inside a tensor-/sequence-parallel decoder, axon/trainer/megatron_trainer.py:164-173,
routing replay from axon/monkey_patches/megatron/moe_replay.py:167-401.)
"""
from __future__ import annotations

import torch

from .config import ModelConfig
from .moe import MoEModel
from .tp_dense import TPDenseModel


class TPMoEModel(TPDenseModel):
    SPARSE = True

    def __init__(self, cfg: ModelConfig, tp, ep=None, device="cuda", dtype=torch.bfloat16, vocab_parallel_head: bool = False):
        """``tp``: the group's ``TPContext``; ``ep``: an ``EPContext`` over the SAME ranks - or None for expert TENSOR
        parallelism: every rank then keeps 1 / W of the intermediate units of EVERY expert (``expert_tensor_parallel_size``
        = W with ``expert_model_parallel_size`` = 1) and the MLP is column / row parallel like a dense one, over all tokens."""
        if ep is not None:
            assert ep.world == tp.world and ep.rank == tp.rank, "experts are divided over the tensor-parallel group's own ranks"
            assert cfg.num_experts % tp.world == 0, f"{cfg.num_experts} experts do not divide over {tp.world} ranks"
            self.ep = ep if ep.world > 1 else None
            self.ep_world = ep.world
        else:
            assert cfg.moe_intermediate_size % tp.world == 0, f"expert width {cfg.moe_intermediate_size} does not divide over {tp.world} ranks"
            self.ep = None
            self.etp_world = tp.world
        super().__init__(cfg, tp, device=device, dtype=dtype, vocab_parallel_head=vocab_parallel_head)
        self.params.expert_offset = tp.rank * (cfg.num_experts // tp.world) if self.ep_world > 1 else 0
        self.capture_routing, self.last_routing = False, None
        self._ids: dict[int, torch.Tensor] = {}        # layer -> expert ids chosen in the latest forward (local rows)

    # the routing, dispatch and expert arithmetic are the unsharded sparse model's, on this rank's rows
    _route = MoEModel._route
    _experts = MoEModel._experts
    _combine = MoEModel._combine
    _moe_rebuild = MoEModel.mlp_rebuild
    _moe_bwd = MoEModel.mlp_bwd

    def _replay_local(self, l: int, batch):
        rm = getattr(batch, "routermap", None)
        if rm is None or l >= rm.shape[1]:
            return None
        return rm[self.local_slice(batch.input_ids.numel()), l, :].contiguous()

    # ---- expert tensor parallelism: every rank works on ALL tokens with its slice of every expert
    def _etp_experts(self, l, hf, ids):
        from ..ops import activation as A
        from ..ops import moe as M
        lay = M.align(ids, self.cfg.num_experts)
        xs = M.gather(hf, lay)
        gu = M.grouped_fwd(xs, self._p(l, "mlp.experts.w13_weight"), lay)
        a = A.swiglu_fwd(gu)
        return lay, xs, gu, a, M.grouped_fwd(a, self._p(l, "mlp.experts.w2_weight"), lay)       # partial sums over the ranks' slices

    def _etp_fwd(self, l, h2, batch):
        from ..ops import moe as M
        hf = self.tp.all_gather_rows(h2)
        rm = getattr(batch, "routermap", None)
        logits, ids, w = self._route(l, hf, None if rm is None or l >= rm.shape[1] else rm[:, l, :].contiguous())
        lay, _, _, _, ys = self._etp_experts(l, hf, ids)
        self._ids[l] = ids
        if self.capture_routing:
            if self.last_routing is None:
                self.last_routing = []
            self.last_routing.append(ids[self.local_slice(hf.shape[0])])
        return self.tp.reduce_scatter_rows(M.combine(ys, w, lay))

    def _etp_bwd(self, l, h2, dx_out, batch):
        from ..ops import activation as A
        from ..ops import gemm as G
        from ..ops import moe as M
        c, tp = self.cfg, self.tp
        hf, dy = tp.all_gather_rows(h2), tp.all_gather_rows(dx_out)      # the output was a sum over the ranks: each slice sees the whole gradient
        ids = self._ids[l]
        gate = self._p(l, "mlp.gate.weight")
        logits = G.gemm_nt(hf, gate, out_dtype=torch.float32)
        w = M.route_weights_from_probs(logits, ids, c.norm_topk_prob)
        lay, xs, gu, a, ys = self._etp_experts(l, hf, ids)
        dys, dw = M.combine_bwd(dy, ys, w.detach(), lay)
        tp.all_reduce_(dw)                                               # <dy, y> over the whole expert output
        M.grouped_wgrad(dys, a, self._g(l, "mlp.experts.w2_weight"), lay, accumulate=True)
        dgu = A.swiglu_bwd(M.grouped_dgrad(dys, self._p(l, "mlp.experts.w2_weight"), lay), gu)
        M.grouped_wgrad(dgu, xs, self._g(l, "mlp.experts.w13_weight"), lay, accumulate=True)
        dhf = M.scatter_sum(M.grouped_dgrad(dgu, self._p(l, "mlp.experts.w13_weight"), lay), lay)       # partial over the slices
        lg = logits.detach().requires_grad_(True)
        with torch.enable_grad():
            (M.route_weights_from_probs(lg, ids, c.norm_topk_prob) * dw).sum().backward()
        sl = self.local_slice(hf.shape[0])
        dlog = lg.grad[sl].to(h2.dtype)                                  # the router is replicated: each rank accounts for its own rows
        G.gemm_tn(dlog, h2, out=self._g(l, "mlp.gate.weight"), accumulate=True)
        return tp.reduce_scatter_rows(dhf) + G.gemm_nn(dlog, gate)

    def _mlp_fwd(self, l, h2, batch):
        if self.etp_world > 1:
            return self._etp_fwd(l, h2, batch)
        logits, ids, w = self._route(l, h2, self._replay_local(l, batch))
        lay, xs, gu, a, ys = self._experts(l, h2, ids, w, False)
        self._ids[l] = ids
        if self.capture_routing:
            if self.last_routing is None:
                self.last_routing = []
            self.last_routing.append(ids)
        return self._combine(ys, w, lay)

    def _mlp_bwd(self, l, h2, dx_out, batch):
        if self.etp_world > 1:
            return self._etp_bwd(l, h2, dx_out, batch)
        k = {"h2": h2, "moe_ids": self._ids[l]}
        self._moe_rebuild(l, k, batch)
        return self._moe_bwd(l, k, dx_out)
