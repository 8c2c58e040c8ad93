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

    def __init__(self, cfg: ModelConfig, tp, ep, device="cuda", dtype=torch.bfloat16, vocab_parallel_head: bool = False):
        """``tp``: the group's ``TPContext``; ``ep``: an ``EPContext`` over the SAME ranks."""
        assert ep.world == tp.world and ep.rank == tp.rank, "experts are divided over the tensor-parallel group's own ranks"
        assert cfg.num_experts % tp.world == 0, f"{cfg.num_experts} experts do not divide over {tp.world} ranks"
        self.ep = ep if ep.world > 1 else None
        self.ep_world = ep.world
        super().__init__(cfg, tp, device=device, dtype=dtype, vocab_parallel_head=vocab_parallel_head)
        self.params.expert_offset = tp.rank * (cfg.num_experts // tp.world)
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
        if rm is None:
            return None
        return rm[self.local_slice(batch.input_ids.numel()), l, :].contiguous()

    def _mlp_fwd(self, l, h2, batch):
        logits, ids, w = self._route(l, h2, self._replay_local(l, batch))
        lay, xs, gu, a, ys = self._experts(l, h2, ids, w, False)
        self._ids[l] = ids
        if self.capture_routing:
            if self.last_routing is None:
                self.last_routing = []
            self.last_routing.append(ids)
        return self._combine(ys, w, lay)

    def _mlp_bwd(self, l, h2, dx_out, batch):
        k = {"h2": h2, "moe_ids": self._ids[l]}
        self._moe_rebuild(l, k, batch)
        return self._moe_bwd(l, k, dx_out)
