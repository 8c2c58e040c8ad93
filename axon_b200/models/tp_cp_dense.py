"""Tensor parallelism inside context-parallel ranks: ``world = dp x cp x tp``.

A context-parallel rank holds two zigzag chunks of every sequence (``parallel/cp.py``); here that rank is a
tensor-parallel group. The group runs ``tp_dense.TPDenseModel`` on the rank's tokens - heads divided over the
group, the residual stream cut again by rows - and only the attention kernel call changes: each member gathers
the K|V of ITS heads from the same member of the other context-parallel ranks and merges the blocks through
log-sum-exp (``parallel.cp.attn_fwd`` / ``attn_bwd`` with the local head counts), so the K|V exchange per
member shrinks by tp. Around the model sit the two adapters of the separate strategies: the context-parallel
one pads every sequence to a multiple of 2 cp tokens and the rank's token count to a multiple of 128 tp, hands
out the zigzag chunks and gathers per-token results over the context-parallel group; inside it the
tensor-parallel one gathers them over the tensor-parallel group.

Weights are tensor-parallel shards, the same on every context-parallel rank; their gradients are partial sums
over the rank's tokens and are completed by the optimizer's reduce-scatter, whose group spans the data- and
context-parallel ranks with the same place in their tensor-parallel group.

(reference: ``context_parallel_size`` together with ``tensor_model_parallel_size`` of the Megatron trainer -
sequences padded to a multiple of 2 cp tp, axon/utils/megatron/cp_utils.py, loss on the local chunks.)
"""
from __future__ import annotations

import torch

from ..parallel import cp as CP
from ..parallel.tp import TPContext
from .config import ModelConfig
from .tp_dense import TPDenseModel


class TPCPDenseModel(TPDenseModel):
    def __init__(self, cfg: ModelConfig, tp: TPContext, cp: CP.ContextParallel, device="cuda", dtype=torch.bfloat16):
        super().__init__(cfg, tp, device=device, dtype=dtype)
        self.cp = cp
        assert cp.kv_width == 2 * self.hkv * cfg.head_dim, "the K|V exchange carries this rank's key / value heads"

    def _attn_kernel(self, qkv_r, batch, need_lse):
        return CP.attn_fwd(self.cp, qkv_r, batch.cu_seqlens, self.hq, self.hkv, self.cfg.head_dim)

    def _attn_bwd(self, do, qkv_r, o, lse, batch):
        return CP.attn_bwd(self.cp, do, qkv_r, o, lse, batch.cu_seqlens, self.hq, self.hkv, self.cfg.head_dim)
