"""Dense decoder under context parallelism (reference: ``megatron.context_parallel_size`` of the Megatron
trainer, axon/trainer/megatron_trainer.py, with the zigzag batch slicing of axon/utils/megatron/).

Every rank of the group runs the whole model on its two chunks of every sequence (``parallel/cp.py``):
norms, projections, MLP and the vocabulary head are token-wise and need nothing from the peers; attention
gathers K|V once per layer. Weights are full on every rank; their gradients are partial sums over the
local tokens and are completed by the optimizer's reduce-scatter, whose group spans the context-parallel
ranks as well.
"""
from __future__ import annotations

import torch

from ..parallel import cp as CP
from .config import ModelConfig
from .dense import DenseModel, PackedBatch
from .mtp import SlicedModuleMixin, shifted_inputs


class CPDenseModel(DenseModel):
    def __init__(self, cfg: ModelConfig, cp: CP.ContextParallel, device="cuda", dtype=torch.bfloat16, params=None):
        super().__init__(cfg, device, dtype, params)
        self.cp = cp

    def _attn_fwd(self, qkv_r, batch: PackedBatch, need_lse: bool):
        c = self.cfg
        return CP.attn_fwd(self.cp, qkv_r, batch.cu_seqlens, c.num_attention_heads, c.num_key_value_heads, c.head_dim)

    def _attn_bwd(self, do, qkv_r, o, lse, batch: PackedBatch):
        c = self.cfg
        return CP.attn_bwd(self.cp, do, qkv_r, o, lse, batch.cu_seqlens, c.num_attention_heads, c.num_key_value_heads, c.head_dim)


class CPModelAdapter(SlicedModuleMixin):
    """The interface of ``DenseModel`` (full packed batch in, full log-probs out, full-batch gradients in)
    on top of the context-parallel model: pads every sequence to a multiple of ``2 W`` tokens, hands the
    rank its zigzag chunks and puts the per-token results back into the order of the batch."""

    def __init__(self, model, token_multiple: int = 128):
        """``model``: a ``CPDenseModel`` - or the tensor-parallel adapter around a model whose attention is
        context-parallel, with ``token_multiple = 128 tp`` so that the rank's tokens divide over its tensor-parallel group."""
        self.inner, self.cp = model, model.cp
        self.cfg, self.params, self.device, self.dtype = model.cfg, model.params, model.device, model.dtype
        self._maps = None
        self._token_multiple = int(token_multiple)
        self.same_rows_ranks = self.cp.world

    def _mtp_group(self):
        return self.cp.group if self.cp.world > 1 else None

    @property
    def recompute(self):
        return self.inner.recompute

    @recompute.setter
    def recompute(self, v):
        self.inner.recompute = v

    def _local(self, batch: PackedBatch) -> PackedBatch:
        W, me, dev = self.cp.world, self.cp.rank, batch.input_ids.device
        new_cu, orig_pos, off = CP.pad_layout(batch.cu_seqlens, W, self._token_multiple)
        T_pad = int(new_cu[-1])
        idx_all = [CP.local_index(new_cu, r, W) for r in range(W)]
        orig_pos_d = orig_pos.to(dev)

        def padded(src, fill):
            full = torch.full((T_pad,), fill, dtype=src.dtype, device=dev)
            full[orig_pos_d] = src
            return full
        mine = idx_all[me].to(dev)
        self._maps = (T_pad, orig_pos_d, torch.cat(idx_all).to(dev), mine)
        cu_half = (new_cu // (2 * W)).to(dev, batch.cu_seqlens.dtype)
        pos = off.to(dev, batch.position_ids.dtype)
        # positions of real tokens come from the batch (they need not start at 0), pads count on from 0
        pos[orig_pos_d] = batch.position_ids
        longest = int((new_cu[1:] - new_cu[:-1]).max())
        local = PackedBatch(padded(batch.input_ids, 0)[mine].contiguous(), pos[mine].contiguous(), cu_half,
                            padded(batch.labels, -100)[mine].contiguous(), max(int(batch.max_seqlen or 0), longest))
        if self._wants_mtp():          # shifted within the whole sequences of the batch, then laid out like the ids
            nxt, lab2 = shifted_inputs(batch)
            local.mtp_inputs = (padded(nxt, 0)[mine].contiguous(), padded(lab2, -100)[mine].contiguous())
        return local

    def forward(self, batch: PackedBatch, temperature: float = 1.0, save_for_backward: bool = False):
        lp, ent = self.inner.forward(self._local(batch), temperature, save_for_backward)
        T_pad, orig_pos, idx_cat, _ = self._maps

        def back(x):
            full = torch.empty(T_pad, dtype=x.dtype, device=x.device)
            full[idx_cat] = self._all_gather(x)
            return full[orig_pos]
        return back(lp), back(ent)

    def _all_gather(self, x: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        if self.cp.world == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(self.cp.world)]
        dist.all_gather(parts, x.contiguous(), group=self.cp.group)
        return torch.cat(parts)

    def backward(self, g_logprob, g_entropy=None) -> None:
        T_pad, orig_pos, _, mine = self._maps

        def cut(g):
            if g is None:
                return None
            full = torch.zeros(T_pad, dtype=torch.float32, device=g.device)
            full[orig_pos] = g.float()
            return full[mine].contiguous()
        self.inner.backward(cut(g_logprob), cut(g_entropy))

    def flops_per_token(self, seqlen: int) -> float:
        return self.inner.flops_per_token(seqlen) / self.cp.world

    def __getattr__(self, name):          # weights, prefill / decode ...: the wrapped model's
        return getattr(self.inner, name)
