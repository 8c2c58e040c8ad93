"""Dense decoder under Ulysses sequence parallelism (reference: ``ulysses_sequence_parallel_size`` of the
FSDP trainer, axon/trainer/fsdp_trainer.py:132-184; padding and slicing of the packed batch,
axon/utils/ulysses.py:272-319; attention patch, axon/monkey_patches/transformers/monkey_patch.py:48-117).

Every rank of the group runs the whole model on its contiguous ``T / W`` slice of the packed tokens -
norms, projections, MLP, vocabulary head - and only attention sees whole sequences, on ``heads / W``
heads, through the exchange of ``parallel/ulysses.py``. Weights are full on every rank; their gradients
are partial sums over the local tokens and are completed by the optimizer's reduce-scatter, whose group
spans the sequence-parallel ranks as well (no separate all-reduce of 4 bytes per parameter).
"""
from __future__ import annotations

import torch

from ..ops import attention as AT
from ..parallel.ulysses import UlyssesContext
from .config import ModelConfig
from .dense import DenseModel, PackedBatch
from .mtp import SlicedModuleMixin, shifted_inputs
from .tp_dense import pad_packed_batch


class UlyssesDenseModel(DenseModel):
    def __init__(self, cfg: ModelConfig, sp: UlyssesContext, device="cuda", dtype=torch.bfloat16, params=None):
        super().__init__(cfg, device, dtype, params)
        W = sp.world
        assert cfg.num_attention_heads % W == 0 and cfg.num_key_value_heads % W == 0, \
            f"heads ({cfg.num_attention_heads} query / {cfg.num_key_value_heads} kv) must divide by the sequence-parallel size {W}"
        self.sp = sp
        D = cfg.head_dim
        self.wq, self.wkv = cfg.num_attention_heads // W * D, cfg.num_key_value_heads // W * D
        q, kv = cfg.q_size, cfg.kv_size
        # (src offset, per-rank width, dst offset): full-head row <-> this rank's heads
        self.seg_qkv_out = [(0, self.wq, 0), (q, self.wkv, self.wq), (q + kv, self.wkv, self.wq + self.wkv)]
        self.seg_qkv_back = [(0, self.wq, 0), (self.wq, self.wkv, q), (self.wq + self.wkv, self.wkv, q + kv)]
        self.seg_o = [(0, self.wq, 0)]

    def _heads(self):
        W = self.sp.world
        return self.cfg.num_attention_heads // W, self.cfg.num_key_value_heads // W

    def _attn_fwd(self, qkv_r, batch: PackedBatch, need_lse: bool):
        hq, hkv = self._heads()
        qkv_h = self.sp.scatter_cols(qkv_r, self.seg_qkv_out, self.wq + 2 * self.wkv, copy=False)     # [T, my heads], consumed at once
        o_h, lse = AT.attn_fwd(qkv_h, batch.cu_seqlens, hq, hkv, self.cfg.head_dim, need_lse=need_lse)
        o = self.sp.scatter_rows(o_h, self.seg_o, self.cfg.q_size)                                   # [T/W, all heads]
        return o, lse

    def _attn_bwd(self, do, qkv_r, o, lse, batch: PackedBatch):
        hq, hkv = self._heads()
        qkv_h = self.sp.scatter_cols(qkv_r, self.seg_qkv_out, self.wq + 2 * self.wkv)
        o_h = self.sp.scatter_cols(o, self.seg_o, self.wq)
        do_h = self.sp.scatter_cols(do, self.seg_o, self.wq)
        dqkv_h = AT.attn_bwd(do_h, qkv_h, o_h, lse, batch.cu_seqlens, hq, hkv, self.cfg.head_dim)
        return self.sp.scatter_rows(dqkv_h, self.seg_qkv_back, self.cfg.qkv_size)


class UlyssesModelAdapter(SlicedModuleMixin):
    """The interface of ``DenseModel`` (full packed batch in, full log-probs out, full-batch gradients in)
    on top of the sequence-parallel model: pads the batch to a multiple of 128 tokens per rank, hands
    the local slice to the model and gathers the per-token results."""

    def __init__(self, model: UlyssesDenseModel):
        self.inner, self.sp = model, model.sp
        self.cfg, self.params, self.device, self.dtype = model.cfg, model.params, model.device, model.dtype
        self._T = self._T_real = 0
        self.same_rows_ranks = self.sp.world

    def _mtp_group(self):
        return self.sp.group if self.sp.world > 1 else None

    @property
    def recompute(self):
        return self.inner.recompute

    @recompute.setter
    def recompute(self, v):
        self.inner.recompute = v

    def _local(self, batch: PackedBatch) -> PackedBatch:
        padded, self._T_real = pad_packed_batch(batch, 128 * self.sp.world)
        self._T = padded.input_ids.numel()
        n = self._T // self.sp.world
        sl = slice(self.sp.rank * n, (self.sp.rank + 1) * n)
        local = PackedBatch(padded.input_ids[sl].contiguous(), padded.position_ids[sl].contiguous(), padded.cu_seqlens,
                            padded.labels[sl].contiguous(), padded.max_seqlen)
        if self._wants_mtp():          # next tokens and second-next labels are shifted within whole sequences, then cut
            nxt, lab2 = shifted_inputs(padded)
            local.mtp_inputs = (nxt[sl].contiguous(), lab2[sl].contiguous())
        return local

    def forward(self, batch: PackedBatch, temperature: float = 1.0, save_for_backward: bool = False):
        lp, ent = self.inner.forward(self._local(batch), temperature, save_for_backward)
        return self.sp.all_gather_rows(lp)[: self._T_real], self.sp.all_gather_rows(ent)[: self._T_real]

    def backward(self, g_logprob, g_entropy=None) -> None:
        n = self._T // self.sp.world
        sl = slice(self.sp.rank * n, (self.sp.rank + 1) * n)

        def cut(g):
            if g is None:
                return None
            full = torch.zeros(self._T, dtype=torch.float32, device=g.device)
            full[: self._T_real] = g.float()
            return full[sl].contiguous()
        self.inner.backward(cut(g_logprob), cut(g_entropy))

    def flops_per_token(self, seqlen: int) -> float:
        return self.inner.flops_per_token(seqlen) / self.sp.world

    def __getattr__(self, name):          # prefill / decode / weights ...: the wrapped model's
        return getattr(self.inner, name)
