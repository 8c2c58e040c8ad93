"""Sparse attention of the GLM-5 / DeepSeek-V3.2 family: the "lightning indexer" that scores keys per query,
and multi-head latent attention over the top-k keys it selects.

Reference: axon/models/glm5_ops/ - ``tilelang_indexer_fwd.py`` (logits + window cleaning), ``tilelang_indexer_bwd.py``
(gradients at the selected indices), ``tilelang_sparse_mla_fwd.py`` / ``tilelang_sparse_mla_bwd.py`` (attention over
gathered latent rows: 512 value dims + 64 rotary dims, all heads share one key row).

    logits[s, j] = sum_h w[s, h] * relu(q[s, h] . k[j])        for ks[s] <= j < ke[s], -inf outside
    idx[s]       = top-k of logits[s]
    out[s, h]    = softmax_j in idx[s] (scale * q_mla[s, h] . kv[j]) @ kv[j, :512]

Native paths. The indexer forward is one tcgen05 GEMM ``[S * heads, D] x [Skv, D]^T`` whose epilogue applies the
ReLU and the head weight and sums the 32 accumulator rows of a query across the lanes of a warp
(``csrc/gemm.cu``: ``IndexerEpi``), so the per-head scores never leave the SM. The rest has PyTorch
implementations here (fp32, chunked over queries so the gathered rows stay small), which are also the oracles.
"""
from __future__ import annotations

import ctypes

import torch

from . import _common as C

NEG_INF = float("-inf")


# ---------------------------------------------------------------------- indexer
def indexer_logits_ref(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor, ks: torch.Tensor, ke: torch.Tensor) -> torch.Tensor:
    """q [S, Hi, D], k [Skv, D], w [S, Hi], window [ks, ke) per query -> fp32 logits [S, Skv]."""
    S, Skv = q.shape[0], k.shape[0]
    out = torch.empty(S, Skv, dtype=torch.float32, device=q.device)
    kf = k.float()
    for s0 in range(0, S, 256):
        sl = slice(s0, min(S, s0 + 256))
        sc = torch.einsum("shd,jd->shj", q[sl].float(), kf).relu_()
        out[sl] = (sc * w[sl].float().unsqueeze(-1)).sum(1)
    j = torch.arange(Skv, device=q.device)[None, :]
    return out.masked_fill((j < ks[:, None]) | (j >= ke[:, None]), NEG_INF)


def indexer_logits(q, k, w, ks, ke) -> torch.Tensor:
    S, Hi, D = q.shape
    if not C.use_native(q) or Hi % 32 != 0 or D % 64 != 0:
        return indexer_logits_ref(q, k, w, ks, ke)
    Skv = k.shape[0]
    q2 = q.reshape(S * Hi, D)
    assert q2.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and q2.stride(1) == 1 and k.stride(1) == 1
    wf = w.float().contiguous()
    ld = (Skv + 3) // 4 * 4
    out = (torch.zeros if Hi > 32 else torch.empty)(S, ld, dtype=torch.float32, device=q.device)
    rc = C.lib().axb_indexer_fwd(C.ptr(q2), C.ptr(k), C.ptr(wf), C.ptr(ks.int().contiguous()), C.ptr(ke.int().contiguous()),
                                 C.ptr(out), S, Hi, Skv, D, ctypes.c_longlong(q2.stride(0)), ctypes.c_longlong(k.stride(0)),
                                 ctypes.c_longlong(ld), C.ptr(C.status(q.device)), C.stream())
    C.launched(rc, "indexer_fwd")
    return out[:, :Skv]


def indexer_topk(logits: torch.Tensor, topk: int) -> torch.Tensor:
    """Indices of the ``topk`` largest logits per query, -1 where the window holds fewer keys."""
    kk = min(topk, logits.shape[1])
    val, idx = logits.topk(kk, dim=1)
    idx = idx.masked_fill(val == NEG_INF, -1).int()
    if kk < topk:
        idx = torch.cat([idx, idx.new_full((idx.shape[0], topk - kk), -1)], 1)
    return idx


def indexer_bwd_ref(g: torch.Tensor, idx: torch.Tensor, q: torch.Tensor, k: torch.Tensor, w: torch.Tensor):
    """Gradients of the logits at the selected indices: g [S, topk] (0 where idx < 0) -> (dq, dk, dw) in fp32."""
    S, Hi, D = q.shape
    dq = torch.zeros(S, Hi, D, dtype=torch.float32, device=q.device)
    dk = torch.zeros(k.shape[0], D, dtype=torch.float32, device=q.device)
    dw = torch.zeros(S, Hi, dtype=torch.float32, device=q.device)
    kf = k.float()
    for s0 in range(0, S, 64):
        sl = slice(s0, min(S, s0 + 64))
        ix = idx[sl].long()
        ok = (ix >= 0)
        ixc = ix.clamp_min(0)
        ksel = kf[ixc]                                              # [s, topk, D]
        sc = torch.einsum("shd,sjd->shj", q[sl].float(), ksel)
        gj = (g[sl].float() * ok)[:, None, :]                       # [s, 1, topk]
        dw[sl] = (sc.relu() * gj).sum(-1)
        coef = (sc > 0).float() * gj * w[sl].float().unsqueeze(-1)  # [s, Hi, topk]
        dq[sl] = torch.einsum("shj,sjd->shd", coef, ksel)
        dk.index_add_(0, ixc.reshape(-1), torch.einsum("shj,shd->sjd", coef, q[sl].float()).reshape(-1, D))
    return dq, dk, dw


# ---------------------------------------------------------------------- sparse latent attention
def sparse_mla_fwd_ref(q: torch.Tensor, kv: torch.Tensor, idx: torch.Tensor, scale: float, d_v: int = 512, chunk: int = 32):
    """q [S, H, Dk], kv [Skv, Dk] (values = the first ``d_v`` dims of a row), idx [S, topk] (-1 = none)
    -> (out [S, H, d_v] in q's dtype, lse fp32 [S, H]). A query without any key gives zeros and lse = -inf."""
    S, H, _ = q.shape
    out = torch.zeros(S, H, d_v, dtype=torch.float32, device=q.device)
    lse = torch.full((S, H), NEG_INF, dtype=torch.float32, device=q.device)
    kvf = kv.float()
    for s0 in range(0, S, chunk):
        sl = slice(s0, min(S, s0 + chunk))
        ix = idx[sl].long()
        rows = kvf[ix.clamp_min(0)]                                 # [s, topk, Dk]
        sc = torch.einsum("shd,sjd->shj", q[sl].float(), rows) * scale
        sc = sc.masked_fill((ix < 0)[:, None, :], NEG_INF)
        l = torch.logsumexp(sc, -1)
        p = torch.exp(sc - l.masked_fill(l == NEG_INF, 0.0).unsqueeze(-1))
        out[sl] = torch.einsum("shj,sjd->shd", p, rows[..., :d_v])
        lse[sl] = l
    return out.to(q.dtype), lse


def sparse_mla_bwd_ref(do: torch.Tensor, q: torch.Tensor, kv: torch.Tensor, out: torch.Tensor, lse: torch.Tensor,
                       idx: torch.Tensor, scale: float, d_v: int = 512, chunk: int = 32):
    """Returns (dq in q's dtype, dkv fp32 [Skv, Dk])."""
    S, H, Dk = q.shape
    dq = torch.zeros(S, H, Dk, dtype=torch.float32, device=q.device)
    dkv = torch.zeros(kv.shape[0], Dk, dtype=torch.float32, device=q.device)
    kvf = kv.float()
    for s0 in range(0, S, chunk):
        sl = slice(s0, min(S, s0 + chunk))
        ix = idx[sl].long()
        ixc = ix.clamp_min(0)
        rows = kvf[ixc]
        qf, dof = q[sl].float(), do[sl].float()
        sc = torch.einsum("shd,sjd->shj", qf, rows) * scale
        l = lse[sl]
        p = torch.exp(sc - l.masked_fill(l == NEG_INF, 0.0).unsqueeze(-1)).masked_fill((ix < 0)[:, None, :], 0.0)
        dp = torch.einsum("shd,sjd->shj", dof, rows[..., :d_v])
        delta = (dof * out[sl].float()).sum(-1, keepdim=True)
        ds = p * (dp - delta) * scale
        dq[sl] = torch.einsum("shj,sjd->shd", ds, rows)
        drows = torch.einsum("shj,shd->sjd", ds, qf)
        drows[..., :d_v] += torch.einsum("shj,shd->sjd", p, dof)
        dkv.index_add_(0, ixc.reshape(-1), drows.reshape(-1, Dk))
    return dq.to(q.dtype), dkv


class _SparseMLA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, kv, idx, scale, d_v):
        out, lse = sparse_mla_fwd_ref(q, kv, idx, scale, d_v)
        ctx.save_for_backward(q, kv, idx, out, lse)
        ctx.scale, ctx.d_v = scale, d_v
        return out, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, kv, idx, out, lse = ctx.saved_tensors
        dq, dkv = sparse_mla_bwd_ref(do, q, kv, out, lse, idx, ctx.scale, ctx.d_v)
        return dq, dkv.to(kv.dtype), None, None, None


def sparse_mla(q, kv, idx, scale: float, d_v: int = 512):
    """Differentiable sparse latent attention: (out, lse)."""
    return _SparseMLA.apply(q, kv, idx, scale, d_v)


class _IndexerLogitsAt(torch.autograd.Function):
    """Logits of the indexer at given indices (what its training loss reads): gradients flow to q, k and w
    through ``indexer_bwd_ref``, restricted to the selected keys."""

    @staticmethod
    def forward(ctx, q, k, w, idx):
        ctx.save_for_backward(q, k, w, idx)
        S = q.shape[0]
        ksel = k.float()[idx.long().clamp_min(0)]
        sc = torch.einsum("shd,sjd->shj", q.float(), ksel).relu_()
        return (sc * w.float().unsqueeze(-1)).sum(1).masked_fill(idx < 0, 0.0)

    @staticmethod
    def backward(ctx, g):
        q, k, w, idx = ctx.saved_tensors
        dq, dk, dw = indexer_bwd_ref(g, idx, q, k, w)
        return dq.to(q.dtype), dk.to(k.dtype), dw.to(w.dtype), None


def indexer_logits_at(q, k, w, idx):
    return _IndexerLogitsAt.apply(q, k, w, idx)
