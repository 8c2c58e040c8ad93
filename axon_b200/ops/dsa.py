"""Sparse attention of the GLM-5 / DeepSeek-V3.2 family: the "lightning indexer" that scores keys per query,
and multi-head latent attention over the top-k keys it selects.

Reference: axon/models/glm5_ops/ - ``tilelang_indexer_fwd.py`` (logits + window cleaning), ``tilelang_indexer_bwd.py``
(gradients at the selected indices), ``tilelang_sparse_mla_fwd.py`` / ``tilelang_sparse_mla_bwd.py`` (attention over
gathered latent rows: 512 value dims + 64 rotary dims, all heads share one key row).

    logits[s, j] = sum_h w[s, h] * relu(q[s, h] . k[j])        for ks[s] <= j < ke[s], -inf outside
    idx[s]       = top-k of logits[s]
    out[s, h]    = softmax_j in idx[s] (scale * q_mla[s, h] . kv[j]) @ kv[j, :512]

Native paths. The indexer forward is one tcgen05 GEMM ``[Skv, D] x [S * heads, D]^T`` (keys on the 128-row side)
whose epilogue applies the ReLU and the head weight and sums the 32 heads a thread holds in its accumulator
registers (``csrc/gemm.cu``: ``IndexerEpi``), so the per-head scores never leave the SM; its backward at the selected keys is
``csrc/dsa.cu`` (one block per query, warp per key, transposing butterfly for the 32 head dot products). The rest has PyTorch
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
    if not C.use_native(q) or Hi not in (32, 64, 128, 256) or D % 64 != 0:
        return indexer_logits_ref(q, k, w, ks, ke)
    Skv = k.shape[0]
    q2 = q.reshape(S * Hi, D)
    assert q2.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and q2.stride(1) == 1 and k.stride(1) == 1
    wf = w.float().contiguous()
    ld = (Skv + 3) // 4 * 4
    out = torch.empty(S, ld, dtype=torch.float32, device=q.device)
    ks_i, ke_i = ks.int().contiguous(), ke.int().contiguous()          # named: they must outlive the launch call
    rc = C.lib().axb_indexer_fwd(C.ptr(q2), C.ptr(k), C.ptr(wf), C.ptr(ks_i), C.ptr(ke_i),
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


def indexer_bwd(g: torch.Tensor, idx: torch.Tensor, q: torch.Tensor, k: torch.Tensor, w: torch.Tensor):
    """(dq, dk, dw) in fp32; native kernel for bf16 inputs with head dim 128 and 32 / 64 heads."""
    S, Hi, D = q.shape
    if not C.use_native(q) or Hi % 32 != 0 or Hi > 64 or D != 128 or q.dtype != torch.bfloat16:
        return indexer_bwd_ref(g, idx, q, k, w)
    q2, kc = q.reshape(S * Hi, D), k.contiguous()
    assert q2.stride(1) == 1 and k.dtype == torch.bfloat16
    gf, ix, wf = g.float().contiguous(), idx.int().contiguous(), w.float().contiguous()
    dq = torch.empty(S, Hi, D, dtype=torch.float32, device=q.device)
    dk = torch.zeros(k.shape[0], D, dtype=torch.float32, device=q.device)
    dw = torch.empty(S, Hi, dtype=torch.float32, device=q.device)
    rc = C.lib().axb_indexer_bwd(C.ptr(gf), C.ptr(ix), C.ptr(q2), C.ptr(kc), C.ptr(wf), C.ptr(dq), C.ptr(dk), C.ptr(dw),
                                 S, Hi, ix.shape[1], k.shape[0], D, ctypes.c_longlong(q2.stride(0)),
                                 ctypes.c_longlong(kc.stride(0)), C.stream())
    C.launched(rc, "indexer_bwd")
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
        out, lse = sparse_mla_fwd(q, kv, idx, scale, d_v)
        ctx.save_for_backward(q, kv, idx, out, lse)
        ctx.scale, ctx.d_v = scale, d_v
        return out, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, kv, idx, out, lse = ctx.saved_tensors
        dq, dkv = sparse_mla_bwd(do, q, kv, out, lse, idx, ctx.scale, ctx.d_v)
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
        dq, dk, dw = indexer_bwd(g, idx, q, k, w)
        return dq.to(q.dtype), dk.to(k.dtype), dw.to(w.dtype), None


def indexer_logits_at(q, k, w, idx):
    return _IndexerLogitsAt.apply(q, k, w, idx)


# ---------------------------------------------------------------------- sparse latent attention on the tensor cores
# Dense-masked formulation: per chunk of queries, scores against ALL keys run as one tcgen05 GEMM
# ([queries x heads, Dk] x [Skv, Dk]^T - every head of a query shares the key rows, so the product is a plain
# matrix product), keys outside a query's selection are masked, and P @ V is a second GEMM. This spends
# Skv / topk times the FLOPs of a gathering kernel but runs them at GEMM speed without materialising
# gathered rows; it is the CUDA path for contexts up to a few times ``topk``. A gathering tcgen05 kernel
# (selected rows copied into swizzled shared memory, value dims split over a CTA pair because a
# 128 x 512 fp32 accumulator fills tensor memory) is not built.
_SCORE_BYTES = 256 << 20


def _allowed(idx: torch.Tensor, skv_pad: int) -> torch.Tensor:
    m = torch.zeros(idx.shape[0], skv_pad + 1, dtype=torch.bool, device=idx.device)
    m.scatter_(1, torch.where(idx >= 0, idx, torch.full_like(idx, skv_pad)).long(), True)
    return m[:, :skv_pad]


def _pad_rows(kv: torch.Tensor, mult: int = 64) -> torch.Tensor:
    n = kv.shape[0]
    pad = (-n) % mult
    return kv.contiguous() if pad == 0 else torch.cat([kv, kv.new_zeros(pad, kv.shape[1])])


def _probs(qc, kvp, allowed, scale, H, lse=None):
    """bf16-valued probabilities [s * H, Skv_pad] (and lse [s, H]) of one query chunk. On CUDA the mask, the
    scale, the log-sum-exp and the exponent are one kernel over the fp32 scores (``axb_masked_softmax``)."""
    from . import gemm as G
    s = qc.shape[0]
    sc = G.gemm_nt(qc.reshape(s * H, -1), kvp, out_dtype=torch.float32)
    n = sc.shape[1]
    if C.use_native(sc):
        p = torch.empty(s * H, n, dtype=torch.bfloat16, device=sc.device)
        ok = allowed.to(torch.uint8).contiguous()
        lse_in = None if lse is None else lse.reshape(-1).float().contiguous()
        lse_out = torch.empty(s * H, dtype=torch.float32, device=sc.device) if lse is None else None
        rc = C.lib().axb_masked_softmax(C.ptr(sc), C.ptr(ok), C.ptr(p), C.ptr(lse_out), C.ptr(lse_in), ctypes.c_longlong(s * H), H, n,
                                        ctypes.c_longlong(sc.stride(0)), ctypes.c_longlong(n), ctypes.c_float(scale), C.stream())
        C.launched(rc, "masked_softmax")
        return p, (lse if lse is not None else lse_out.view(s, H))
    sc = sc.view(s, H, -1)
    sc.mul_(scale).masked_fill_(~allowed[:, None, :], NEG_INF)
    if lse is None:
        lse = torch.logsumexp(sc, -1)
    p = torch.exp_(sc.sub_(lse.masked_fill(lse == NEG_INF, 0.0).unsqueeze(-1)))
    return p.view(s * H, -1), lse


def _dscores(p, dp, delta, scale):
    """bf16 ``p * (dp - delta) * scale``."""
    if C.use_native(p) and p.dtype == torch.bfloat16:
        ds = torch.empty_like(p)
        d = delta.reshape(-1).float().contiguous()
        rc = C.lib().axb_softmax_bwd(C.ptr(p), C.ptr(dp), C.ptr(d), C.ptr(ds), ctypes.c_longlong(p.shape[0]), p.shape[1],
                                     ctypes.c_longlong(p.stride(0)), ctypes.c_longlong(dp.stride(0)), ctypes.c_float(scale), C.stream())
        C.launched(rc, "softmax_bwd")
        return ds
    return (p.float() * (dp - delta) * scale).to(torch.bfloat16)


def sparse_mla_fwd_tc(q, kv, idx, scale: float, d_v: int = 512):
    from . import gemm as G
    S, H, Dk = q.shape
    kvp = _pad_rows(kv)
    step = max(1, _SCORE_BYTES // (H * kvp.shape[0] * 4))
    out = torch.empty(S, H, d_v, dtype=q.dtype, device=q.device)
    lse = torch.empty(S, H, dtype=torch.float32, device=q.device)
    v = kvp[:, :d_v]
    for s0 in range(0, S, step):
        sl = slice(s0, min(S, s0 + step))
        p, l = _probs(q[sl].contiguous(), kvp, _allowed(idx[sl], kvp.shape[0]), scale, H)
        out[sl] = G.gemm_nn(p.to(torch.bfloat16), v).view(-1, H, d_v)
        lse[sl] = l
    return out, lse


def sparse_mla_bwd_tc(do, q, kv, out, lse, idx, scale: float, d_v: int = 512):
    from . import gemm as G
    S, H, Dk = q.shape
    kvp = _pad_rows(kv)
    n = kvp.shape[0]
    step = max(1, _SCORE_BYTES // (H * n * 4))
    dq = torch.empty_like(q)
    dkv = torch.zeros(n, Dk, dtype=torch.float32, device=q.device)
    dv = torch.zeros(n, d_v, dtype=torch.float32, device=q.device)
    vk = kvp[:, :d_v].contiguous()                                   # [Skv, d_v]: K-major operand of dP = dO V^T
    for s0 in range(0, S, step):
        sl = slice(s0, min(S, s0 + step))
        qc, doc = q[sl].contiguous(), do[sl].contiguous().to(q.dtype)
        s = qc.shape[0]
        p, _ = _probs(qc, kvp, _allowed(idx[sl], n), scale, H, lse=lse[sl])
        dp = G.gemm_nt(doc.view(s * H, d_v), vk, out_dtype=torch.float32)
        delta = (doc.float() * out[sl].float()).sum(-1).view(s * H, 1)
        pb = p.to(torch.bfloat16)
        ds = _dscores(pb if p.is_cuda else p, dp, delta, scale)
        dq[sl] = G.gemm_nn(ds, kvp).view(s, H, Dk)
        G.gemm_tn(ds, qc.view(s * H, Dk), out=dkv, accumulate=True)
        G.gemm_tn(pb, doc.view(s * H, d_v), out=dv, accumulate=True)
    dkv[:, :d_v] += dv
    return dq, dkv[: kv.shape[0]]


def sparse_mla_fwd(q, kv, idx, scale: float, d_v: int = 512):
    if C.use_native(q) and q.dtype == torch.bfloat16 and q.shape[2] % 8 == 0 and d_v % 8 == 0:
        return sparse_mla_fwd_tc(q, kv, idx, scale, d_v)
    return sparse_mla_fwd_ref(q, kv, idx, scale, d_v)


def sparse_mla_bwd(do, q, kv, out, lse, idx, scale: float, d_v: int = 512):
    if C.use_native(q) and q.dtype == torch.bfloat16 and q.shape[2] % 8 == 0 and d_v % 8 == 0:
        return sparse_mla_bwd_tc(do, q, kv, out, lse, idx, scale, d_v)
    return sparse_mla_bwd_ref(do, q, kv, out, lse, idx, scale, d_v)


# ---------------------------------------------------------------------- the two stages together
def causal_windows(cu_seqlens: torch.Tensor, total: int):
    """Per packed position t of sequence b: keys [start of b, t] -> (ks, ke) int32 [T]."""
    cu = cu_seqlens.long()
    pos = torch.arange(total, device=cu.device)
    seq = torch.searchsorted(cu[1:].contiguous(), pos, right=True)
    return cu[seq].int(), (pos + 1).int()


def dsa_attention(q: torch.Tensor, kv: torch.Tensor, q_idx: torch.Tensor, k_idx: torch.Tensor, w_idx: torch.Tensor,
                  cu_seqlens: torch.Tensor, topk: int, scale: float, d_v: int = 512):
    """Sparse attention layer of the GLM-5 / DeepSeek-V3.2 family over a packed batch (reference: the attention
    of axon/models/mbridge/glm5.py built on glm5_ops): the indexer scores the causal window of every query, the
    ``topk`` best keys are selected (no gradient through the selection) and latent attention runs over them.
    q [T, H, Dk], kv [T, Dk], q_idx [T, Hi, Di], k_idx [T, Di], w_idx [T, Hi] -> (out [T, H, d_v], idx [T, topk]).
    With ``topk`` >= the longest sequence this is plain causal attention."""
    ks, ke = causal_windows(cu_seqlens, q.shape[0])
    with torch.no_grad():
        idx = indexer_topk(indexer_logits(q_idx, k_idx, w_idx, ks, ke), topk)
    out, _ = sparse_mla(q, kv, idx, scale, d_v)
    return out, idx
