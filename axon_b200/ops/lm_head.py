"""Fused vocabulary head: per-token log-prob of the label and softmax entropy from hidden states
and the (tied or untied) output embedding, never materialising ``[T, V]`` logits in the forward.

``linear_logprob_entropy(hidden, weight, labels, temperature)`` is the autograd entry point with
the contract of the reference's ``linear_cross_entropy``
(axon/utils/kernel/linear_cross_entropy.py:50-131): it returns ``(logprobs[T], entropy[T])`` with
``logprobs[t] = log softmax(hidden[t] W^T / temperature)[labels[t]]``.
"""
from __future__ import annotations

import ctypes

import torch

from . import _common as C
from . import gemm as G

BWD_CHUNK = 8192  # rows of dlogits materialised at a time in the backward pass


def ref_logprob_entropy(hidden, weight, labels, temperature=1.0, chunk=2048):
    """fp32 chunked reference (also the CPU implementation)."""
    T = hidden.shape[0]
    lp = torch.empty(T, dtype=torch.float32, device=hidden.device)
    ent = torch.empty_like(lp)
    lse = torch.empty_like(lp)
    for s in range(0, T, chunk):
        z = hidden[s:s + chunk].float() @ weight.float().t() / temperature
        l = torch.logsumexp(z, -1)
        p = torch.softmax(z, -1)
        lab = labels[s:s + chunk].long()
        lp[s:s + chunk] = torch.where(lab >= 0, z.gather(1, lab.clamp(min=0)[:, None])[:, 0] - l,
                                      torch.zeros_like(l))
        ent[s:s + chunk] = l - (p * z).sum(-1)
        lse[s:s + chunk] = l
    return lp, ent, lse


def lmhead_fwd(hidden, weight, labels, temperature=1.0):
    """Returns (logprob, entropy, lse), fp32 [T]."""
    if not C.use_native(hidden):
        return ref_logprob_entropy(hidden, weight, labels, temperature)
    T, H = hidden.shape
    V = weight.shape[0]
    lib = C.lib()
    lib.axb_lmhead_scratch_bytes.restype = ctypes.c_longlong
    nbytes = lib.axb_lmhead_scratch_bytes(ctypes.c_longlong(T), V)
    scratch = C.workspace(hidden.device, nbytes, "lmhead")
    lp = torch.empty(T, dtype=torch.float32, device=hidden.device)
    ent = torch.empty_like(lp)
    lse = torch.empty_like(lp)
    rc = lib.axb_lmhead_fwd(C.ptr(hidden), C.ptr(weight), C.ptr(labels), C.ptr(lp), C.ptr(ent), C.ptr(lse), T, V, H,
                            ctypes.c_longlong(hidden.stride(0)), ctypes.c_longlong(weight.stride(0)),
                            ctypes.c_float(temperature), C.ptr(scratch), C.ptr(C.status(hidden.device)),
                            C.stream())
    C.launched(rc, "lmhead_fwd", 2)
    return lp, ent, lse


def lmhead_bwd(hidden, weight, labels, lse, ent, g_lp, g_ent, temperature=1.0, dweight=None,
               need_dhidden=True):
    """Returns dhidden (bf16 [T,H]); accumulates dW into ``dweight`` (fp32 [V,H]) when given."""
    T, H = hidden.shape
    V = weight.shape[0]
    if not C.use_native(hidden):
        dh = torch.zeros(T, H, dtype=torch.float32)
        for s in range(0, T, 2048):
            e = min(T, s + 2048)
            z = hidden[s:e].float() @ weight.float().t() / temperature
            p = torch.exp(z - lse[s:e, None])
            lab = labels[s:e].long()
            glp = torch.where(lab >= 0, g_lp[s:e] if g_lp is not None else torch.zeros(e - s), torch.zeros(e - s))
            ge = g_ent[s:e] if g_ent is not None else torch.zeros(e - s)
            d = -glp[:, None] * p - ge[:, None] * p * (z - lse[s:e, None] + ent[s:e, None])
            d[torch.arange(e - s), lab.clamp(min=0)] += glp
            d = d / temperature
            dh[s:e] = d @ weight.float()
            if dweight is not None:
                dweight.add_(d.t() @ hidden[s:e].float())
        return dh.to(hidden.dtype)
    lib = C.lib()
    dh = torch.empty_like(hidden) if need_dhidden else None
    chunk = min(BWD_CHUNK, T)
    dl = C.workspace(hidden.device, chunk * V * 2, "lmhead_dlogits").view(torch.bfloat16)[: chunk * V].view(chunk, V)
    for s in range(0, T, chunk):
        e = min(T, s + chunk)
        n = e - s
        rc = lib.axb_lmhead_dlogits(
            C.ptr(hidden[s:e]), C.ptr(weight), C.ptr(labels[s:e]), C.ptr(lse[s:e]), C.ptr(ent[s:e]),
            C.ptr(None if g_lp is None else g_lp[s:e]), C.ptr(None if g_ent is None else g_ent[s:e]),
            C.ptr(dl), ctypes.c_longlong(V), n, V, H, ctypes.c_longlong(hidden.stride(0)),
            ctypes.c_longlong(weight.stride(0)), ctypes.c_float(temperature),
            C.ptr(C.status(hidden.device)), C.stream())
        C.launched(rc, "lmhead_dlogits")
        if need_dhidden:
            G.gemm_nn(dl[:n], weight, out=dh[s:e])
        if dweight is not None:
            G.gemm_tn(dl[:n], hidden[s:e], out=dweight, accumulate=True)
    return dh


class _LinearLogprobEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, temperature):
        lp, ent, lse = lmhead_fwd(hidden, weight, labels, temperature)
        ctx.save_for_backward(hidden, weight, labels, lse, ent)
        ctx.temperature = temperature
        return lp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        hidden, weight, labels, lse, ent = ctx.saved_tensors
        dw = None
        if ctx.needs_input_grad[1]:
            dw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        g_lp = None if g_lp is None else g_lp.float().contiguous()
        g_ent = None if g_ent is None else g_ent.float().contiguous()
        dh = lmhead_bwd(hidden, weight, labels, lse, ent, g_lp, g_ent, ctx.temperature, dweight=dw,
                        need_dhidden=ctx.needs_input_grad[0])
        return dh, (None if dw is None else dw.to(weight.dtype)), None, None


def linear_logprob_entropy(hidden, weight, labels, temperature: float = 1.0):
    """Autograd-enabled fused head. hidden [T,H], weight [V,H], labels int32 [T] (<0 = ignore)."""
    return _LinearLogprobEntropy.apply(hidden, weight, labels, float(temperature))
