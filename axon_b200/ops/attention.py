"""Packed (varlen) causal GQA attention. Native tcgen05 kernels on CUDA; fp32 PyTorch on CPU.

``attn_fwd(qkv, cu_seqlens, ...)`` reads q, k and v as strided head slices of the fused
projection buffer ``[T, Hq + 2*Hkv, D]`` (no split/copy) and returns ``o[T, Hq*D]`` and the
log-sum-exp ``lse[Hq, T]`` needed by the backward pass. Replaces flash-attn varlen
(reference: HF flash_attention_2 under axon/trainer/fsdp_trainer.py:223-233).
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _common as C


def _ref_fwd(qkv, cu, Hq, Hkv, D, scale, causal=True):
    T = qkv.shape[0]
    x = qkv.view(T, Hq + 2 * Hkv, D).float()
    q, k, v = x[:, :Hq], x[:, Hq:Hq + Hkv], x[:, Hq + Hkv:]
    rep = Hq // Hkv
    o = torch.zeros(T, Hq, D, dtype=torch.float32, device=qkv.device)
    lse = torch.zeros(Hq, T, dtype=torch.float32, device=qkv.device)
    cu_l = cu.tolist()
    for b in range(len(cu_l) - 1):
        s, e = cu_l[b], cu_l[b + 1]
        if e <= s:
            continue
        qb = q[s:e].transpose(0, 1)                      # [Hq, L, D]
        kb = k[s:e].transpose(0, 1).repeat_interleave(rep, 0)
        vb = v[s:e].transpose(0, 1).repeat_interleave(rep, 0)
        sc = qb @ kb.transpose(1, 2) * scale
        if causal:
            L = e - s
            sc = sc.masked_fill(torch.ones(L, L, dtype=torch.bool, device=qkv.device).triu(1), float("-inf"))
        lse[:, s:e] = torch.logsumexp(sc, -1)
        o[s:e] = (torch.softmax(sc, -1) @ vb).transpose(0, 1)
    return o.reshape(T, Hq * D).to(qkv.dtype), lse


def attn_fwd(qkv, cu_seqlens, Hq, Hkv, D, scale=None, causal=True, need_lse=True):
    T = qkv.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not C.use_native(qkv):
        return _ref_fwd(qkv, cu_seqlens, Hq, Hkv, D, scale, causal)
    lib = C.lib()
    B = cu_seqlens.numel() - 1
    o = torch.empty(T, Hq * D, dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty(Hq, T, dtype=torch.float32, device=qkv.device) if need_lse else None
    ntiles = lib.axb_attn_max_tiles(ctypes.c_longlong(T), B)
    scratch = C.workspace(qkv.device, ntiles * 16 + 16, "attn_tiles")
    HT = Hq + 2 * Hkv
    q = qkv.view(T, HT * D)
    row = ctypes.c_longlong(HT * D)
    rc = lib.axb_attn_fwd(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(q.data_ptr() + Hq * D * 2),
        ctypes.c_void_p(q.data_ptr() + (Hq + Hkv) * D * 2), C.ptr(o), C.ptr(lse), C.ptr(cu_seqlens), B,
        ctypes.c_longlong(T), Hq, Hkv, D, row, row, ctypes.c_longlong(Hq * D), ctypes.c_float(scale),
        int(causal), C.ptr(scratch), C.ptr(C.status(qkv.device)), C.stream())
    C.launched(rc, "attn_fwd", 2)
    return o, lse


def _ref_bwd(do, qkv, o, lse, cu, Hq, Hkv, D, scale, causal=True):
    T = qkv.shape[0]
    x = qkv.view(T, Hq + 2 * Hkv, D).float()
    q, k, v = x[:, :Hq], x[:, Hq:Hq + Hkv], x[:, Hq + Hkv:]
    rep = Hq // Hkv
    dq = torch.zeros_like(q)
    dk = torch.zeros_like(k)
    dv = torch.zeros_like(v)
    dof = do.view(T, Hq, D).float()
    of = o.view(T, Hq, D).float()
    cu_l = cu.tolist()
    for b in range(len(cu_l) - 1):
        s, e = cu_l[b], cu_l[b + 1]
        if e <= s:
            continue
        L = e - s
        qb = q[s:e].transpose(0, 1)
        kb = k[s:e].transpose(0, 1).repeat_interleave(rep, 0)
        vb = v[s:e].transpose(0, 1).repeat_interleave(rep, 0)
        dob = dof[s:e].transpose(0, 1)
        sc = qb @ kb.transpose(1, 2) * scale
        if causal:
            sc = sc.masked_fill(torch.ones(L, L, dtype=torch.bool, device=qkv.device).triu(1), float("-inf"))
        p = torch.exp(sc - lse[:, s:e, None])
        dvb = p.transpose(1, 2) @ dob
        dp = dob @ vb.transpose(1, 2)
        delta = (dob * of[s:e].transpose(0, 1)).sum(-1, keepdim=True)
        ds = p * (dp - delta) * scale
        dq[s:e] = (ds @ kb).transpose(0, 1)
        dkb = ds.transpose(1, 2) @ qb
        dk[s:e] = dkb.view(Hkv, rep, L, D).sum(1).transpose(0, 1)
        dv[s:e] = dvb.view(Hkv, rep, L, D).sum(1).transpose(0, 1)
    return torch.cat([dq, dk, dv], 1).reshape(T, -1).to(qkv.dtype)


def attn_bwd(do, qkv, o, lse, cu_seqlens, Hq, Hkv, D, scale=None, causal=True):
    """Returns dqkv with the layout of qkv."""
    T = qkv.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not C.use_native(qkv):
        return _ref_bwd(do, qkv, o, lse, cu_seqlens, Hq, Hkv, D, scale, causal)
    lib = C.lib()
    B = cu_seqlens.numel() - 1
    HT = Hq + 2 * Hkv
    dqkv = torch.empty_like(qkv)
    delta = torch.empty(Hq, T, dtype=torch.float32, device=qkv.device)
    ntiles = lib.axb_attn_max_tiles(ctypes.c_longlong(T), B)
    scratch = C.workspace(qkv.device, ntiles * 16 + 16, "attn_tiles")
    base = qkv.data_ptr()
    dbase = dqkv.data_ptr()
    row = ctypes.c_longlong(HT * D)
    rc = lib.axb_attn_bwd(
        ctypes.c_void_p(base), ctypes.c_void_p(base + Hq * D * 2), ctypes.c_void_p(base + (Hq + Hkv) * D * 2),
        C.ptr(o), C.ptr(do), C.ptr(lse), C.ptr(delta),
        ctypes.c_void_p(dbase), ctypes.c_void_p(dbase + Hq * D * 2), ctypes.c_void_p(dbase + (Hq + Hkv) * D * 2),
        C.ptr(cu_seqlens), B, ctypes.c_longlong(T), Hq, Hkv, D, row, ctypes.c_longlong(Hq * D),
        ctypes.c_float(scale), int(causal), C.ptr(scratch), C.ptr(C.status(qkv.device)), C.stream())
    C.launched(rc, "attn_bwd", 4)
    return dqkv
