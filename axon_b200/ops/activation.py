"""SwiGLU on the fused gate|up projection output, embedding gather/scatter, residual add."""
from __future__ import annotations

import ctypes

import torch

from . import _common as C


def swiglu_fwd(gu):
    T, F2 = gu.shape
    F = F2 // 2
    if not C.use_native(gu):
        g, u = gu[:, :F].float(), gu[:, F:].float()
        return (torch.nn.functional.silu(g) * u).to(gu.dtype)
    a = torch.empty(T, F, dtype=gu.dtype, device=gu.device)
    rc = C.lib().axb_swiglu_fwd(C.ptr(gu), C.ptr(a), ctypes.c_longlong(T), F, C.stream())
    C.launched(rc, "swiglu_fwd")
    return a


def swiglu_bwd(da, gu):
    T, F2 = gu.shape
    F = F2 // 2
    if not C.use_native(gu):
        g, u, d = gu[:, :F].float(), gu[:, F:].float(), da.float()
        s = torch.sigmoid(g)
        silu = g * s
        return torch.cat([d * u * (s + silu * (1 - s)), d * silu], 1).to(gu.dtype)
    dgu = torch.empty_like(gu)
    rc = C.lib().axb_swiglu_bwd(C.ptr(da), C.ptr(gu), C.ptr(dgu), ctypes.c_longlong(T), F, C.stream())
    C.launched(rc, "swiglu_bwd")
    return dgu


def embedding_fwd(ids, table):
    T = ids.numel()
    V, H = table.shape
    if not C.use_native(table):
        return table[ids.long().clamp(0, V - 1)]
    out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    rc = C.lib().axb_embedding_fwd(C.ptr(ids), C.ptr(table), C.ptr(out), ctypes.c_longlong(T), H, V, C.stream())
    C.launched(rc, "embedding_fwd")
    return out


def embedding_bwd(ids, dy, dtable):
    """dtable[ids[t]] += dy[t]; dtable is fp32 [V,H]."""
    T = ids.numel()
    V, H = dtable.shape
    if not C.use_native(dy):
        dtable.index_add_(0, ids.long(), dy.float())
        return dtable
    rc = C.lib().axb_embedding_bwd(C.ptr(ids), C.ptr(dy), C.ptr(dtable), ctypes.c_longlong(T), H, V, C.stream())
    C.launched(rc, "embedding_bwd")
    return dtable


def add(a, b):
    if not C.use_native(a):
        return (a.float() + b.float()).to(a.dtype)
    y = torch.empty_like(a)
    rc = C.lib().axb_add_bf16(C.ptr(a), C.ptr(b), C.ptr(y), ctypes.c_longlong(a.numel()), C.stream())
    C.launched(rc, "add_bf16")
    return y
