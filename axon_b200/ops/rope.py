"""Per-head QK RMSNorm (Qwen3) fused with rotary position embedding, forward/backward.

Operates on the fused projection output ``qkv[T, Hq + 2*Hkv, D]``: query and key heads are
optionally RMS-normalised over D with their own weight and rotated (rotate-half convention,
pairs i and i + D/2, as in HF ``apply_rotary_pos_emb``); value heads are copied.
"""
from __future__ import annotations

import ctypes

import torch

from . import _common as C

_TABLES: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def rope_tables(max_pos: int, dim: int, theta: float, device, rotary_dim: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos/sin tables [max_pos, dim/2] (cached per device). With ``rotary_dim < dim`` (partial rotary
    embeddings) only the first ``rotary_dim / 2`` pairs turn, with frequencies over ``rotary_dim``; the other
    pairs get angle 0 (cos 1, sin 0), so the kernels that rotate every pair (i, i + dim/2) leave them as they are."""
    rd = dim if rotary_dim is None else int(rotary_dim)
    key = (str(device), dim, float(theta), rd)
    tab = _TABLES.get(key)
    if tab is None or tab[0].shape[0] < max_pos:
        n = max(max_pos, 1024)
        inv = torch.zeros(dim // 2, dtype=torch.float64)
        inv[: rd // 2] = 1.0 / (theta ** (torch.arange(0, rd, 2, dtype=torch.float64) / rd))
        ang = torch.arange(n, dtype=torch.float64)[:, None] * inv[None, :]
        tab = (ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous())
        _TABLES[key] = tab
    return tab


def _rot(x, cos, sin):  # x [T,h,D] fp32
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)


def _rot_t(g, cos, sin):  # transpose (inverse) rotation applied to grads
    d = g.shape[-1] // 2
    g1, g2 = g[..., :d], g[..., d:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([g1 * c + g2 * s, g2 * c - g1 * s], -1)


def qknorm_rope_fwd(qkv, pos, cos_t, sin_t, Hq, Hkv, D, qw=None, kw=None, eps=1e-6, kv_cache=None):
    """QK-norm + RoPE of packed qkv rows. ``kv_cache = (kcache, vcache, tok_seq, block_table)``: the rotated K rows
    and the V rows are also written to their pages of the paged KV cache (token t at position ``pos[t]`` of block
    table row ``tok_seq[t]``) in the same launch."""
    T = qkv.shape[0]
    if kv_cache is not None and not C.use_native(qkv):
        from .paged import kv_write
        out = qknorm_rope_fwd(qkv, pos, cos_t, sin_t, Hq, Hkv, D, qw, kw, eps)
        kv_write(out, kv_cache[0], kv_cache[1], kv_cache[2], pos, kv_cache[3], Hq, Hkv, D)
        return out
    if not C.use_native(qkv):
        x = qkv.view(T, Hq + 2 * Hkv, D).float()
        cos, sin = cos_t[pos.long()], sin_t[pos.long()]
        outs = []
        for sl, w in ((slice(0, Hq), qw), (slice(Hq, Hq + Hkv), kw)):
            h = x[:, sl]
            if w is not None:
                h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * w.float()
            outs.append(_rot(h, cos, sin))
        outs.append(x[:, Hq + Hkv:])
        return torch.cat(outs, 1).to(qkv.dtype).view_as(qkv)
    out = torch.empty_like(qkv)
    if kv_cache is not None:
        kc, vc, tok_seq, bt = kv_cache
        rc = C.lib().axb_qknorm_rope_fwd_kv(C.ptr(qkv), C.ptr(out), C.ptr(qw), C.ptr(kw), C.ptr(pos), C.ptr(cos_t), C.ptr(sin_t),
                                            ctypes.c_longlong(T), Hq, Hkv, D, ctypes.c_float(eps), C.ptr(kc), C.ptr(vc), C.ptr(tok_seq),
                                            C.ptr(bt), bt.shape[1], kc.shape[0], kc.shape[2], C.stream())
        C.launched(rc, "qknorm_rope_fwd_kv")
        return out
    rc = C.lib().axb_qknorm_rope_fwd(C.ptr(qkv), C.ptr(out), C.ptr(qw), C.ptr(kw), C.ptr(pos), C.ptr(cos_t),
                                     C.ptr(sin_t), ctypes.c_longlong(T), Hq, Hkv, D, ctypes.c_float(eps),
                                     C.stream())
    C.launched(rc, "qknorm_rope_fwd")
    return out


def qknorm_rope_bwd(dout, qkv, pos, cos_t, sin_t, Hq, Hkv, D, qw=None, kw=None, dqw=None, dkw=None,
                    eps=1e-6, accumulate_dw: bool = True):
    """Returns dqkv; accumulates fp32 norm-weight grads into dqw/dkw when the model has QK-norm."""
    T = qkv.shape[0]
    if not C.use_native(qkv):
        x = qkv.view(T, Hq + 2 * Hkv, D).float()
        g = dout.view(T, Hq + 2 * Hkv, D).float()
        cos, sin = cos_t[pos.long()], sin_t[pos.long()]
        outs = []
        for sl, w, dw in ((slice(0, Hq), qw, dqw), (slice(Hq, Hq + Hkv), kw, dkw)):
            gh = _rot_t(g[:, sl], cos, sin)
            if w is not None:
                h = x[:, sl]
                r = torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
                xh = h * r
                dwn = (gh * xh).sum((0, 1))
                dw.copy_(dw + dwn if accumulate_dw else dwn)
                gw = gh * w.float()
                gh = r * (gw - xh * (gw * xh).mean(-1, keepdim=True))
            outs.append(gh)
        outs.append(g[:, Hq + Hkv:])
        return torch.cat(outs, 1).to(qkv.dtype).view_as(qkv)
    lib = C.lib()
    dqkv = torch.empty_like(qkv)
    P = lib.axb_qknorm_rope_bwd_partials(ctypes.c_longlong(T), Hq, Hkv)
    scratch = C.workspace(qkv.device, (P + 1) * 2 * D * 4, "norm")
    rc = lib.axb_qknorm_rope_bwd(C.ptr(dout), C.ptr(qkv), C.ptr(dqkv), C.ptr(qw), C.ptr(kw), C.ptr(pos),
                                 C.ptr(cos_t), C.ptr(sin_t), C.ptr(dqw), C.ptr(dkw), int(accumulate_dw),
                                 C.ptr(scratch), ctypes.c_longlong(T), Hq, Hkv, D, ctypes.c_float(eps),
                                 C.stream())
    C.launched(rc, "qknorm_rope_bwd", 4 if qw is not None else 1)
    return dqkv
