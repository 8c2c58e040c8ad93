"""Gated delta rule (Gated DeltaNet linear attention) over packed sequences.

    S <- exp(g_t) S ;  u_t = beta_t (v_t - S^T k_t) ;  S <- S + k_t u_t^T ;  o_t = scale * S^T q_t

``gated_delta_rule`` runs the recurrent CUDA kernel (``csrc/gdn.cu``) on GPU tensors and the PyTorch
recurrence on CPU tensors; it is differentiable: on the GPU backward is the reverse sweep of ``axb_gdn_bwd`` (chunk-start states from a forward
sweep, the states inside a chunk replayed into scratch memory, so no division by the decay); elsewhere the PyTorch
recurrence is replayed under autograd (reference: the FLA ``chunk_gated_delta_rule``
call behind axon/monkey_patches/transformers/qwen3_5_gdn.py; a chunked tensor-core forward / backward is the
open follow-up).
"""
from __future__ import annotations

import ctypes

import torch

from . import _common as C


def gated_delta_rule_ref(q, k, v, g, beta, cu_seqlens, scale=None, initial_state=None):
    """fp32 PyTorch recurrence (differentiable). q,k [T,H,dk]; v [T,H,dv]; g,beta [T,H]. Returns (o [T,H,dv], state [B,H,dk,dv])."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    cu = [int(x) for x in cu_seqlens.tolist()]
    outs, finals = [], []
    for b in range(len(cu) - 1):
        S = torch.zeros(H, dk, dv, dtype=torch.float32, device=q.device) if initial_state is None else initial_state[b].float()
        for t in range(cu[b], cu[b + 1]):
            qt, kt, vt = q[t].float(), k[t].float(), v[t].float()
            S = S * torch.exp(g[t].float())[:, None, None]
            u = beta[t].float()[:, None] * (vt - torch.einsum("hkv,hk->hv", S, kt))
            S = S + kt[:, :, None] * u[:, None, :]
            outs.append(scale * torch.einsum("hkv,hk->hv", S, qt))
        finals.append(S)
    o = torch.stack(outs) if outs else torch.zeros(0, H, dv, device=q.device)
    return o, torch.stack(finals)


def _native_fwd(q, k, v, g, beta, cu_seqlens, scale, initial_state, want_state):
    T, H, dk = q.shape
    dv = v.shape[-1]
    B = cu_seqlens.numel() - 1
    o = torch.empty(T, H, dv, dtype=torch.bfloat16, device=q.device)
    st = torch.empty(B, H, dk, dv, dtype=torch.float32, device=q.device) if want_state else None
    rc = C.lib().axb_gdn_fwd(C.ptr(q.contiguous()), C.ptr(k.contiguous()), C.ptr(v.contiguous()), C.ptr(g.float().contiguous()),
                             C.ptr(beta.float().contiguous()), C.ptr(cu_seqlens.to(torch.int32)), B, H, dk, dv, ctypes.c_float(scale),
                             C.ptr(None if initial_state is None else initial_state.float().contiguous()), C.ptr(st), C.ptr(o), C.stream())
    C.launched(rc, "gdn_fwd")
    return o, st


class _GatedDeltaRule(torch.autograd.Function):
    CHUNK = 64

    @staticmethod
    def forward(ctx, q, k, v, g, beta, cu_seqlens, scale, initial_state):
        ctx.save_for_backward(q, k, v, g, beta, cu_seqlens, initial_state if initial_state is not None else torch.empty(0))
        ctx.scale, ctx.has_init = scale, initial_state is not None
        o, st = _native_fwd(q, k, v, g, beta, cu_seqlens, scale, initial_state, True)
        return o, st

    @staticmethod
    def backward(ctx, do, dstate):
        q, k, v, g, beta, cu, init = ctx.saved_tensors
        init = init if ctx.has_init else None
        if NATIVE_BACKWARD and q.dtype == torch.bfloat16:
            dq, dk_, dv_, dg, db, dinit = _native_bwd(q, k, v, g, beta, cu, ctx.scale, init, do, dstate)
            return dq, dk_, dv_, dg.to(g.dtype), db.to(beta.dtype), None, None, dinit if ctx.has_init else None
        leaves = [t.detach().float().requires_grad_(True) for t in (q, k, v, g, beta)]
        init_leaf = init.detach().float().requires_grad_(True) if init is not None else None
        with torch.enable_grad():
            o, st = gated_delta_rule_ref(*leaves, cu, ctx.scale, init_leaf)
            loss = (o * do.float()).sum() + ((st * dstate.float()).sum() if dstate is not None else 0.0)
        grads = torch.autograd.grad(loss, leaves + ([init_leaf] if init_leaf is not None else []), allow_unused=True)
        dq, dk_, dv_, dg, db = (None if x is None else x.to(t.dtype) for x, t in zip(grads[:5], (q, k, v, g, beta)))
        return dq, dk_, dv_, dg, db, None, None, (grads[5] if init_leaf is not None else None)


NATIVE_BACKWARD = True      # False: replay the PyTorch recurrence under autograd (the oracle of the kernel's test)
_BWD_CHUNK = 32             # tokens per chunk of the reverse sweep (GDN_CHUNK in csrc/gdn.cu)


def _native_bwd(q, k, v, g, beta, cu_seqlens, scale, initial_state, do, dstate):
    """Reverse sweep of the recurrence on the GPU (``axb_gdn_bwd``): chunk-start states from a forward sweep, the states
    inside a chunk replayed into a scratch area, gradients of q / k / g / beta as per-value-slice partials summed here."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    cu = cu_seqlens.to(torch.int32)
    B = cu.numel() - 1
    lens = (cu[1:] - cu[:-1])
    max_chunks = max(1, (int(lens.max()) + _BWD_CHUNK - 1) // _BWD_CHUNK)
    n_vb = (dv + 31) // 32
    dev, f32 = q.device, torch.float32
    chunk_states = torch.empty(B * H * n_vb * max_chunks * dk * 32, dtype=f32, device=dev)
    scratch = torch.empty(B * H * n_vb * (_BWD_CHUNK + 1) * dk * 32, dtype=f32, device=dev)
    dq_p = torch.zeros(n_vb, T, H, dk, dtype=f32, device=dev)
    dk_p = torch.zeros(n_vb, T, H, dk, dtype=f32, device=dev)
    dg_p = torch.zeros(n_vb, T, H, dtype=f32, device=dev)
    db_p = torch.zeros(n_vb, T, H, dtype=f32, device=dev)
    dv_o = torch.zeros(T, H, dv, dtype=f32, device=dev)
    dinit = torch.empty(B, H, dk, dv, dtype=f32, device=dev) if initial_state is not None else None
    dst = None if dstate is None else dstate.float().contiguous()
    rc = C.lib().axb_gdn_bwd(C.ptr(q.contiguous()), C.ptr(k.contiguous()), C.ptr(v.contiguous()), C.ptr(g.float().contiguous()),
                             C.ptr(beta.float().contiguous()), C.ptr(cu), B, H, dk, dv, T, max_chunks, ctypes.c_float(scale),
                             C.ptr(None if initial_state is None else initial_state.float().contiguous()),
                             C.ptr(do.to(torch.bfloat16).contiguous()), C.ptr(dst), C.ptr(chunk_states), C.ptr(scratch), C.ptr(dq_p),
                             C.ptr(dk_p), C.ptr(dg_p), C.ptr(db_p), C.ptr(dv_o), C.ptr(dinit), C.stream())
    C.launched(rc, "gdn_bwd")
    return dq_p.sum(0).to(q.dtype), dk_p.sum(0).to(k.dtype), dv_o.to(v.dtype), dg_p.sum(0), db_p.sum(0), dinit


def gated_delta_rule(q, k, v, g, beta, cu_seqlens, scale=None, initial_state=None):
    """Returns (o [T,H,dv], final state [B,H,dk,dv] fp32)."""
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    if not C.use_native(q):
        o, st = gated_delta_rule_ref(q, k, v, g, beta, cu_seqlens, scale, initial_state)
        return o.to(q.dtype), st
    assert q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
    if torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, g, beta)):
        return _GatedDeltaRule.apply(q, k, v, g, beta, cu_seqlens, scale, initial_state)
    return _native_fwd(q, k, v, g, beta, cu_seqlens, scale, initial_state, True)
