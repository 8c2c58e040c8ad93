"""Fused AdamW over flat fp32 master shards (+ bf16 working copy), grad-norm and clipping.

The clip coefficient and the non-finite skip flag live in a 4-float device ``state`` so an
optimizer step needs no host synchronisation. Equivalent of ``torch.optim.AdamW`` +
``clip_grad_norm_`` with the skip-on-non-finite rule of axon/trainer/fsdp_trainer.py:674-771.
"""
from __future__ import annotations

import ctypes

import torch

from . import _common as C


def sumsq(g: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out[0] (+)= sum(g**2); out is an fp32 device tensor with at least one element."""
    if not C.use_native(g):
        s = g.float().pow(2).sum()
        out[0] = out[0] + s if accumulate else s
        return out
    lib = C.lib()
    scratch = C.workspace(g.device, lib.axb_sumsq_partials() * 4, "optim")
    rc = lib.axb_sumsq(C.ptr(g), ctypes.c_longlong(g.numel()), int(g.dtype == torch.bfloat16), C.ptr(scratch),
                       C.ptr(out), int(accumulate), C.stream())
    C.launched(rc, "sumsq", 2)
    return out


def clip_coef(state: torch.Tensor, max_norm: float, skip_threshold: float = 0.0, grad_scale: float = 1.0):
    """state[0]=sumsq (in) -> state[1]=norm, state[2]=coef (includes grad_scale), state[3]=skip flag."""
    if not C.use_native(state):
        norm = state[0].sqrt() * grad_scale
        finite = bool(torch.isfinite(norm))
        skip = (not finite) or (skip_threshold > 0 and float(norm) > skip_threshold)
        coef = grad_scale
        if max_norm > 0 and finite:
            coef = grad_scale * min(1.0, max_norm / (float(norm) + 1e-6))
        state[1] = norm
        state[2] = 0.0 if skip else coef
        state[3] = 1.0 if skip else 0.0
        return state
    rc = C.lib().axb_clip_coef(C.ptr(state), ctypes.c_float(max_norm), ctypes.c_float(skip_threshold),
                               ctypes.c_float(grad_scale), C.stream())
    C.launched(rc, "clip_coef")
    return state


def adamw_step(master, param, grad, m, v, lr, beta1, beta2, eps, wd, step, state=None):
    """One AdamW step on flat tensors. ``param`` (bf16 working copy) may be None."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if not C.use_native(master):
        coef = 1.0
        if state is not None:
            if float(state[3]) != 0.0:
                return
            coef = float(state[2])
        g = grad.float() * coef
        m.mul_(beta1).add_(g, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        master.mul_(1 - lr * wd)
        master.addcdiv_(m / bc1, (v.sqrt() / (bc2 ** 0.5)).add_(eps), value=-lr)
        if param is not None:
            param.copy_(master)
        return
    rc = C.lib().axb_adamw(C.ptr(master), C.ptr(param), C.ptr(grad), int(grad.dtype == torch.bfloat16),
                           C.ptr(m), C.ptr(v), ctypes.c_longlong(master.numel()), ctypes.c_float(lr),
                           ctypes.c_float(beta1), ctypes.c_float(beta2), ctypes.c_float(eps),
                           ctypes.c_float(wd), ctypes.c_float(bc1), ctypes.c_float(bc2), C.ptr(state),
                           C.stream())
    C.launched(rc, "adamw")
