"""RMSNorm (optionally fused with the residual add) forward/backward.

Native kernels on CUDA, PyTorch fp32 math on CPU. Equivalent of the TE / HF RMSNorm modules the
reference relies on (fusions listed in recipes/frozenlake/train_frozenlake_qwen_30b_a3b.yaml:138-148).
"""
from __future__ import annotations

import ctypes

import torch

from . import _common as C


def rmsnorm_fwd(x, w, eps: float, delta=None):
    """Returns (y, rstd, xsum). ``xsum = x + delta`` (new residual stream) when delta is given, else x."""
    T, H = x.shape
    if not C.use_native(x):
        xs = x if delta is None else (x.float() + delta.float()).to(x.dtype)
        xf = xs.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
        y = (xf * rstd[:, None] * w.float()).to(x.dtype)
        return y, rstd, xs
    y = torch.empty_like(x)
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    xsum = torch.empty_like(x) if delta is not None else None
    rc = C.lib().axb_rmsnorm_fwd(C.ptr(x), C.ptr(delta), C.ptr(w), C.ptr(xsum), C.ptr(y), C.ptr(rstd),
                                 ctypes.c_longlong(T), H, ctypes.c_float(eps), C.stream())
    C.launched(rc, "rmsnorm_fwd")
    return y, rstd, (xsum if delta is not None else x)


def rmsnorm_bwd(dy, x, w, rstd, dw, dres=None, accumulate_dw: bool = True):
    """dx = dres + d(rmsnorm)/dx ; dw (+)= sum_t dy * xhat. dw is fp32 [H]."""
    T, H = x.shape
    if not C.use_native(x):
        xh = x.float() * rstd[:, None]
        g = dy.float() * w.float()
        dx = rstd[:, None] * (g - xh * (g * xh).mean(-1, keepdim=True))
        if dres is not None:
            dx = dx + dres.float()
        dwn = (dy.float() * xh).sum(0)
        dw.copy_(dw + dwn if accumulate_dw else dwn)
        return dx.to(x.dtype)
    lib = C.lib()
    P = lib.axb_rmsnorm_bwd_partials(ctypes.c_longlong(T))
    scratch = C.workspace(x.device, P * H * 4, "norm")
    dx = torch.empty_like(x)
    rc = lib.axb_rmsnorm_bwd(C.ptr(dy), C.ptr(x), C.ptr(w), C.ptr(rstd), C.ptr(dres), C.ptr(dx), C.ptr(dw),
                             int(accumulate_dw), C.ptr(scratch), ctypes.c_longlong(T), H, C.stream())
    C.launched(rc, "rmsnorm_bwd", 2)
    return dx
