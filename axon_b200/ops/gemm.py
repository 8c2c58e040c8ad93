"""bf16 GEMM on the tcgen05 tensor cores (native) with a PyTorch reference for CPU tensors.

``gemm(a, b, trans_a, trans_b)`` computes ``op(a) @ op(b)^T``-style products without ever
materialising a transpose: the kernel reads K-major or MN-major operands straight from their
row-major storage. The three products a linear layer needs are exposed as
``linear_fwd`` (y = x Wᵀ), ``linear_dgrad`` (dx = dy W) and ``linear_wgrad`` (dW (+)= dyᵀ x).
Replaces the cuBLAS / TransformerEngine calls behind ``torch.nn.Linear`` in the reference
(FSDP path ``axon/trainer/fsdp_trainer.py:362-422``).
"""
from __future__ import annotations

import ctypes

import torch

from . import _common as C

OUT_BF16, OUT_F32, ACC_F32, ACC_BF16 = 0, 1, 2, 3


def _native_gemm(a, b, out, M, N, K, a_mn, b_mn, mode, alpha=1.0, bn_hint=0, max_ctas=0):
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and out.stride(-1) == 1
    rc = C.lib().axb_gemm_bf16(
        C.ptr(a), C.ptr(b), C.ptr(out), M, N, K,
        ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(b.stride(0)), ctypes.c_longlong(out.stride(0)),
        int(a_mn), int(b_mn), int(mode), ctypes.c_float(alpha), int(bn_hint), int(max_ctas),
        C.ptr(C.status(a.device)), C.stream())
    C.launched(rc, "gemm_bf16")
    return out


SMALL_M = 256  # token batches up to this size take the swap-AB + split-K path (decode)


FIXED_CONFIG = False        # batch-invariant mode: one tile width, no K split, whatever the batch size
USE_CLUSTER_DECODE = True   # cluster split-K kernel (partials reduced through distributed shared memory)


def _native_gemm_smallm(x, w, out, M, N, K):
    lib = C.lib()
    if USE_CLUSTER_DECODE and lib.axb_gemm_decode_cluster_size(M, N, K) >= 2:
        rc = lib.axb_gemm_decode_cluster(C.ptr(x), C.ptr(w), C.ptr(out), M, N, K, ctypes.c_longlong(x.stride(0)),
                                         ctypes.c_longlong(w.stride(0)), ctypes.c_longlong(out.stride(0)),
                                         int(out.dtype == torch.float32), C.ptr(C.status(x.device)), C.stream())
        C.launched(rc, "gemm_decode_cluster", 1)
        return out
    splits = lib.axb_gemm_smallm_splits(M, N, K)
    ws = C.workspace(x.device, splits * M * N * 4, "gemm_splitk") if splits > 1 else None
    rc = lib.axb_gemm_bf16_smallm(C.ptr(x), C.ptr(w), C.ptr(out), M, N, K, ctypes.c_longlong(x.stride(0)),
                                  ctypes.c_longlong(w.stride(0)), ctypes.c_longlong(out.stride(0)),
                                  int(out.dtype == torch.float32), C.ptr(ws), C.ptr(C.status(x.device)), C.stream())
    C.launched(rc, "gemm_bf16_smallm", 2 if splits > 1 else 1)
    return out


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None,
            out_dtype=None, accumulate: bool = False, alpha: float = 1.0,
            bn_hint: int = 0, max_ctas: int = 0) -> torch.Tensor:
    """``out[M,N] (+)= alpha * a[M,K] @ b[N,K]^T``."""
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
        assert not accumulate
    if not C.use_native(a):
        r = alpha * (a.float() @ b.float().t())
        out.copy_(out.float() + r if accumulate else r)
        return out
    if FIXED_CONFIG:
        bn_hint = bn_hint or 128
    elif M <= SMALL_M and not accumulate and alpha == 1.0 and bn_hint == 0 and N >= 512:
        return _native_gemm_smallm(a, b, out, M, N, K)
    mode = {torch.bfloat16: ACC_BF16 if accumulate else OUT_BF16,
            torch.float32: ACC_F32 if accumulate else OUT_F32}[out.dtype]
    return _native_gemm(a, b, out, M, N, K, 0, 0, mode, alpha, bn_hint, max_ctas)


def gemm_nn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None,
            out_dtype=None, accumulate: bool = False, alpha: float = 1.0) -> torch.Tensor:
    """``out[M,N] (+)= alpha * a[M,K] @ b[K,N]`` (b is read MN-major, no transpose)."""
    M, K = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
        assert not accumulate
    if not C.use_native(a):
        r = alpha * (a.float() @ b.float())
        out.copy_(out.float() + r if accumulate else r)
        return out
    mode = {torch.bfloat16: ACC_BF16 if accumulate else OUT_BF16,
            torch.float32: ACC_F32 if accumulate else OUT_F32}[out.dtype]
    return _native_gemm(a, b, out, M, N, K, 0, 1, mode, alpha)


def gemm_tn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None,
            out_dtype=None, accumulate: bool = False, alpha: float = 1.0) -> torch.Tensor:
    """``out[M,N] (+)= alpha * a[K,M]^T @ b[K,N]`` (both operands read MN-major)."""
    K, M = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
        assert not accumulate
    if not C.use_native(a):
        r = alpha * (a.float().t() @ b.float())
        out.copy_(out.float() + r if accumulate else r)
        return out
    mode = {torch.bfloat16: ACC_BF16 if accumulate else OUT_BF16,
            torch.float32: ACC_F32 if accumulate else OUT_F32}[out.dtype]
    return _native_gemm(a, b, out, M, N, K, 1, 1, mode, alpha)


def linear_fwd(x, w, out=None, out_dtype=None):
    """y[T,out] = x[T,in] @ w[out,in]^T."""
    return gemm_nt(x, w, out=out, out_dtype=out_dtype)


def linear_dgrad(dy, w, out=None, accumulate=False):
    """dx[T,in] = dy[T,out] @ w[out,in]."""
    return gemm_nn(dy, w, out=out, accumulate=accumulate)


def linear_wgrad(dy, x, out=None, out_dtype=torch.float32, accumulate=False):
    """dw[out,in] (+)= dy[T,out]^T @ x[T,in]."""
    return gemm_tn(dy, x, out=out, out_dtype=out_dtype, accumulate=accumulate)
