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


STREAM_MAX_M = 128
USE_STREAM_DECODE = True    # weight-streaming kernel (run-time token width, last-arriver split-K reduction)
_STREAM_PLANS: dict = {}
_STREAM_COUNTERS: dict = {}
_STREAM_ACC: dict = {}
_STREAM_TUNE_VERSION = 0


_STREAM_KNOBS = {"force_splits": 0, "max_bn": 1, "ring_kb_one": 2, "ring_kb_two": 3, "two_per_sm_tiles": 4, "x_depth": 5,
                 "min_kblocks": 6, "pdl": 7, "accumulate": 8}
STREAM_DEFAULTS = dict(force_splits=0, max_bn=128, ring_kb_one=208, ring_kb_two=104, two_per_sm_tiles=1, x_depth=0,
                       min_kblocks=8, pdl=1, accumulate=1)


def stream_tune(**knobs) -> None:
    """Experiment hook: set planning knobs of the weight-streaming kernel (names of ``STREAM_DEFAULTS``;
    ``accumulate``: 1 = split-K partials added by L2 reductions, 0 = summed in split order, bit-reproducible)."""
    global _STREAM_TUNE_VERSION
    for k, v in knobs.items():
        C.lib().axb_gemm_stream_knob(_STREAM_KNOBS[k], int(v))
    _STREAM_TUNE_VERSION += 1


def _native_gemm_stream(x, w, out, M, N, K):
    lib = C.lib()
    key = (M, N, K, _STREAM_TUNE_VERSION)
    plan = _STREAM_PLANS.get(key)
    if plan is None:
        wsf, nc, sp, bn, zr = ctypes.c_longlong(0), ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
        rc = lib.axb_gemm_stream_workspace(M, N, K, ctypes.byref(wsf), ctypes.byref(nc), ctypes.byref(sp), ctypes.byref(bn), ctypes.byref(zr))
        C.launched(rc, "gemm_stream_workspace", 0)
        plan = _STREAM_PLANS[key] = (wsf.value, nc.value, sp.value, bn.value, zr.value)
    ws_floats, n_counters, splits, _, zeroed = plan
    ws = cnt = None
    if splits > 1:
        if zeroed:      # accumulation tiles: zero once, every launch leaves them zero
            ws = _STREAM_ACC.get(x.device.index)
            if ws is None or ws.numel() < ws_floats:
                ws = _STREAM_ACC[x.device.index] = torch.zeros(max(1 << 22, 2 * ws_floats), dtype=torch.float32, device=x.device)
        else:
            ws = C.workspace(x.device, ws_floats * 4, "gemm_stream")
        cnt = _STREAM_COUNTERS.get(x.device.index)
        if cnt is None or cnt.numel() < n_counters:
            cnt = _STREAM_COUNTERS[x.device.index] = torch.zeros(max(4096, 2 * n_counters), dtype=torch.int32, device=x.device)
    rc = lib.axb_gemm_stream(C.ptr(x), C.ptr(w), C.ptr(out), M, N, K, ctypes.c_longlong(x.stride(0)),
                             ctypes.c_longlong(w.stride(0)), ctypes.c_longlong(out.stride(0)),
                             int(out.dtype == torch.float32), C.ptr(ws), C.ptr(cnt), C.ptr(C.status(x.device)), C.stream())
    C.launched(rc, "gemm_stream", 1)
    return out


def _native_gemm_smallm(x, w, out, M, N, K):
    lib = C.lib()
    # up to 128 tokens (one token tile) the weight-streaming kernel wins; above, the two-tile plan re-reads W
    # and the cluster / split-K kernels below measured faster inside the decode graph
    if USE_STREAM_DECODE and M <= STREAM_MAX_M and N % 4 == 0 and out.stride(0) % 4 == 0 and x.stride(0) % 8 == 0 \
            and w.stride(0) % 8 == 0:
        return _native_gemm_stream(x, w, out, M, N, K)
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
