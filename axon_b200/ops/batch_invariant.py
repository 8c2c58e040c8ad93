"""Batch-invariant mode: results for one row never depend on the other rows of the batch
(reference: axon/monkey_patches/vllm/batch_invariant_ops.py:81-512, which swaps aten mm / addmm /
log_softmax / mean for persistent Triton kernels).

The kernels here are deterministic already (fixed tile rasterisation, no atomics in reductions). What
can still differ between batch sizes is the *configuration*: the small-batch GEMM path picks its tile
width and its K split from the number of tokens, which changes the order in which K is summed. Inside
``batch_invariant_mode()`` every ``gemm_nt`` uses one fixed configuration (128-wide tiles, no split),
and ``log_softmax`` / ``mean_dim`` below use one block per row with a fixed-order reduction.
"""
from __future__ import annotations

import ctypes
from contextlib import contextmanager

import torch

from . import _common as C
from . import gemm as G

_ENABLED = False


def is_batch_invariant_mode_enabled() -> bool:
    return _ENABLED


def enable_batch_invariant_mode() -> None:
    global _ENABLED
    if not _ENABLED:
        _ENABLED = True
        G.FIXED_CONFIG = True


def disable_batch_invariant_mode() -> None:
    global _ENABLED
    _ENABLED = False
    G.FIXED_CONFIG = False


@contextmanager
def batch_invariant_mode(enabled: bool = True):
    prev = _ENABLED
    (enable_batch_invariant_mode if enabled else disable_batch_invariant_mode)()
    try:
        yield
    finally:
        (enable_batch_invariant_mode if prev else disable_batch_invariant_mode)()


def _rows(x: torch.Tensor):
    x2 = x.reshape(-1, x.shape[-1])
    return x2 if x2.stride(-1) == 1 else x2.contiguous()


def log_softmax(x: torch.Tensor) -> torch.Tensor:
    """fp32 log-softmax over the last dim."""
    if not (C.use_native(x) and x.dtype in (torch.float32, torch.bfloat16)):
        return torch.log_softmax(x.float(), dim=-1)
    x2 = _rows(x)
    out = torch.empty(x2.shape, dtype=torch.float32, device=x.device)
    rc = C.lib().axb_log_softmax_rows(C.ptr(x2), int(x.dtype == torch.bfloat16), C.ptr(out), ctypes.c_longlong(x2.shape[0]),
                                      x2.shape[1], ctypes.c_longlong(x2.stride(0)), C.stream())
    C.launched(rc, "log_softmax_rows")
    return out.view(x.shape)


def mean_dim(x: torch.Tensor) -> torch.Tensor:
    """fp32 mean over the last dim."""
    if not (C.use_native(x) and x.dtype in (torch.float32, torch.bfloat16)):
        return x.float().mean(-1)
    x2 = _rows(x)
    out = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    rc = C.lib().axb_mean_rows(C.ptr(x2), int(x.dtype == torch.bfloat16), C.ptr(out), ctypes.c_longlong(x2.shape[0]),
                               x2.shape[1], ctypes.c_longlong(x2.stride(0)), C.stream())
    C.launched(rc, "mean_rows")
    return out.view(x.shape[:-1])
