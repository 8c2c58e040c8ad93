"""Weight quantisers for low-precision samplers: fp8 128x128 blocks, int4 groups (packed), mxfp8.

CUDA tensors go through the native kernels; CPU tensors (and the oracles of the GPU tests) use the
PyTorch formulations below, which define the formats (reference formats: axon/utils/sglang/fp8.py,
int4.py:61-307, mxfp8.py:81-119 and axon/monkey_patches/vllm/fp8/vllm_fp8_patch.py:1211-1261).
"""
from __future__ import annotations

import ctypes

import torch

from . import _common as C

MXFP8_GROUP = 32


# ------------------------------------------------------------------------------------------- int4
def int4_group_quant_ref(w: torch.Tensor, group_size: int = 128):
    """(q int8 in [-8, 7], scale in w.dtype [M, N/group]). scale = max(absmax/7, 1e-5), round half even."""
    M, N = w.shape
    g = w.float().reshape(M, N // group_size, group_size)
    scale = (g.abs().amax(-1, keepdim=True) / 7.0).clamp(min=1e-5)
    q = torch.round(g / scale).clamp(-8, 7).to(torch.int8).reshape(M, N)
    return q, scale.squeeze(-1).to(w.dtype)


def pack_int4_to_int32(q: torch.Tensor) -> torch.Tensor:
    """Eight signed 4-bit values per int32 along the last dim, value i in bits 4i..4i+3, stored +8."""
    M, N = q.shape
    assert N % 8 == 0
    u = (q.to(torch.int32) + 8).reshape(M, N // 8, 8) & 0xF
    shifts = torch.arange(8, dtype=torch.int32, device=q.device) * 4
    word = (u.to(torch.int64) << shifts.to(torch.int64)).sum(-1)
    return torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)


def unpack_int32_to_int4(packed: torch.Tensor) -> torch.Tensor:
    shifts = torch.arange(8, dtype=torch.int64, device=packed.device) * 4
    u = (packed.to(torch.int64).unsqueeze(-1) >> shifts) & 0xF
    return (u - 8).to(torch.int8).reshape(packed.shape[0], -1)


def int4_quant_pack(w: torch.Tensor, group_size: int = 128):
    """bf16 [M, N] -> (packed int32 [M, N/8], scales [M, N/group]) in one pass."""
    assert w.dim() == 2 and w.shape[1] % group_size == 0 and w.shape[1] % 8 == 0
    if not (C.use_native(w) and w.dtype == torch.bfloat16 and group_size in (32, 64, 128)):
        q, s = int4_group_quant_ref(w, group_size)
        return pack_int4_to_int32(q), s
    M, N = w.shape
    w = w if w.stride(1) == 1 else w.contiguous()
    packed = torch.empty(M, N // 8, dtype=torch.int32, device=w.device)
    scales = torch.empty(M, N // group_size, dtype=torch.bfloat16, device=w.device)
    rc = C.lib().axb_int4_group_quant_pack(C.ptr(w), C.ptr(packed), C.ptr(scales), ctypes.c_longlong(M), N,
                                           ctypes.c_longlong(w.stride(0)), group_size, C.stream())
    C.launched(rc, "int4_group_quant_pack")
    return packed, scales


def int4_dequant(packed: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    q = unpack_int32_to_int4(packed).float()
    return (q.reshape(q.shape[0], -1, group_size) * scales.float().unsqueeze(-1)).reshape(q.shape[0], -1)


# ------------------------------------------------------------------------------------------ mxfp8
def mxfp8_quant_ref(w: torch.Tensor):
    """(e4m3 [M, N], UE8M0 uint8 [M, N/32]): the shared scale is the smallest power of two 2^e with
    absmax / 2^e <= 448 (e clamped to [-127, 127], all-zero groups use e = -127)."""
    M, N = w.shape
    g = w.float().reshape(M, N // MXFP8_GROUP, MXFP8_GROUP)
    amax = g.abs().amax(-1)
    e = torch.ceil(torch.log2(amax / 448.0))
    e = torch.where(amax > 448.0 * torch.exp2(e), e + 1, e)
    e = torch.where((amax <= 448.0 * torch.exp2(e - 1)) & (e > -127), e - 1, e)
    e = torch.where((amax > 0) & torch.isfinite(amax), e, torch.full_like(e, -127.0)).clamp(-127, 127)
    q = (g * torch.exp2(-e).unsqueeze(-1)).clamp(-448, 448).reshape(M, N).to(torch.float8_e4m3fn)
    return q, (e + 127).to(torch.uint8)


def mxfp8_quant(w: torch.Tensor):
    assert w.dim() == 2 and w.shape[1] % MXFP8_GROUP == 0
    if not (C.use_native(w) and w.dtype == torch.bfloat16):
        return mxfp8_quant_ref(w)
    M, N = w.shape
    w = w if w.stride(1) == 1 else w.contiguous()
    q = torch.empty(M, N, dtype=torch.float8_e4m3fn, device=w.device)
    s = torch.empty(M, N // MXFP8_GROUP, dtype=torch.uint8, device=w.device)
    rc = C.lib().axb_mxfp8_quant(C.ptr(w), C.ptr(q), C.ptr(s), ctypes.c_longlong(M), N, ctypes.c_longlong(w.stride(0)), C.stream())
    C.launched(rc, "mxfp8_quant")
    return q, s


def mxfp8_dequant(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    M, N = q.shape
    e = scales.float() - 127.0
    return (q.float().reshape(M, N // MXFP8_GROUP, MXFP8_GROUP) * torch.exp2(e).unsqueeze(-1)).reshape(M, N)


# -------------------------------------------------------------------------------------- fp8 blocks
def fp8_block_quant(w: torch.Tensor):
    """128x128 blocks: (e4m3 [M, N], fp32 scales [ceil(M/128), ceil(N/128)]), dequant = q * scale."""
    from ..utils.p2p.plan import fp8_block_quant_ref
    if not (C.use_native(w) and w.dtype == torch.bfloat16):
        return fp8_block_quant_ref(w)
    M, N = w.shape
    w = w if w.stride(1) == 1 else w.contiguous()
    q = torch.empty(M, N, dtype=torch.float8_e4m3fn, device=w.device)
    s = torch.empty((M + 127) // 128, (N + 127) // 128, dtype=torch.float32, device=w.device)
    rc = C.lib().axb_fp8_block_quant(C.ptr(w), C.ptr(q), C.ptr(s), M, N, ctypes.c_longlong(w.stride(0)),
                                     ctypes.c_longlong(q.stride(0)), C.stream())
    C.launched(rc, "fp8_block_quant")
    return q, s


def fp8_block_dequant(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    M, N = q.shape
    s = scales.repeat_interleave(128, 0)[:M].repeat_interleave(128, 1)[:, :N]
    return q.float() * s
