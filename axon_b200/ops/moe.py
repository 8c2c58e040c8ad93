"""Mixture-of-experts building blocks: routing (with routing replay), expert-sorted token layout,
grouped expert GEMMs and the weighted combine.

Layout: the ``T*k`` (token, slot) assignments are sorted by expert, token order inside an expert,
each expert's block padded to 128 rows so that every 128-row GEMM tile belongs to one expert.
``MoELayout`` carries the device-side index tensors; nothing is read back to the host.

CUDA tensors use the native kernels (csrc/moe.cu, grouped tile maps of the tcgen05 GEMM core); CPU
tensors use the PyTorch formulations below, which are also the oracles of the GPU tests. Replaces the
reference's fused-MoE Triton path (axon/utils/kernel/fused_moe.py:66-352, fused_moe_backward.py)
and routing replay / probability placement patches (axon/monkey_patches/megatron/moe_replay.py:167-401,
moe_prob_placement.py).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _common as C

PAD = 128


@dataclass
class MoELayout:
    num_tokens: int
    top_k: int
    num_experts: int
    max_rows: int                 # capacity of the sorted buffers (multiple of 128)
    counts: torch.Tensor          # int32 [E]
    offsets: torch.Tensor         # int32 [E+1], offsets[E] = padded rows in use
    tile_expert: torch.Tensor     # int32 [max_rows/128]
    row_of: torch.Tensor          # int32 [T*k]  destination row of assignment i = t*k + j
    token_of: torch.Tensor        # int32 [max_rows]  source token of a row (-1: padding)


def max_rows_for(num_tokens: int, top_k: int, num_experts: int) -> int:
    worst = num_tokens * top_k + num_experts * (PAD - 1)
    return (worst + PAD - 1) // PAD * PAD


# ------------------------------------------------------------------------------------------ routing
def route_ref(logits: torch.Tensor, top_k: int, normalize: bool = True, replay: torch.Tensor | None = None):
    p = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(p, top_k, dim=-1)
    if replay is not None:
        rp = replay.to(torch.long)
        E = logits.shape[-1]
        out_ids = torch.empty_like(ids)
        for t in range(logits.shape[0]):                    # replay slots first-come, computed ones fill the rest
            taken, row = set(), []
            pt = p[t].clone()
            for j in range(top_k):
                f = int(rp[t, j])
                if 0 <= f < E:
                    e = f
                else:
                    masked = pt.clone()
                    if taken:
                        masked[list(taken)] = -1
                    e = int(torch.argmax(masked))
                taken.add(e)
                row.append(e)
            out_ids[t] = torch.tensor(row)
        ids = out_ids
        w = p.gather(-1, ids)
    if normalize:
        w = w / w.sum(-1, keepdim=True)
    return ids.to(torch.int32), w


def route(logits: torch.Tensor, top_k: int, normalize: bool = True, replay: torch.Tensor | None = None):
    """logits fp32 [T, E] -> (ids int32 [T, k], weights fp32 [T, k])."""
    if not C.use_native(logits):
        return route_ref(logits, top_k, normalize, replay)
    T, E = logits.shape
    logits = logits.float().contiguous()
    ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    rp = replay.to(torch.int32).contiguous() if replay is not None else None
    rc = C.lib().axb_moe_route(C.ptr(logits), C.ptr(rp), C.ptr(ids), C.ptr(w), ctypes.c_longlong(T), E, top_k,
                               int(normalize), C.stream())
    C.launched(rc, "moe_route")
    return ids, w


def route_weights_from_probs(logits: torch.Tensor, ids: torch.Tensor, normalize: bool = True) -> torch.Tensor:
    """Differentiable weights of the chosen experts (for the router's backward pass)."""
    p = torch.softmax(logits.float(), dim=-1)
    w = p.gather(-1, ids.to(torch.long))
    return w / w.sum(-1, keepdim=True) if normalize else w


# ------------------------------------------------------------------------------------------ layout
def align(ids: torch.Tensor, num_experts: int) -> MoELayout:
    T, k = ids.shape
    cap = max_rows_for(T, k, num_experts)
    dev = ids.device
    if not C.use_native(ids):
        flat_all = ids.reshape(-1).to(torch.long)
        held = (flat_all >= 0) & (flat_all < num_experts)       # ids outside [0, E): experts of another rank, no row
        flat = flat_all[held]
        counts = torch.bincount(flat, minlength=num_experts).to(torch.int32)
        padded = (counts + PAD - 1) // PAD * PAD
        offsets = torch.zeros(num_experts + 1, dtype=torch.int32)
        offsets[1:] = torch.cumsum(padded, 0)
        order = torch.argsort(flat, stable=True)
        rank_in_expert = torch.empty_like(flat)
        starts = torch.cumsum(counts.to(torch.long), 0) - counts.to(torch.long)
        rank_in_expert[order] = torch.arange(flat.numel()) - starts[flat[order]]
        row_of = torch.full((flat_all.numel(),), -1, dtype=torch.int32)
        rows = (offsets[:-1].to(torch.long)[flat] + rank_in_expert)
        row_of[held] = rows.to(torch.int32)
        token_of = torch.full((cap,), -1, dtype=torch.int32)
        token_of[rows] = (torch.arange(flat_all.numel())[held] // k).to(torch.int32)
        tile_expert = torch.full((cap // PAD,), -1, dtype=torch.int32)
        for e in range(num_experts):
            tile_expert[int(offsets[e]) // PAD:int(offsets[e + 1]) // PAD] = e
        return MoELayout(T, k, num_experts, cap, counts, offsets, tile_expert, row_of, token_of)
    ids = ids.to(torch.int32).contiguous()
    counts = torch.empty(num_experts, dtype=torch.int32, device=dev)
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(cap // PAD, dtype=torch.int32, device=dev)
    row_of = torch.empty(T * k, dtype=torch.int32, device=dev)
    token_of = torch.empty(cap, dtype=torch.int32, device=dev)
    rc = C.lib().axb_moe_align(C.ptr(ids), ctypes.c_longlong(T), k, num_experts, C.ptr(counts), C.ptr(offsets),
                               C.ptr(tile_expert), cap // PAD, C.ptr(row_of), C.ptr(token_of), C.stream())
    C.launched(rc, "moe_align", 4)
    return MoELayout(T, k, num_experts, cap, counts, offsets, tile_expert, row_of, token_of)


def gather(x: torch.Tensor, lay: MoELayout) -> torch.Tensor:
    """x [T, H] -> expert-sorted rows [max_rows, H] (padding rows zero)."""
    H = x.shape[1]
    if not C.use_native(x):
        out = torch.zeros(lay.max_rows, H, dtype=x.dtype)
        live = lay.token_of >= 0
        out[live] = x[lay.token_of[live].to(torch.long)]
        return out
    xs = torch.empty(lay.max_rows, H, dtype=x.dtype, device=x.device)
    rc = C.lib().axb_moe_gather(C.ptr(x), C.ptr(lay.token_of), C.ptr(xs), ctypes.c_longlong(lay.max_rows), H, C.stream())
    C.launched(rc, "moe_gather")
    return xs


def scatter_sum(dxs: torch.Tensor, lay: MoELayout, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """Backward of ``gather``: dx[t] (+)= sum_j dxs[row_of[t, j]]."""
    T, k, H = lay.num_tokens, lay.top_k, dxs.shape[1]
    if out is None:
        out = torch.empty(T, H, dtype=dxs.dtype, device=dxs.device)
        accumulate = False
    if not C.use_native(dxs):
        s = dxs[lay.row_of.to(torch.long)].view(T, k, H).float().sum(1)
        out.copy_((out.float() + s) if accumulate else s)
        return out
    rc = C.lib().axb_moe_scatter_sum(C.ptr(dxs), C.ptr(lay.row_of), C.ptr(out), ctypes.c_longlong(T), k, H,
                                     int(accumulate), C.stream())
    C.launched(rc, "moe_scatter_sum")
    return out


def combine(ys: torch.Tensor, w: torch.Tensor, lay: MoELayout) -> torch.Tensor:
    """out[t] = sum_j w[t, j] * ys[row_of[t, j]]  (weights applied after the second projection)."""
    T, k, H = lay.num_tokens, lay.top_k, ys.shape[1]
    if not C.use_native(ys):
        rows = lay.row_of.to(torch.long)
        picked = ys[rows.clamp(min=0)].view(T, k, H).float() * (rows >= 0).view(T, k, 1)
        return (picked * w.view(T, k, 1).float()).sum(1).to(ys.dtype)
    out = torch.empty(T, H, dtype=ys.dtype, device=ys.device)
    rc = C.lib().axb_moe_combine(C.ptr(ys), C.ptr(lay.row_of), C.ptr(w.contiguous()), C.ptr(out), ctypes.c_longlong(T), k, H,
                                 C.stream())
    C.launched(rc, "moe_combine")
    return out


def combine_bwd(dout: torch.Tensor, ys: torch.Tensor, w: torch.Tensor, lay: MoELayout):
    """-> (dys [max_rows, H] with zero padding rows, dw fp32 [T, k])."""
    T, k, H = lay.num_tokens, lay.top_k, ys.shape[1]
    if not C.use_native(ys):
        rows = lay.row_of.to(torch.long)
        dys = torch.zeros_like(ys)
        dys[rows] = (dout.float().repeat_interleave(k, 0) * w.reshape(-1, 1).float()).to(ys.dtype)
        dw = (dout.float().repeat_interleave(k, 0) * ys[rows].float()).sum(-1).view(T, k)
        return dys, dw
    dys = torch.zeros_like(ys)
    dw = torch.empty(T, k, dtype=torch.float32, device=ys.device)
    rc = C.lib().axb_moe_combine_bwd(C.ptr(dout), C.ptr(ys), C.ptr(lay.row_of), C.ptr(w.contiguous()), C.ptr(dys), C.ptr(dw),
                                     ctypes.c_longlong(T), k, H, C.stream())
    C.launched(rc, "moe_combine_bwd")
    return dys, dw


# ------------------------------------------------------------------------------------ grouped GEMMs
def _expert_rows(lay: MoELayout):
    off = lay.offsets.tolist()
    return [(e, off[e], off[e + 1]) for e in range(lay.num_experts) if off[e + 1] > off[e]]


def grouped_fwd(xs: torch.Tensor, w: torch.Tensor, lay: MoELayout) -> torch.Tensor:
    """xs [P, K] (sorted), w [E, N, K] -> ys [P, N]."""
    E, N, K = w.shape
    if not C.use_native(xs):
        ys = torch.zeros(xs.shape[0], N, dtype=xs.dtype)
        for e, a, b in _expert_rows(lay):
            ys[a:b] = (xs[a:b].float() @ w[e].float().t()).to(xs.dtype)
        return ys
    ys = torch.empty(xs.shape[0], N, dtype=xs.dtype, device=xs.device)
    rc = C.lib().axb_gemm_grouped_fwd(C.ptr(xs), C.ptr(w), C.ptr(ys), xs.shape[0], N, K, E, ctypes.c_longlong(xs.stride(0)),
                                      ctypes.c_longlong(K), ctypes.c_longlong(N), C.ptr(lay.tile_expert),
                                      C.ptr(lay.offsets[E:]), C.ptr(C.status(xs.device)), C.stream())
    C.launched(rc, "gemm_grouped_fwd")
    return ys


def grouped_dgrad(dys: torch.Tensor, w: torch.Tensor, lay: MoELayout) -> torch.Tensor:
    """dys [P, N], w [E, N, K] -> dxs [P, K]."""
    E, N, K = w.shape
    if not C.use_native(dys):
        dxs = torch.zeros(dys.shape[0], K, dtype=dys.dtype)
        for e, a, b in _expert_rows(lay):
            dxs[a:b] = (dys[a:b].float() @ w[e].float()).to(dys.dtype)
        return dxs
    dxs = torch.empty(dys.shape[0], K, dtype=dys.dtype, device=dys.device)
    rc = C.lib().axb_gemm_grouped_dgrad(C.ptr(dys), C.ptr(w), C.ptr(dxs), dys.shape[0], N, K, E,
                                        ctypes.c_longlong(dys.stride(0)), ctypes.c_longlong(K), ctypes.c_longlong(K),
                                        C.ptr(lay.tile_expert), C.ptr(lay.offsets[E:]), C.ptr(C.status(dys.device)), C.stream())
    C.launched(rc, "gemm_grouped_dgrad")
    return dxs


def grouped_wgrad(dys: torch.Tensor, xs: torch.Tensor, dw: torch.Tensor, lay: MoELayout, accumulate: bool = True) -> torch.Tensor:
    """dw [E, N, K] fp32 (+)= dys_e^T xs_e for every expert that has rows (others are left untouched)."""
    E, N, K = dw.shape
    if not C.use_native(dys):
        for e, a, b in _expert_rows(lay):
            g = dys[a:b].float().t() @ xs[a:b].float()
            dw[e] = dw[e] + g if accumulate else g
        return dw
    rc = C.lib().axb_gemm_grouped_wgrad(C.ptr(dys), C.ptr(xs), C.ptr(dw), dys.shape[0], N, K, E,
                                        ctypes.c_longlong(dys.stride(0)), ctypes.c_longlong(xs.stride(0)), C.ptr(lay.offsets),
                                        int(accumulate), C.ptr(C.status(dys.device)), C.stream())
    C.launched(rc, "gemm_grouped_wgrad")
    return dw
