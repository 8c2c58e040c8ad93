"""Ulysses sequence parallelism: the sequence <-> head exchange around attention.

Ranks of a sequence-parallel group hold the same packed batch, each working on ``T / W`` of its tokens
with full weights; attention needs every token of a sequence, so heads are dealt out instead:
``[T/W, all heads] -> [T, heads/W]`` before the kernel, the inverse after it (reference:
``SeqAllToAll`` / ``gather_seq_scatter_heads`` / ``gather_heads_scatter_seq``, axon/utils/ulysses.py:133-192,
used by ``_ulysses_flash_attention_forward``, axon/monkey_patches/transformers/monkey_patch.py:48-117).

On NVLink the exchange is one peer-store kernel per direction (``csrc/ulysses.cu``): q, k and v travel
together and land in the attention kernel's layout; two symmetric buffers per direction alternate, so
a buffer is rewritten only after a further barrier has shown that every peer is past reading it.
On CPU / gloo the same index maps run on an all-gather (host-side logic and tests).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _common as C
from .symm import PeerBarrier, SymmetricBuffer


class UlyssesContext:
    def __init__(self, group, device, max_rows_per_rank: int, max_width: int, fused: bool | None = None):
        """``max_rows_per_rank``: local tokens per exchange at most; ``max_width``: widest row (q|k|v of all heads)."""
        live = dist.is_initialized() and group is not None
        self.group = group
        self.world = dist.get_world_size(group) if live else 1
        self.rank = dist.get_rank(group) if live else 0
        self.device = torch.device(device)
        if fused is None:
            fused = self.world > 1 and self.device.type == "cuda" and dist.get_backend(group) == "nccl"
        self.fused = bool(fused)
        self.cap = max_rows_per_rank * max_width
        if self.fused:
            assert self.world <= 8
            self.bufs = {kind: [SymmetricBuffer(self.cap, torch.bfloat16, group, self.device) for _ in range(2)] for kind in ("cols", "rows")}
            self.turn = {"cols": 0, "rows": 0}
            self.barrier = PeerBarrier(group, self.device)
            self._sync = torch.zeros(1, device=self.device)

    # ------------------------------------------------------------------ the two index maps
    def scatter_cols(self, x: torch.Tensor, segs: list[tuple[int, int, int]], out_width: int, copy: bool = True) -> torch.Tensor:
        """x [rows, ld] on every rank -> [W * rows, out_width]:
        ``out[r * rows + t, dst + c] = x_r[t, src + me * w + c]`` for every segment (src, w, dst)."""
        return self._exchange("cols", x, segs, out_width, copy)

    def scatter_rows(self, x: torch.Tensor, segs: list[tuple[int, int, int]], out_width: int, copy: bool = True) -> torch.Tensor:
        """x [W * rows, ld] on every rank -> [rows, out_width]:
        ``out[t, dst + r * w + c] = x_r[me * rows + t, src + c]``."""
        return self._exchange("rows", x, segs, out_width, copy)

    def _exchange(self, kind: str, x: torch.Tensor, segs, out_width: int, copy: bool) -> torch.Tensor:
        W, me = self.world, self.rank
        by_rows = kind == "rows"
        rows = x.shape[0] // W if by_rows else x.shape[0]
        out_rows = rows if by_rows else W * rows
        if W == 1:
            out = torch.empty(out_rows, out_width, dtype=x.dtype, device=x.device)
            for s, w, d in segs:
                out[:, d:d + w] = x[:, s:s + w]
            return out
        if not self.fused:
            parts = [torch.empty_like(x) for _ in range(W)]
            dist.all_gather(parts, x.contiguous(), group=self.group)
            out = torch.empty(out_rows, out_width, dtype=x.dtype, device=x.device)
            for r, xr in enumerate(parts):
                for s, w, d in segs:
                    if by_rows:
                        out[:, d + r * w:d + (r + 1) * w] = xr[me * rows:(me + 1) * rows, s:s + w]
                    else:
                        out[r * rows:(r + 1) * rows, d:d + w] = xr[:, s + me * w:s + (me + 1) * w]
            return out
        assert x.dtype == torch.bfloat16 and x.stride(-1) == 1
        assert out_rows * out_width <= self.cap, f"exchange of {out_rows} x {out_width} exceeds the symmetric buffers ({self.cap} elements)"
        i = self.turn[kind]
        self.turn[kind] = i ^ 1
        buf = self.bufs[kind][i]
        flat = (ctypes.c_int * (3 * len(segs)))(*[v for sg in segs for v in sg])
        rc = C.lib().axb_ulysses_scatter(C.ptr(x), ctypes.c_longlong(x.stride(0)), buf.ptr_array(), ctypes.c_longlong(out_width),
                                         W, me, rows, flat, len(segs), int(by_rows), C.stream())
        C.launched(rc, "ulysses_scatter")
        dist.all_reduce(self._sync, group=self.group)       # line the streams up (the device barrier's wait is bounded)
        self.barrier()
        out = buf.tensor[: out_rows * out_width].view(out_rows, out_width)
        return out.clone() if copy else out

    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(self.world)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts)
