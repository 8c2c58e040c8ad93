"""Context parallelism: every sequence is cut over the ranks of a group, attention sees all of it.

Reference: ``context_parallel_size`` of the Megatron trainer (axon/trainer/megatron_trainer.py; batches cut by
``get_batch_on_this_cp_rank`` style zigzag slicing in axon/utils/megatron/, attention through
TransformerEngine's ring exchange of K/V).

Layout. A sequence (padded to a multiple of ``2 W`` tokens) is cut into ``2 W`` chunks; rank ``r`` holds
chunks ``r`` and ``2 W - 1 - r`` ("zigzag"), so causal work is the same on every rank. Local tokens are
stored half-major - first chunk ``r`` of every sequence, then chunk ``2 W - 1 - r`` of every sequence - which
makes each half a packed batch with cumulative lengths ``cu / (2 W)``.

Exchange. NVSwitch gives every rank full bandwidth to every peer, so instead of W - 1 ring hops each rank
pushes its K|V rows once into every peer's symmetric buffer (one launch of the strided peer-copy plan
kernel of ``csrc/comm.cu``), and attention then runs block by block from local memory: the diagonal
blocks causal, earlier chunks unmasked, later chunks skipped, partial results merged through their
log-sum-exp. Backward recomputes the gather, runs the block backward against the merged output and
log-sum-exp, and returns the K|V gradient partials to their owners the same way (push, then a local sum in
fp32). On CPU / gloo the pushes become all-gather / all-reduce, so the block logic is testable anywhere.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from ..ops import attention as AT
from .symm import PeerBarrier, SymmetricBuffer


def chunk_id(rank: int, half: int, world: int) -> int:
    return rank if half == 0 else 2 * world - 1 - rank


def pad_layout(cu_seqlens: torch.Tensor, world: int, token_multiple: int = 128):
    """Per-sequence padding to a multiple of ``2 W`` plus one dummy sequence so that every rank gets a
    multiple of ``token_multiple`` tokens. Returns (cu of the padded batch [B'+1], positions of the
    original tokens inside the padded batch [T], offset of every padded token in its sequence [T'])."""
    cu = cu_seqlens.to("cpu", torch.int64)
    lens = cu[1:] - cu[:-1]
    m = 2 * world
    plens = (lens + m - 1) // m * m
    extra = int((-int(plens.sum())) % (token_multiple * world))
    if extra:
        plens = torch.cat([plens, torch.tensor([extra])])
        lens = torch.cat([lens, torch.tensor([0])])
    new_cu = torch.cat([torch.zeros(1, dtype=torch.int64), plens.cumsum(0)])
    seq = torch.repeat_interleave(torch.arange(plens.numel()), plens)
    off = torch.arange(int(new_cu[-1])) - new_cu[seq]
    valid = off < lens[seq]
    orig_pos = torch.nonzero(valid).flatten()
    return new_cu, orig_pos, off


def local_index(new_cu: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Positions (in the padded batch) of rank ``rank``'s tokens, half-major."""
    m = 2 * world
    cl = (new_cu[1:] - new_cu[:-1]) // m
    cu_half = torch.cat([torch.zeros(1, dtype=torch.int64), cl.cumsum(0)])
    seq = torch.repeat_interleave(torch.arange(cl.numel()), cl)
    off = torch.arange(int(cu_half[-1])) - cu_half[seq]
    parts = [new_cu[seq] + chunk_id(rank, h, world) * cl[seq] + off for h in (0, 1)]
    return torch.cat(parts)


class ContextParallel:
    """K|V all-gather and K|V-gradient return over one context-parallel group."""

    def __init__(self, group, device, max_local_tokens: int, kv_width: int, fused: bool | None = None):
        live = dist.is_initialized() and group is not None
        self.group = group
        self.world = dist.get_world_size(group) if live else 1
        self.rank = dist.get_rank(group) if live else 0
        self.device = torch.device(device)
        if fused is None:
            fused = self.world > 1 and self.device.type == "cuda" and dist.get_backend(group) == "nccl"
        self.fused = bool(fused)
        self.kv_width = kv_width
        self.cap = max_local_tokens
        self._plans: dict = {}
        if self.fused:
            assert self.world <= 8 and kv_width % 8 == 0
            n = self.world * max_local_tokens * kv_width
            # two buffers per direction alternate: a buffer is rewritten only after a further barrier has
            # shown that every peer is past reading it
            self.bufs = {k: [SymmetricBuffer(n, torch.bfloat16, group, self.device) for _ in range(2)] for k in ("kv", "dkv")}
            self.turn = {"kv": 0, "dkv": 0}
            self.barrier = PeerBarrier(group, self.device)
            self._sync = torch.zeros(1, device=self.device)

    # ------------------------------------------------------------------ pushes
    def _push(self, kind: str, src: torch.Tensor, descs_key, make_descs) -> torch.Tensor:
        from ..utils.p2p.plan import execute_plan, plan_from_descs
        plan = self._plans.get(descs_key)
        if plan is None:
            plan = self._plans[descs_key] = plan_from_descs(make_descs())
        i = self.turn[kind]
        self.turn[kind] = i ^ 1
        buf = self.bufs[kind][i]
        execute_plan(plan, src, [None] * self.world, dst_ptrs=buf.ptrs)
        dist.all_reduce(self._sync, group=self.group)       # line the streams up (the device barrier's wait is bounded)
        self.barrier()
        return buf.tensor

    def gather_kv(self, qkv: torch.Tensor, col0: int) -> torch.Tensor:
        """qkv [n, ld] on every rank -> [W, n, kv_width]: rank r's columns ``col0 : col0 + kv_width``."""
        W, me, n, kw = self.world, self.rank, qkv.shape[0], self.kv_width
        if W == 1:
            return qkv[:, col0:col0 + kw].unsqueeze(0)
        if not self.fused:
            mine = qkv[:, col0:col0 + kw].contiguous()
            parts = [torch.empty_like(mine) for _ in range(W)]
            dist.all_gather(parts, mine, group=self.group)
            return torch.stack(parts)
        from ..utils.p2p.plan import copy_desc
        assert n <= self.cap and qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and col0 % 8 == 0
        ld = qkv.stride(0)
        out = self._push("kv", qkv, ("kv", n, ld, col0),
                         lambda: [copy_desc(col0, me * n * kw, n, kw, ld, kw, d) for d in range(W)])
        return out[: W * n * kw].view(W, n, kw)

    def return_dkv(self, dkv_all: torch.Tensor) -> torch.Tensor:
        """dkv_all [W, n, kv_width] (this rank's partial gradient of every rank's K|V rows) -> fp32
        [n, kv_width]: the sum over ranks of the partials of this rank's rows."""
        W, me, n, kw = self.world, self.rank, dkv_all.shape[1], self.kv_width
        if W == 1:
            return dkv_all[0].float()
        if not self.fused:
            full = dkv_all.float().contiguous()
            dist.all_reduce(full, group=self.group)
            return full[me]
        from ..utils.p2p.plan import copy_desc
        src = dkv_all.to(torch.bfloat16).contiguous()
        out = self._push("dkv", src, ("dkv", n),
                         lambda: [copy_desc(d * n * kw, me * n * kw, n, kw, kw, kw, d) for d in range(W)])
        return out[: W * n * kw].view(W, n, kw).float().sum(0)


# ---------------------------------------------------------------------- block attention
def _blocks(me: int, world: int):
    """For each local query half: the (rank, half, causal) K|V blocks it attends, diagonal first."""
    out = []
    for a in (0, 1):
        qa = chunk_id(me, a, world)
        row = [(me, a, True)]
        for s in range(world):
            for h in (0, 1):
                if chunk_id(s, h, world) < qa:
                    row.append((s, h, False))
        out.append(row)
    return out


def _pair(q_rows: torch.Tensor, kv_rows: torch.Tensor) -> torch.Tensor:
    return torch.cat([q_rows, kv_rows], dim=1)


def attn_fwd(cp: ContextParallel, qkv: torch.Tensor, cu_half: torch.Tensor, Hq: int, Hkv: int, D: int):
    """qkv [2 n, (Hq + 2 Hkv) D] of the local tokens (half-major) -> (o [2 n, Hq D], lse fp32 [Hq, 2 n]) of
    causal attention over whole sequences."""
    n, qs = qkv.shape[0] // 2, Hq * D
    kv_all = cp.gather_kv(qkv, qs)
    o_out = torch.empty(2 * n, qs, dtype=qkv.dtype, device=qkv.device)
    lse_out = torch.empty(Hq, 2 * n, dtype=torch.float32, device=qkv.device)
    for a, row in enumerate(_blocks(cp.rank, cp.world)):
        q = qkv[a * n:(a + 1) * n, :qs]
        acc = lse = None
        for s, h, causal in row:
            o_b, lse_b = AT.attn_fwd(_pair(q, kv_all[s, h * n:(h + 1) * n]), cu_half, Hq, Hkv, D, causal=causal, need_lse=True)
            if acc is None:
                acc, lse = o_b.float().view(n, Hq, D), lse_b
                continue
            new = torch.logaddexp(lse, lse_b)
            acc = acc * torch.exp(lse - new).t().unsqueeze(-1) + o_b.float().view(n, Hq, D) * torch.exp(lse_b - new).t().unsqueeze(-1)
            lse = new
        o_out[a * n:(a + 1) * n] = acc.reshape(n, qs).to(qkv.dtype)
        lse_out[:, a * n:(a + 1) * n] = lse
    return o_out, lse_out


def attn_bwd(cp: ContextParallel, do: torch.Tensor, qkv: torch.Tensor, o: torch.Tensor, lse: torch.Tensor,
             cu_half: torch.Tensor, Hq: int, Hkv: int, D: int) -> torch.Tensor:
    """Gradient of ``attn_fwd`` in the layout of ``qkv``. Every block runs the ordinary backward against
    the merged output and log-sum-exp (which makes its partial gradients exact), query gradients add up
    locally, K|V gradients go back to the rank that owns the rows."""
    n, qs = qkv.shape[0] // 2, Hq * D
    kv_all = cp.gather_kv(qkv, qs)
    dq = torch.zeros(2 * n, qs, dtype=torch.float32, device=qkv.device)
    dkv_all = torch.zeros(cp.world, 2 * n, cp.kv_width, dtype=torch.float32, device=qkv.device)
    for a, row in enumerate(_blocks(cp.rank, cp.world)):
        sl = slice(a * n, (a + 1) * n)
        q, do_a, o_a, lse_a = qkv[sl, :qs], do[sl].contiguous(), o[sl].contiguous(), lse[:, sl].contiguous()
        for s, h, causal in row:
            d_b = AT.attn_bwd(do_a, _pair(q, kv_all[s, h * n:(h + 1) * n]), o_a, lse_a, cu_half, Hq, Hkv, D, causal=causal)
            dq[sl] += d_b[:, :qs]
            dkv_all[s, h * n:(h + 1) * n] += d_b[:, qs:]
    dkv = cp.return_dkv(dkv_all)
    return torch.cat([dq, dkv], dim=1).to(qkv.dtype)
