"""Expert parallelism: tokens travel to the rank that owns their expert, and back, through NVLink
peer memory written and read directly by the dispatch / combine kernels (``csrc/moe.cu``, second
half). The expert computation on the owner is the grouped tcgen05 GEMM pair of the single-GPU path.

Replaces the reference's token dispatchers (NCCL ``all_to_all_single`` or DeepEP under Megatron-Core's
MoE layer: axon/config/sampler/sampler.yaml all2all_backend, megatron's moe_token_dispatcher_type): no all-to-all collective, no
permute / unpermute staging copies, the layout is derived from one W x E count matrix that every rank
reads in place. Three device barriers per layer and direction order the phases.

CPU / gloo groups use the same layout mathematics with all-gathers of the payloads (a test oracle and
a functional fallback, not a fast path).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops import _common as C
from ..ops import moe as M
from .symm import PeerBarrier, SymmetricBuffer

PAD = 128


@dataclass
class EPLayout:
    num_tokens: int
    top_k: int
    ids: torch.Tensor            # int32 [T, k] global expert ids of the local tokens
    row_of: torch.Tensor         # int32 [T*k] destination row on the owner
    owner: M.MoELayout           # layout of the rows this rank RECEIVES (its local experts)
    counts_all: torch.Tensor | None = None    # [W, E] (CPU path)


class EPContext:
    def __init__(self, group, device, num_experts: int, hidden: int, ffn: int, max_tokens: int, top_k: int, fused: bool | None = None):
        live = dist.is_initialized() and group is not None
        self.group = group
        self.world = dist.get_world_size(group) if live else 1
        self.rank = dist.get_rank(group) if live else 0
        self.device = torch.device(device)
        self.E, self.H, self.F, self.k = num_experts, hidden, ffn, top_k
        assert num_experts % self.world == 0, "experts must split evenly over the expert-parallel group"
        self.epr = num_experts // self.world
        if fused is None:
            fused = self.world > 1 and self.device.type == "cuda" and dist.get_backend(group) == "nccl"
        self.fused = bool(fused)
        # worst case: every rank sends all its assignments to this rank
        self.max_rows = (self.world * max_tokens * top_k + self.epr * (PAD - 1) + PAD - 1) // PAD * PAD
        if self.fused:
            sb = lambda n, dt: SymmetricBuffer(n, dt, group, self.device)      # noqa: E731
            self.counts = sb(num_experts, torch.int32)
            self.xs = sb(self.max_rows * hidden, torch.bfloat16)       # received tokens / their input gradients
            self.ys = sb(self.max_rows * hidden, torch.bfloat16)       # expert outputs; in backward: input gradients on their way home
            self.gs = sb(self.max_rows * hidden, torch.bfloat16)       # gradients of the expert outputs arriving from the token owners
            self.barrier = PeerBarrier(group, self.device)
            self._sync = torch.zeros(1, device=self.device)

    def sync(self) -> None:
        if self.fused:
            dist.all_reduce(self._sync, group=self.group)     # line the streams up (bounded device wait follows)
            self.barrier()

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t

    def local_experts(self) -> slice:
        return slice(self.rank * self.epr, (self.rank + 1) * self.epr)

    # ------------------------------------------------------------------ layout
    def align(self, ids: torch.Tensor) -> EPLayout:
        T, k = ids.shape
        ids = ids.to(torch.int32).contiguous()
        if self.fused:
            lib = C.lib()
            rc = lib.axb_moe_ep_count(C.ptr(ids), ctypes.c_longlong(T), k, self.E, C.ptr(self.counts.tensor), C.stream())
            C.launched(rc, "moe_ep_count")
            self.sync()
            dev = self.device
            tiles = self.max_rows // PAD
            my_base = torch.empty(self.E, dtype=torch.int32, device=dev)
            offsets = torch.empty(self.epr + 1, dtype=torch.int32, device=dev)
            tile_expert = torch.empty(tiles, dtype=torch.int32, device=dev)
            row_of = torch.empty(T * k, dtype=torch.int32, device=dev)
            scratch = C.workspace(dev, self.max_rows * 4, "moe_ep_token_of").view(torch.int32)
            rc = lib.axb_moe_ep_layout(self.counts.ptr_array(), self.world, self.rank, C.ptr(ids), ctypes.c_longlong(T), k, self.E,
                                       C.ptr(my_base), C.ptr(offsets), C.ptr(tile_expert), tiles, C.ptr(row_of), C.ptr(scratch), C.stream())
            C.launched(rc, "moe_ep_layout", 2)
            owner = M.MoELayout(0, k, self.epr, self.max_rows, None, offsets, tile_expert, None, None)
            return EPLayout(T, k, ids, row_of, owner)
        # ---- reference path: same layout from gathered counts
        flat = ids.reshape(-1).to(torch.long)
        mine = torch.bincount(flat, minlength=self.E).to(torch.int64)
        allc = [torch.zeros_like(mine) for _ in range(self.world)]
        if self.world > 1:
            dist.all_gather(allc, mine, group=self.group)
        else:
            allc = [mine]
        counts = torch.stack(allc)                                        # [W, E]
        tot = counts.sum(0)
        padded = (tot + PAD - 1) // PAD * PAD
        base = torch.zeros(self.E, dtype=torch.int64)
        for o in range(self.world):
            sl = slice(o * self.epr, (o + 1) * self.epr)
            base[sl] = torch.cumsum(padded[sl], 0) - padded[sl]
        my_base = base + counts[: self.rank].sum(0)
        order = torch.argsort(flat, stable=True)
        starts = torch.cumsum(mine, 0) - mine
        rank_in = torch.empty_like(flat)
        rank_in[order] = torch.arange(flat.numel()) - starts[flat[order]]
        row_of = (my_base[flat] + rank_in).to(torch.int32)
        sl = self.local_experts()
        offsets = torch.zeros(self.epr + 1, dtype=torch.int32)
        offsets[1:] = torch.cumsum(padded[sl], 0)
        tile_expert = torch.full((self.max_rows // PAD,), -1, dtype=torch.int32)
        for le in range(self.epr):
            tile_expert[int(offsets[le]) // PAD:int(offsets[le + 1]) // PAD] = le
        owner = M.MoELayout(0, k, self.epr, self.max_rows, None, offsets, tile_expert, None, None)
        return EPLayout(T, k, ids, row_of, owner, counts)

    # ------------------------------------------------------------------ CPU helpers: move rows between ranks
    def _exchange_rows(self, payload: torch.Tensor, lay: EPLayout, width: int) -> torch.Tensor:
        """Every rank's (owner, row, vector) triples -> the rows addressed to this rank (zeros elsewhere)."""
        owners = (lay.ids.reshape(-1).to(torch.long) // self.epr)
        pack = torch.cat([owners[:, None].float(), lay.row_of[:, None].float(), payload.float()], 1)
        n = torch.tensor([pack.shape[0]])
        ns = [torch.zeros_like(n) for _ in range(self.world)]
        dist.all_gather(ns, n, group=self.group) if self.world > 1 else ns.__setitem__(0, n)
        cap = int(max(x.item() for x in ns))
        buf = torch.zeros(cap, pack.shape[1])
        buf[: pack.shape[0]] = pack
        bufs = [torch.zeros_like(buf) for _ in range(self.world)]
        dist.all_gather(bufs, buf, group=self.group) if self.world > 1 else bufs.__setitem__(0, buf)
        out = torch.zeros(self.max_rows, width)
        for s in range(self.world):                              # source-rank order: deterministic
            b = bufs[s][: int(ns[s].item())]
            sel = b[:, 0].long() == self.rank
            out[b[sel, 1].long()] = b[sel, 2:]
        return out

    def _fetch_rows(self, table: torch.Tensor, lay: EPLayout) -> torch.Tensor:
        """rows[i] = table_of_owner(i)[row_of[i]] for this rank's assignments (gathers every owner's table)."""
        tabs = [torch.zeros_like(table) for _ in range(self.world)]
        dist.all_gather(tabs, table.contiguous(), group=self.group) if self.world > 1 else tabs.__setitem__(0, table)
        owners = (lay.ids.reshape(-1).to(torch.long) // self.epr)
        allt = torch.stack(tabs)
        return allt[owners, lay.row_of.to(torch.long)]

    # ------------------------------------------------------------------ data movement
    def dispatch(self, x: torch.Tensor, lay: EPLayout) -> torch.Tensor:
        """x [T, H] local tokens -> rows this rank received, [max_rows, H] (padding rows zero)."""
        T, k = lay.num_tokens, lay.top_k
        if not self.fused:
            return self._exchange_rows(x.repeat_interleave(k, 0), lay, x.shape[1]).to(x.dtype)
        xs = self.xs.tensor[: self.max_rows * self.H].view(self.max_rows, self.H)
        xs.zero_()                                                   # padding rows feed the weight gradients
        self.sync()                                                  # every owner's buffer is cleared and free
        rc = C.lib().axb_moe_ep_dispatch(C.ptr(x), C.ptr(lay.ids), C.ptr(lay.row_of), self.xs.ptr_array(), self.world,
                                         ctypes.c_longlong(T), k, self.H, self.E, C.stream())
        C.launched(rc, "moe_ep_dispatch")
        self.sync()                                                  # all tokens have arrived
        return xs

    def publish(self, ys: torch.Tensor) -> None:
        """Make this owner's expert outputs (or gradients) readable by the peers."""
        if self.fused:
            buf = self.ys.tensor[: ys.numel()].view_as(ys)
            if buf.data_ptr() != ys.data_ptr():
                buf.copy_(ys)
            self.sync()

    def ys_buffer(self) -> torch.Tensor:
        """Where the owner's second grouped GEMM should write so that no publish copy is needed."""
        return self.ys.tensor[: self.max_rows * self.H].view(self.max_rows, self.H) if self.fused else None

    def combine(self, ys: torch.Tensor, w: torch.Tensor, lay: EPLayout) -> torch.Tensor:
        T, k = lay.num_tokens, lay.top_k
        if not self.fused:
            rows = self._fetch_rows(ys.float(), lay).view(T, k, -1)
            return (rows * w.view(T, k, 1).float()).sum(1).to(ys.dtype)
        self.publish(ys)
        out = torch.empty(T, self.H, dtype=torch.bfloat16, device=self.device)
        rc = C.lib().axb_moe_ep_combine(self.ys.ptr_array(), self.world, C.ptr(lay.ids), C.ptr(lay.row_of), C.ptr(w.contiguous()),
                                        C.ptr(out), ctypes.c_longlong(T), k, self.H, self.E, C.stream())
        C.launched(rc, "moe_ep_combine")
        return out

    def combine_bwd(self, dout: torch.Tensor, ys: torch.Tensor, w: torch.Tensor, lay: EPLayout):
        """-> (dys rows this rank received [max_rows, H], dw [T, k]). ``ys`` must be the published outputs."""
        T, k = lay.num_tokens, lay.top_k
        if not self.fused:
            yrows = self._fetch_rows(ys.float(), lay)
            dw = (dout.float().repeat_interleave(k, 0) * yrows).sum(-1).view(T, k)
            dys = self._exchange_rows(dout.float().repeat_interleave(k, 0) * w.reshape(-1, 1).float(), lay, dout.shape[1])
            return dys.to(ys.dtype), dw
        self.publish(ys)
        dys = self.gs.tensor[: self.max_rows * self.H].view(self.max_rows, self.H)
        dys.zero_()                                                  # padding rows feed the weight gradients
        self.sync()
        dw = torch.empty(T, k, dtype=torch.float32, device=self.device)
        rc = C.lib().axb_moe_ep_combine_bwd(C.ptr(dout), self.ys.ptr_array(), self.gs.ptr_array(), self.world, C.ptr(lay.ids),
                                            C.ptr(lay.row_of), C.ptr(w.contiguous()), C.ptr(dw), ctypes.c_longlong(T), k, self.H,
                                            self.E, C.stream())
        C.launched(rc, "moe_ep_combine_bwd")
        self.sync()
        return dys, dw

    def collect(self, dxs: torch.Tensor, lay: EPLayout) -> torch.Tensor:
        """Backward of dispatch: dx[t] = sum_j dxs_owner[row]."""
        T, k = lay.num_tokens, lay.top_k
        if not self.fused:
            return self._fetch_rows(dxs.float(), lay).view(T, k, -1).sum(1).to(dxs.dtype)
        self.publish(dxs)
        dx = torch.empty(T, self.H, dtype=torch.bfloat16, device=self.device)
        rc = C.lib().axb_moe_ep_collect(self.ys.ptr_array(), self.world, C.ptr(lay.ids), C.ptr(lay.row_of), C.ptr(dx),
                                        ctypes.c_longlong(T), k, self.H, self.E, C.stream())
        C.launched(rc, "moe_ep_collect")
        self.sync()                                                  # peers are done reading before buffers are reused
        return dx
