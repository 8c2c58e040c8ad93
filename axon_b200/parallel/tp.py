"""Tensor parallelism with sequence-parallel activations: the two collectives that bracket every
sharded linear layer, fused with the GEMM through NVLink peer memory.

    all-gather -> GEMM     column-parallel layers (QKV, gate/up): the [T/W, K] activation shards stay
                           where they are; each rank's GEMM streams the A tiles of the other ranks with
                           TMA directly out of their memory (``axb_gemm_allgather_a``). No gathered
                           copy, no separate collective.
    GEMM -> reduce-scatter row-parallel layers (attention output, down projection) and the dgrad of
                           column-parallel layers: the GEMM epilogue stores every finished tile into the
                           staging slot of the rank that owns those rows (``axb_gemm_scatter``), a device
                           barrier follows, and a fixed-order sum over the W slots produces the local
                           [T/W, N] rows (``axb_rs_reduce``) — deterministic, bf16 on the wire like the
                           NCCL reduce-scatter it replaces.

(reference: Megatron-Core tensor/sequence parallel linears used through
axon/trainer/megatron_trainer.py:164-173 and axon/utils/megatron/tensor_parallel.py:52-94.)
CPU tensors and single-rank groups fall back to ``torch.distributed`` collectives + plain GEMMs.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _common as C
from ..ops import gemm as G
from .symm import PeerBarrier, SymmetricBuffer


class TPContext:
    """Per-process state of one tensor-parallel group: symmetric workspaces and the device barrier."""

    def __init__(self, group=None, device=None, max_rows_per_rank: int = 0, max_width: int = 0, fused: bool | None = None):
        self.group = group
        live = dist.is_initialized() and group is not None
        self.world = dist.get_world_size(group) if live else 1
        self.rank = dist.get_rank(group) if live else 0
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        if fused is None:
            fused = self.world > 1 and self.device.type == "cuda" and dist.get_backend(group) == "nccl"
        self.fused = bool(fused)
        self.rows, self.width = max_rows_per_rank, max_width
        self._ag = self._st = None
        self._side = None
        self.fused_max_cols = 512      # wider outputs take the chunked path of ``allgather_gemm``
        self._ag_turn = self._rs_turn = 0      # one counter per buffer kind, so that consecutive calls of a kind alternate
        self._aligned = False
        if self.fused:
            assert max_rows_per_rank % 128 == 0 and max_rows_per_rank > 0 and max_width > 0
            # Two sets per kind, used in turn: a rank that runs ahead into the next all-gather -> GEMM writes the
            # OTHER activation buffer while a slower peer may still read the previous one; the device barrier of
            # the call after that orders the reuse. Likewise for the reduce-scatter staging slots.
            self._ag = [SymmetricBuffer(max_rows_per_rank * max_width, torch.bfloat16, group, self.device) for _ in range(2)]
            self._st = [SymmetricBuffer(self.world * max_rows_per_rank * max_width, torch.bfloat16, group, self.device)
                        for _ in range(2)]
            self.barrier = PeerBarrier(group, self.device)
            self._sync = torch.zeros(1, device=self.device)

    # ------------------------------------------------------------------ plain collectives (fallback, backward gathers)
    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x
        out = torch.empty(self.world * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
        if dist.get_backend(self.group) == "gloo":
            parts = [torch.empty_like(x) for _ in range(self.world)]
            dist.all_gather(parts, x.contiguous(), group=self.group)
            return torch.cat(parts, 0)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def reduce_scatter_rows(self, x: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x
        n = x.shape[0] // self.world
        if dist.get_backend(self.group) == "gloo":
            y = x.float().contiguous()
            dist.all_reduce(y, group=self.group)
            return y[self.rank * n:(self.rank + 1) * n].to(x.dtype)
        out = torch.empty(n, *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group)
        return out

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t

    # ------------------------------------------------------------------ fused paths
    def begin_pass(self) -> None:
        """Call at the start of a forward or backward pass (every rank of the group does, in the same order). The
        first fused collective after it lines the ranks' streams up with one stream-ordered NCCL all-reduce of one
        element: the device barriers wait a bounded ~2 s, and ranks can enter a pass seconds apart (uneven data
        loading, a checkpoint write). Inside a pass every layer's barriers keep the ranks within microseconds of
        each other, so the later collectives of the pass skip the all-reduce (one NCCL launch per pass instead of
        one per collective)."""
        self._aligned = False

    def _align_streams(self, force: bool = False) -> None:
        if self._aligned and not force:
            return
        dist.all_reduce(self._sync, group=self.group)
        self._aligned = True

    def allgather_gemm(self, x_local: torch.Tensor, w: torch.Tensor, w_is_kn: bool = False, out_dtype=None) -> torch.Tensor:
        """x_local [T/W, K] (this rank's rows) -> concat(x)[T, K] @ (w [N, K]^T, or w [K, N] when ``w_is_kn``)."""
        out_dtype = out_dtype or x_local.dtype
        if not self.fused:
            xf = self.all_gather_rows(x_local)
            return G.gemm_nn(xf, w, out_dtype=out_dtype) if w_is_kn else G.gemm_nt(xf, w, out_dtype=out_dtype)
        rows, K = x_local.shape
        N = w.shape[1] if w_is_kn else w.shape[0]
        assert rows % 128 == 0 and rows * K <= self.rows * self.width, "activation shard exceeds the TP workspace"
        buf = self._ag[self._ag_turn & 1]
        self._ag_turn += 1
        buf.tensor[: rows * K].view(rows, K).copy_(x_local)
        self._align_streams()
        self.barrier()                                           # every rank's shard is in place
        out = torch.empty(self.world * rows, N, dtype=out_dtype, device=x_local.device)
        if N > self.fused_max_cols:
            return self._allgather_gemm_chunked(buf, x_local, w, w_is_kn, out)
        rc = C.lib().axb_gemm_allgather_a(buf.ptr_array(), self.world, self.rank, C.ptr(w), C.ptr(out), rows, N, K,
                                          ctypes.c_longlong(K), ctypes.c_longlong(w.stride(0)), ctypes.c_longlong(N),
                                          int(w_is_kn), int(out_dtype == torch.float32), C.ptr(C.status(self.device)), C.stream())
        C.launched(rc, "gemm_allgather_a")
        return out

    def _allgather_gemm_chunked(self, buf, x_local, w, w_is_kn, out):
        """The same product, one source rank at a time: the next rank's rows are copied into local memory on a side
        stream (each remote byte crosses NVLink once) while the tensor cores work on the rows already here. The
        single-kernel form fetches a remote activation tile once per 256-column tile of the output, which is
        link-bound for wide layers: measured on 2 GPUs, 8192 x 3072 x 4096: 0.78 ms against 0.18 ms for the bare GEMM."""
        rows, K = x_local.shape
        W, me = self.world, self.rank
        main = torch.cuda.current_stream()
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        stage = torch.empty(W - 1, rows, K, dtype=x_local.dtype, device=x_local.device)
        self._side.wait_stream(main)                     # the barrier above is done, the staging memory is ours
        events = []
        with torch.cuda.stream(self._side):
            for i in range(1, W):
                src = buf.peer_tensor((me + i) % W, rows * K)
                stage[i - 1].view(-1).copy_(src, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self._side)
                events.append(ev)
        mm = G.gemm_nn if w_is_kn else G.gemm_nt
        mm(x_local, w, out=out[me * rows:(me + 1) * rows])
        for i in range(1, W):
            r = (me + i) % W
            main.wait_event(events[i - 1])
            mm(stage[i - 1], w, out=out[r * rows:(r + 1) * rows])
        return out

    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, w_is_kn: bool = False, residual: torch.Tensor | None = None):
        """x [T, K_local] @ op(w) summed over the group, rows scattered: returns this rank's [T/W, N] (+ residual)."""
        if not self.fused:
            y = G.gemm_nn(x, w) if w_is_kn else G.gemm_nt(x, w)
            out = self.reduce_scatter_rows(y)
            return out if residual is None else (out.float() + residual.float()).to(out.dtype)
        T, K = x.shape
        N = w.shape[1] if w_is_kn else w.shape[0]
        rows = T // self.world
        assert T % self.world == 0 and rows * N <= self.rows * self.width and N % 8 == 0
        st = self._st[self._rs_turn & 1]
        self._rs_turn += 1
        rc = C.lib().axb_gemm_scatter(C.ptr(x), C.ptr(w), st.ptr_array(), self.world, self.rank, T, N, K,
                                      ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(w.stride(0)), ctypes.c_longlong(N),
                                      int(w_is_kn), C.ptr(C.status(self.device)), C.stream())
        C.launched(rc, "gemm_scatter")
        self._align_streams()
        self.barrier()                                           # all partial tiles have landed in every owner
        out = torch.empty(rows, N, dtype=x.dtype, device=x.device)
        rc = C.lib().axb_rs_reduce(C.ptr(st.tensor), C.ptr(residual), C.ptr(out), self.world, ctypes.c_longlong(rows), N,
                                   ctypes.c_longlong(N), ctypes.c_longlong(N), C.stream())
        C.launched(rc, "rs_reduce")
        return out
