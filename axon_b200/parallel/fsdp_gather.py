"""Parameter all-gather fused into the consuming GEMM (ZeRO-3 / FSDP-style sharded weights).

The reference's FSDP trainer all-gathers a layer's parameters before its forward / backward and re-shards
afterwards (``FSDP(...)`` / ``apply_fsdp2``, axon/trainer/fsdp_trainer.py:362-422). The trainer here keeps bf16
parameters whole (ZeRO-1) because 180 GB per GPU holds them; for models where that no longer fits,
``ShardedLinear`` keeps only a row shard ``[F / W, K]`` of a weight per rank in symmetric memory and computes

    y[T, F] = x[T, K] @ concat_r(W_r)^T

with one kernel whose weight tiles are fetched by TMA from the rank that owns them (own shard first, every
rank starting on a different peer) - the gathered weight never exists in memory and the transfer overlaps the
tensor-core work tile by tile (``axb_gemm_gather_weights``, ``csrc/gemm.cu``; tile map ``PeerGatherTiles``).
``dgrad`` is the same gather on the K side and ``wgrad`` produces full-size gradients that the ZeRO reduce
shards again; both still use the plain kernels on an all-gathered copy here (the forward path is the fused
one). On CPU / gloo the op all-gathers and multiplies (host-side logic and tests).

Cost across NVLink: the kernel fetches a remote weight tile once per 256-token tile of ``x`` (peer memory is not
cached on the reading side), so its link traffic is (remote share of the weight) x (token tiles). It pays for
one to four token tiles (small batches, where a separate gather is pure latency); for long micro-batches the
training model (``models/zero3_dense.py``) gathers the shard once instead.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _common as C
from .symm import PeerBarrier, SymmetricBuffer


class ShardedLinear:
    def __init__(self, full_weight: torch.Tensor | None, out_features: int, in_features: int, group, device, dtype=torch.bfloat16,
                 fused: bool | None = None):
        """``full_weight`` ([F, K], same on every rank) is cut to this rank's rows; pass None and fill ``shard`` later."""
        live = dist.is_initialized() and group is not None
        self.group = group
        self.world = dist.get_world_size(group) if live else 1
        self.rank = dist.get_rank(group) if live else 0
        self.device = torch.device(device)
        self.F, self.K = out_features, in_features
        assert out_features % (128 * self.world) == 0, "rows per rank must be a multiple of 128"
        self.per = out_features // self.world
        if fused is None:
            fused = self.world > 1 and self.device.type == "cuda" and dist.get_backend(group) == "nccl"
        self.fused = bool(fused)
        if self.fused:
            self.buf = SymmetricBuffer(self.per * in_features, dtype, group, self.device)
            self.shard = self.buf.tensor.view(self.per, in_features)
            self.barrier = PeerBarrier(group, self.device)
            self._sync = torch.zeros(1, device=self.device)
        else:
            self.shard = torch.empty(self.per, in_features, dtype=dtype, device=self.device)
        if full_weight is not None:
            self.shard.copy_(full_weight[self.rank * self.per:(self.rank + 1) * self.per].to(self.device).to(dtype))
        self.publish()

    def publish(self) -> None:
        """After the local shard changed (optimizer step): make it visible to the peers' next gather."""
        if self.fused:
            dist.all_reduce(self._sync, group=self.group)       # line the streams up before the bounded device barrier
            self.barrier()

    def gather(self) -> torch.Tensor:
        if self.world == 1:
            return self.shard
        parts = [torch.empty_like(self.shard) for _ in range(self.world)]
        dist.all_gather(parts, self.shard.contiguous(), group=self.group)
        return torch.cat(parts)

    def forward(self, x: torch.Tensor, out_dtype=None) -> torch.Tensor:
        T = x.shape[0]
        if not self.fused:
            w = self.gather()
            return (x.float() @ w.float().t()).to(out_dtype or x.dtype)
        assert x.dtype == torch.bfloat16 and x.stride(-1) == 1
        out = torch.empty(T, self.F, dtype=out_dtype or torch.bfloat16, device=x.device)
        rc = C.lib().axb_gemm_gather_weights(self.buf.ptr_array(), self.world, self.rank, C.ptr(x), C.ptr(out), self.per, T, self.K,
                                             ctypes.c_longlong(self.K), ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(out.stride(0)),
                                             int(out.dtype == torch.float32), C.ptr(C.status(x.device)), C.stream())
        C.launched(rc, "gemm_gather_weights")
        return out
