"""ZeRO-1 optimizer step as fused peer-memory kernels (no NCCL in the data path).

Gradients and the bf16 parameters of every rank live in symmetric buffers. One step is

    barrier  ->  reduce      every rank sums ITS shard over all ranks' fp32 gradient buffers with
                             peer loads (the reduce-scatter) and produces sum-of-squares partials
             ->  norm        partials are published in a symmetric stats buffer; after a barrier each
                             rank reads all of them and derives the same clip coefficient / skip flag
             ->  adamw+bcast fused AdamW on the shard whose epilogue STORES the new bf16 values into
                             every rank's parameter buffer (the all-gather)
             ->  barrier

This replaces ``reduce_scatter_tensor`` + ``all_reduce`` + ``clip_grad_norm_`` + ``AdamW.step`` +
``all_gather_into_tensor`` of the reference's FSDP path (axon/trainer/fsdp_trainer.py:674-771,
axon/utils/fsdp/utils.py:434-448) with three kernels that move each byte over NVLink exactly once.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import _common as C
from ..ops import optim as OPT
from .symm import PeerBarrier, SymmetricBuffer


class FusedZero1:
    def __init__(self, numel: int, group=None, device=None):
        self.grads = SymmetricBuffer(numel, torch.float32, group, device)
        self.params = SymmetricBuffer(numel, torch.bfloat16, group, device)
        self.world, self.rank = self.grads.world, self.grads.rank
        self.device = self.grads.device
        self.barrier = PeerBarrier(group, device)
        lib = C.lib() if self.device.type == "cuda" else None
        self.n_partials = lib.axb_zero1_partials() if lib is not None else 1
        self.stats = SymmetricBuffer(16, torch.float32, group, device)       # slot r: rank r's partial sumsq
        self.partials = torch.zeros(self.n_partials, dtype=torch.float32, device=self.device)
        self.state = torch.zeros(4, dtype=torch.float32, device=self.device)
        per = numel // self.world
        assert per * self.world == numel and per % 128 == 0, "flat size must split evenly into 128-aligned shards"
        self.lo, self.n = self.rank * per, per
        self.reduced = torch.empty(per, dtype=torch.float32, device=self.device)
        self.grads.tensor.zero_()
        self._sync_token = torch.zeros(1, dtype=torch.float32, device=self.device)

    def step(self, master, exp_avg, exp_avg_sq, lr, beta1, beta2, eps, wd, step, max_norm, skip_threshold=0.0):
        """Consumes ``grads.tensor`` (this rank's full local gradient), updates this rank's shard of the
        optimizer state and every rank's ``params.tensor``. Returns the device state [sumsq, norm, coef, skip]."""
        lib = C.lib()
        if self.world > 1:
            # Ranks can reach the optimizer step seconds apart (uneven micro-batches); the device
            # barrier's wait is bounded to about two seconds by design, so first line the streams up
            # with a stream-ordered NCCL all-reduce of one element (plumbing, not data).
            import torch.distributed as dist
            dist.all_reduce(self._sync_token, group=self.grads.group)
        self.barrier()                                                        # all backward passes are done
        rc = lib.axb_zero1_reduce(self.grads.ptr_array(), self.rank, self.world, ctypes.c_longlong(self.lo),
                                  ctypes.c_longlong(self.n), C.ptr(self.reduced), C.ptr(self.partials), C.stream())
        C.launched(rc, "zero1_reduce")
        # this rank's sum of squares -> its slot in everyone's view (each rank reads all slots below)
        mine = self.stats.tensor[self.rank:self.rank + 1]
        torch.sum(self.partials, dim=0, keepdim=True, out=mine)
        self.barrier()
        rc = lib.axb_zero1_total(self.stats.ptr_array(), self.world, C.ptr(self.state), C.stream())   # fixed rank order
        C.launched(rc, "zero1_total")
        OPT.clip_coef(self.state, max_norm, skip_threshold)
        bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
        rc = lib.axb_zero1_adamw_bcast(C.ptr(master), C.ptr(self.reduced), C.ptr(exp_avg), C.ptr(exp_avg_sq),
                                       self.params.ptr_array(), self.world, ctypes.c_longlong(self.lo),
                                       ctypes.c_longlong(self.n), ctypes.c_float(lr), ctypes.c_float(beta1),
                                       ctypes.c_float(beta2), ctypes.c_float(eps), ctypes.c_float(wd),
                                       ctypes.c_float(bc1), ctypes.c_float(bc2), C.ptr(self.state), C.stream())
        C.launched(rc, "zero1_adamw_bcast")
        self.barrier()                                                        # every rank's params are complete
        return self.state
