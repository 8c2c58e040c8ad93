"""Sum over a tensor-parallel group for the sampler's decode path.

A decode step under tensor parallelism sums two small activation tensors per layer over the group
([batch, hidden] bf16: 1 MB at batch 256, hidden 2048). At that size a collective is pure launch and
synchronisation latency, so on CUDA the sum is ONE kernel over NVLink peer memory
(``axb_peer_allreduce``): every block pushes its slice into a staging slot on every rank, raises a
per-block flag, waits (bounded) for the other ranks' flags of the same slice and adds the slots in rank
order, so every rank ends up with the same bits - which lockstep sampling across the group relies on.
The call's epoch is kept in device memory, so a captured CUDA graph can replay the launch. Tensors
larger than the staging slot (prefill activations), other dtypes and CPU tensors use the process
group's all-reduce.

The flag waits are bounded (about two seconds) and report through the device status word instead of
hanging, so the ranks' streams must not drift further apart than that: ``begin_step`` lines them up
with one stream-ordered NCCL all-reduce of a single element, once per engine step.

(reference: the reference's samplers get this from vLLM / SGLang tensor-parallel workers -
axon/sampler/vllm/server.py:379-625 passes ``tensor_parallel_size`` through; their custom
all-reduce plays the role of the kernel here.)
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _common as C
from .symm import SymmetricBuffer


class PeerAllReduce:
    CAP = 1 << 21            # elements per staging slot (4 MB of bf16)
    MAX_BLOCKS = 296

    def __init__(self, group=None, device=None, fused: bool | None = None):
        self.group = group
        live = dist.is_initialized() and group is not None
        self.world = dist.get_world_size(group) if live else 1
        self.rank = dist.get_rank(group) if live else 0
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        if fused is None:
            fused = self.world > 1 and self.device.type == "cuda" and dist.get_backend(group) == "nccl"
        self.fused = bool(fused)
        self.calls = {"fused": 0, "collective": 0}
        if self.fused:
            self._flag_off = 2 * self.world * self.CAP * 2                   # bytes
            flag_elems = 2 * self.world * self.MAX_BLOCKS * 2                # u32 flags counted in bf16 elements
            self._buf = SymmetricBuffer(2 * self.world * self.CAP + flag_elems, torch.bfloat16, group, self.device)
            self._buf.tensor.zero_()
            torch.cuda.current_stream().synchronize()
            self._buf.barrier()
            self._state = torch.zeros(2, dtype=torch.int32, device=self.device)
            self._sync = torch.zeros(1, device=self.device)

    def begin_step(self) -> None:
        """Every rank calls this at the start of every engine step, outside any graph capture."""
        if self.fused:
            dist.all_reduce(self._sync, group=self.group)

    def __call__(self, y: torch.Tensor) -> torch.Tensor:
        """Sum ``y`` over the group in place and return it."""
        if self.world == 1:
            return y
        n = y.numel()
        if not (self.fused and y.dtype == torch.bfloat16 and y.is_contiguous() and n % 8 == 0 and n <= self.CAP):
            self.calls["collective"] += 1
            if y.is_contiguous():
                dist.all_reduce(y, group=self.group)
                return y
            z = y.contiguous()
            dist.all_reduce(z, group=self.group)
            return y.copy_(z)
        self.calls["fused"] += 1
        rc = C.lib().axb_peer_allreduce(self._buf.ptr_array(), self.rank, self.world, C.ptr(y), C.ptr(y), ctypes.c_longlong(n),
                                        ctypes.c_longlong(self.CAP), ctypes.c_longlong(self._flag_off), self.MAX_BLOCKS,
                                        C.ptr(self._state), C.ptr(C.status(self.device)), C.stream())
        C.launched(rc, "peer_allreduce")
        return y
