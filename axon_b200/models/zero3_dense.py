"""Dense decoder with parameter shards (ZeRO-3 / FSDP style; reference: the FSDP wrapping of
axon/trainer/fsdp_trainer.py:362-422). See ``parallel/zero3.py`` for the scheme. The four matrices of every
layer are row shards in a symmetric-memory parameter buffer; everything token-wise is the dense model's code,
only the linear layers' forward / backward go through the hooks below.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import _common as C
from ..ops import gemm as G
from ..parallel.symm import SymmetricBuffer
from ..parallel.zero3 import ShardContext, is_sharded, zero3_layout
from .config import ModelConfig
from .dense import DenseModel
from .params import FlatParams, param_layout


class Zero3DenseModel(DenseModel):
    def __init__(self, cfg: ModelConfig, shard: ShardContext, device="cuda", dtype=torch.bfloat16):
        assert cfg.num_experts == 0, "parameter shards are built for dense models"
        layout = zero3_layout(cfg, shard.world, 128 if shard.fused else 1)
        self._sym = None
        flat = None
        if shard.fused:
            numel = FlatParams(cfg, "meta", dtype, layout=layout).numel
            self._sym = SymmetricBuffer(numel, dtype, shard.group, torch.device(device))
            flat = self._sym.tensor
            flat.zero_()
        super().__init__(cfg, device, dtype, params=FlatParams(cfg, torch.device(device), dtype, flat=flat, layout=layout))
        self.shard = shard
        self.full_layout = param_layout(cfg)
        self._pending: list = []
        # The fused kernel reads a remote weight tile once per 256-token tile of the activations (peer memory is
        # not cached on this side of the link), so its NVLink traffic grows with the token count: measured on 2
        # GPUs at 8192 tokens it is link-bound (135 ms against 84 ms for whole parameters, 4 Qwen3-8B layers).
        # Above this many tokens the shard is gathered once and a plain GEMM follows.
        self.fused_max_tokens = 1024

    # ------------------------------------------------------------------ parameters
    def load_full_state(self, full_views: dict) -> None:
        W, r = self.shard.world, self.shard.rank
        for name, dst in self.params.views.items():
            src = full_views[name]
            if is_sharded(name):
                per = src.shape[0] // W
                src = src[r * per:(r + 1) * per]
            dst.copy_(src.to(dst.device).to(dst.dtype))
        self.shard.publish()

    def init_random(self, std: float = 0.02, seed: int = 0) -> None:
        """Same values as ``FlatParams.init_random`` of the unsharded model with this seed."""
        ref = FlatParams(self.cfg, self.device, self.dtype)
        ref.init_random(std=std, seed=seed)
        self.load_full_state(ref.views)

    def gather_full(self) -> dict:
        """Full tensors of every parameter (CPU), the same on every rank."""
        out = {}
        for name, v in self.params.views.items():
            out[name] = (self.shard.all_gather_rows(v.detach()) if is_sharded(name) else v.detach()).cpu().clone()
        return out

    serves_sampler = False       # a colocated sampler keeps a replica with whole parameters

    def full_named_tensors(self):
        """(name, whole tensor) of every parameter, gathered one at a time; a collective every rank iterates to the end."""
        for name, v in self.params.views.items():
            yield name, (self.shard.all_gather_rows(v.detach()) if is_sharded(name) else v.detach())

    def sum_over_row_peers(self, t: torch.Tensor) -> torch.Tensor:
        """The ranks of the shard group are data-parallel peers outside the optimizer's (single-rank) group: a count over the
        rows of a mini-batch is completed here."""
        return self.shard.all_reduce_(t)

    def replicated_names(self) -> list[str]:
        return [n for n in self.params.layout if not is_sharded(n)]

    def replicated_ranges(self) -> list[tuple[int, int]]:
        keep = set(self.replicated_names())
        spans = sorted((o, o + n) for name, (o, n) in self.params.offsets.items() if name in keep)
        out: list[list[int]] = []
        for a, b in spans:
            if out and out[-1][1] == a:
                out[-1][1] = b
            else:
                out.append([a, b])
        return [(a, b) for a, b in out]

    def sync_replicated_grads(self) -> None:
        """Sum the gradients of the replicated parameters over the ranks (the shards' gradients were
        reduce-scattered micro-batch by micro-batch)."""
        self.finish_grads()
        if self.shard.world == 1 or self.params.grad_flat is None:
            return
        for a, b in self.replicated_ranges():
            self.shard.all_reduce_(self.params.grad_flat[a:b])

    def after_optim_step(self) -> None:
        self.shard.publish()

    # ------------------------------------------------------------------ the linear layers
    def _gathered(self, l: int, name: str) -> torch.Tensor:
        return self.shard.all_gather_rows(self._p(l, name))

    def _lin(self, l: int, name: str, x: torch.Tensor) -> torch.Tensor:
        sh = self.shard
        w = self._p(l, name)
        if not is_sharded(f"model.layers.{l}.{name}") or sh.world == 1:
            return super()._lin(l, name, x)
        T = x.shape[0]
        if not sh.fused or T > self.fused_max_tokens:
            return self._bias_fwd(l, name, G.gemm_nt(x, self._gathered(l, name)))
        per, K = w.shape
        assert x.dtype == torch.bfloat16 and x.stride(-1) == 1
        off = self.params.offsets[f"model.layers.{l}.{name}"][0] * w.element_size()
        ptrs = (ctypes.c_ulonglong * sh.world)(*[p + off for p in self._sym.ptrs])
        out = torch.empty(T, per * sh.world, dtype=torch.bfloat16, device=x.device)
        rc = C.lib().axb_gemm_gather_weights(ptrs, sh.world, sh.rank, C.ptr(x), C.ptr(out), per, T, K, ctypes.c_longlong(K),
                                             ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(out.stride(0)), 0,
                                             C.ptr(C.status(x.device)), C.stream())
        C.launched(rc, "gemm_gather_weights")
        return self._bias_fwd(l, name, out)

    def _lin_bwd(self, l: int, name: str, dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        sh = self.shard
        if not is_sharded(f"model.layers.{l}.{name}") or sh.world == 1:
            return super()._lin_bwd(l, name, dy, x)
        w_full = self._gathered(l, name)
        dx = G.gemm_nn(dy, w_full)
        del w_full
        dw_full = G.gemm_tn(dy, x, out_dtype=torch.float32)
        # the reduce-scatter runs on the communication stream while backward goes on; at most two are pending
        self._pending.append((*sh.reduce_scatter_rows_async(dw_full), self._g(l, name), dw_full))
        while len(self._pending) > 2:
            self._finish_one()
        self._bias_bwd(l, name, dy)
        return dx

    def _finish_one(self) -> None:
        work, part, grad, _keep = self._pending.pop(0)
        if work is not None:
            work.wait()
        grad.add_(part)

    def finish_grads(self) -> None:
        """Fold every pending gradient shard in (before anything reads the gradient buffer)."""
        while self._pending:
            self._finish_one()

    def prefill(self, *a, **k):
        raise NotImplementedError("a model with parameter shards does not serve the sampler; sample from a replica with whole parameters")

    decode = prefill
