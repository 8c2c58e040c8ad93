"""Parameter shards (ZeRO-3 / FSDP style) for the family toolkit: every rank keeps 1/W of every decoder layer.

The in-house dense model shards its layer matrices by rows and multiplies straight out of the owners' memory
(``models/zero3_dense.py``). The families of ``models/families.py`` are autograd programs over a dictionary of named
tensors, so here the unit is the LAYER: all parameters of decoder layer ``l`` form one contiguous flat range (the
offsets ``FlatParams`` would give them), cut into W equal pieces. A layer's forward first all-gathers the pieces
into the full flat range and hands the family's layer function views of it; with full recomputation (the default
of the families) the range is dropped when the layer is done and gathered again when its backward runs, so at any
moment one layer exists in full. The gradient of the gathered range is reduce-scattered in fp32 straight into this
rank's piece of the fp32 gradient buffer. Embedding, head, final norm and a vision tower stay whole on every rank;
their gradients are summed over the ranks once per step. Per rank a 26 B-parameter model then holds 6.5 GB of
bf16 pieces, 13 GB of gradient and 39 GB of optimizer state instead of 52 + 104 + 39 GB.

Ranks see different data and meet in these collectives layer by layer, so they run equal numbers of micro-batches
(the policy engine reads ``model.shard`` for that). A model with parameter shards does not serve the sampler: the
colocated sampler keeps a replica with whole parameters and is refreshed from ``full_named_tensors``.

(reference: the FSDP trainer shards every family the same way - ``apply_fsdp2`` / ``FSDP(...)`` with one unit per
decoder layer, axon/trainer/fsdp_trainer.py:362-422, axon/utils/fsdp/utils.py - and hands whole tensors to
the inference engine, axon/sampler/mixins/sync_mixin.py:86-168.)
"""
from __future__ import annotations

import re
from collections import ChainMap, OrderedDict

import torch

from ..parallel.zero3 import ShardContext
from .config import ModelConfig
from .families import FamilyModel, FamilyParams
from .params import ALIGN

_LAYER = re.compile(r"(?:^|\.)layers\.(\d+)\.")


def layer_of(name: str) -> int | None:
    """Decoder layer a parameter belongs to; None for what every rank keeps whole (embedding, head, norms, vision tower)."""
    if ".visual." in name or ".vision" in name:
        return None
    m = _LAYER.search(name)
    return int(m.group(1)) if m else None


def shard_key(l: int) -> str:
    return f"layers.{l}.__shard__"


class _GatherLayer(torch.autograd.Function):
    """pieces of one layer -> its full flat range; backward: fp32 reduce-scatter into the rank's gradient piece."""

    @staticmethod
    def forward(ctx, piece: torch.Tensor, model: "ShardedFamilyModel", l: int):
        ctx.model, ctx.l = model, l
        return model.shard.all_gather_rows(piece.detach().view(1, -1)).view(-1)

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        m, sh = ctx.model, ctx.model.shard
        part = sh.reduce_scatter_rows(g.float().view(sh.world, -1)).reshape(-1)
        m.params.alloc_grads()
        m.params.grads[shard_key(ctx.l)].add_(part)
        return None, None, None


class ShardedFamilyModel(FamilyModel):
    serves_sampler = False

    def __init__(self, cfg: ModelConfig, shard: ShardContext, device="cuda", dtype=torch.bfloat16):
        self.shard = shard
        super().__init__(cfg, device=device, dtype=dtype)

    # ------------------------------------------------------------------ storage
    def _make_params(self):
        """Local storage: whole tensors for the replicated names, one piece per decoder layer."""
        W = self.shard.world
        self.full_layout = self.layout
        per_layer: dict[int, OrderedDict] = {}
        local = OrderedDict()
        for name, shape in self.full_layout.items():
            l = layer_of(name)
            if l is None:
                local[name] = shape
            else:
                per_layer.setdefault(l, OrderedDict())[name] = shape
        self.layer_layouts = per_layer
        self.layer_offsets: dict[int, dict] = {}
        self.layer_len: dict[int, int] = {}
        for l, lay in sorted(per_layer.items()):
            off, table = 0, {}
            for name, shape in lay.items():
                n = 1
                for s in shape:
                    n *= s
                table[name] = (off, n, tuple(shape))
                off += (n + ALIGN - 1) // ALIGN * ALIGN
            step = W * ALIGN
            self.layer_offsets[l], self.layer_len[l] = table, (off + step - 1) // step * step
            local[shard_key(l)] = (self.layer_len[l] // W,)
        self.layout = local
        return FamilyParams(self.cfg, self.device, self.dtype, local, self.spec)

    def _full_layer_flat(self, l: int, tensors: dict) -> torch.Tensor:
        flat = torch.zeros(self.layer_len[l], dtype=self.dtype, device=self.device)
        for name, (o, n, shape) in self.layer_offsets[l].items():
            flat[o:o + n].copy_(tensors[name].reshape(-1).to(self.device).to(self.dtype))
        return flat

    def _keep_piece(self, l: int, flat: torch.Tensor) -> None:
        n = self.layer_len[l] // self.shard.world
        self.params.views[shard_key(l)].copy_(flat[self.shard.rank * n:(self.shard.rank + 1) * n])

    def load_full_state(self, full_views: dict) -> None:
        """Copy from an unsharded model's named tensors, keeping this rank's pieces."""
        for name, dst in self.params.views.items():
            if name in self.full_layout:
                dst.copy_(full_views[name].reshape(dst.shape).to(dst.device).to(dst.dtype))
        for l in self.layer_offsets:
            self._keep_piece(l, self._full_layer_flat(l, full_views))

    def init_random(self, std: float = 0.02, seed: int = 0) -> None:
        """The family's own initialisation rules. Up to two billion parameters the values are those of the unsharded
        model with this seed (initialised on the host, then cut); larger models are initialised one layer at a time
        with a seed per layer, the same on every rank before the cut."""
        total = sum(torch.Size(s).numel() for s in self.full_layout.values())
        if total <= 2_000_000_000:
            ref = FamilyParams(self.cfg, "cpu", self.dtype, self.full_layout, self.spec)
            ref.init_random(std, seed)
            return self.load_full_state(ref.views)
        whole = OrderedDict((n, s) for n, s in self.layout.items() if n in self.full_layout)
        tmp = FamilyParams(self.cfg, self.device, self.dtype, whole, self.spec)
        tmp.init_random(std, seed)
        for n, v in tmp.views.items():
            self.params.views[n].copy_(v)
        for l, lay in self.layer_layouts.items():
            tmp = FamilyParams(self.cfg, self.device, self.dtype, lay, self.spec)
            tmp.init_random(std, seed + 7919 * (l + 1))
            self._keep_piece(l, self._full_layer_flat(l, tmp.views))

    def load_state_dict(self, sd: dict, strict: bool = True) -> None:
        """Tensors by checkpoint name (per-expert checkpoints are stacked as in the unsharded model), layer by layer."""
        whole = OrderedDict((n, s) for n, s in self.layout.items() if n in self.full_layout)
        tmp = FamilyParams(self.cfg, self.device, self.dtype, whole, self.spec)
        tmp.load_hf_state_dict(sd, strict=strict)
        for n, v in tmp.views.items():
            self.params.views[n].copy_(v)
        for l, lay in self.layer_layouts.items():
            tmp = FamilyParams(self.cfg, self.device, self.dtype, lay, self.spec)
            tmp.load_hf_state_dict(sd, strict=strict)
            self._keep_piece(l, self._full_layer_flat(l, tmp.views))
        for n in list(self.buffers):
            if n in sd:
                self.buffers[n] = sd[n].to(self.device)

    def load_hf_checkpoint(self, path: str) -> None:
        """Stream an HF directory: only one layer's tensors are in memory at a time."""
        import os

        from safetensors import safe_open

        from ..utils.hf_model import normalize_param_name
        where: dict[str, tuple[str, str]] = {}
        for fn in sorted(f for f in os.listdir(path) if f.endswith(".safetensors")):
            with safe_open(os.path.join(path, fn), framework="pt", device="cpu") as f:
                for k in f.keys():
                    where[normalize_param_name(k)] = (fn, k)

        def fetch(names):
            out, by_file = {}, {}
            for n in names:
                by_file.setdefault(where[n][0], []).append(n)
            for fn, ns in by_file.items():
                with safe_open(os.path.join(path, fn), framework="pt", device="cpu") as f:
                    for n in ns:
                        out[n] = f.get_tensor(where[n][1])
            return out
        whole = OrderedDict((n, s) for n, s in self.layout.items() if n in self.full_layout)
        tmp = FamilyParams(self.cfg, self.device, self.dtype, whole, self.spec)
        tmp.load_hf_state_dict(fetch([n for n in where if layer_of(n) is None]), strict=True)
        for n, v in tmp.views.items():
            self.params.views[n].copy_(v)
        for l, lay in self.layer_layouts.items():
            tmp = FamilyParams(self.cfg, self.device, self.dtype, lay, self.spec)
            tmp.load_hf_state_dict(fetch([n for n in where if layer_of(n) == l]), strict=True)
            self._keep_piece(l, self._full_layer_flat(l, tmp.views))

    def full_named_tensors(self):
        """(name, whole tensor) of every parameter, one layer gathered at a time. A collective: every rank iterates it to
        the end. The tensors of a layer are views of one buffer that is reused by the next layer."""
        for name, v in self.params.views.items():
            if name in self.full_layout:
                yield name, v.detach()
        for l in sorted(self.layer_offsets):
            flat = self.shard.all_gather_rows(self.params.views[shard_key(l)].detach().view(1, -1)).view(-1)
            for name, (o, n, shape) in self.layer_offsets[l].items():
                yield name, flat[o:o + n].view(shape)

    def state_dict(self):
        out = OrderedDict((n, t.clone()) for n, t in self.full_named_tensors())
        out.update(self.buffers)
        return out

    # ------------------------------------------------------------------ the policy engine's model-parallel contract
    def replicated_names(self) -> list[str]:
        return [n for n in self.layout if n in self.full_layout]

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
        """Sum the gradients of the whole-on-every-rank parameters over the ranks; the layers' pieces were
        reduce-scattered when their backward ran."""
        if self.shard.world == 1 or self.params.grad_flat is None:
            return
        for a, b in self.replicated_ranges():
            self.shard.all_reduce_(self.params.grad_flat[a:b])

    # ------------------------------------------------------------------ compute
    def _leaves(self, grad: bool) -> dict:
        if not grad:
            return dict(self.params.views)
        out = {}
        for n, v in self.params.views.items():
            whole = n in self.full_layout
            out[n] = v.detach().requires_grad_(self.spec.trainable(n) if whole else True)
        return out

    def _layer_weights(self, W: dict, l: int):
        piece = W[shard_key(l)]
        if piece.requires_grad:
            flat = _GatherLayer.apply(piece, self, l)
        else:
            flat = self.shard.all_gather_rows(piece.view(1, -1)).view(-1)
        views = {name: flat[o:o + n].view(shape) for name, (o, n, shape) in self.layer_offsets[l].items()}
        return ChainMap(views, W)

    def _layer_call(self, W, l, h, ctx):
        return self.spec.layer(self._layer_weights(W, l), l, h, ctx)

    def backward(self, g_logprob, g_entropy=None) -> None:
        assert self._saved is not None, "forward(save_for_backward=True) must come first"
        W, lp, ent = self._saved
        self._saved = None
        self.params.alloc_grads()
        outs, grads = [lp], [g_logprob.to(lp.dtype)]
        if g_entropy is not None:
            outs.append(ent)
            grads.append(g_entropy.to(ent.dtype))
        torch.autograd.backward(outs, grads)
        for n, leaf in W.items():                  # the layers' pieces were accumulated by the gather's backward
            if leaf.grad is not None and n in self.full_layout:
                self.params.grads[n].add_(leaf.grad.float())

    def prefill(self, *a, **k):
        raise NotImplementedError("a model with parameter shards does not serve the sampler; sample from a replica with whole parameters")

    decode = prefill
