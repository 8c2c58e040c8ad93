"""Sampler-side model sharded over a tensor-parallel group (inference only).

Every rank of the group sees the SAME tokens (the engines of the group run in lockstep) and holds

  * the query / key / value rows of its share of the heads and the matching columns of the attention
    output projection, hence also only its heads' pages of the KV cache (a group with more ranks than the
    model has key / value heads gives each rank ONE such head, which several ranks then hold alike),
  * dense MLP: its share of the gate / up rows and of the down-projection columns,
  * sparse MLP: ALL of the router and the whole weights of ``num_experts / world`` experts (expert
    parallelism inside the group): a rank runs the grouped GEMMs over the assignments to its own experts
    only - the layout kernels give assignments to other ranks' experts no row - and the weighted sum of
    its experts' outputs is a partial result like a row-parallel linear's,
  * embedding, norms and the vocabulary head in full.

The two partial results per layer are summed over the group by ``parallel.allreduce.PeerAllReduce``
(one NVLink peer-memory kernel per sum at decode sizes). Because that sum gives every rank the same
bits, logits and therefore sampled tokens agree across the group without exchanging them.

A sharded model is the full model's code running on a "local" configuration (fewer heads, narrower
MLP, fewer experts), so prefill, decode, paged attention and CUDA-graph capture are the single-GPU
paths. ``localize`` cuts a full tensor, named either in this framework's fused layout or as in an HF
checkpoint, down to this rank's part; the weight-sync paths and the checkpoint loader go through it.

(reference: axon/sampler/sampler.py:62-91 and axon/sampler/vllm/server.py:379-625 - the sampler
is launched with ``tensor_model_parallel_size`` / ``enable_expert_parallel`` and vLLM shards the model;
parameter re-slicing for a sharded sampler as in axon/utils/p2p/param_mapper.py:367-413.)
"""
from __future__ import annotations

import dataclasses
import re

import torch
import torch.distributed as dist

from ..ops import activation as A
from ..ops import gemm as G
from ..ops import moe as M
from ..parallel.allreduce import PeerAllReduce
from .config import ModelConfig
from .dense import DenseModel
from .moe import MoEModel
from .params import FlatParams
from .tp_dense import slice_full_param, tp_param_layout

_ROW_PARALLEL = ("self_attn.o_proj.weight", "mlp.down_proj.weight")
_EXPERT = re.compile(r"\.mlp\.experts\.(\d+)\.")


@dataclasses.dataclass
class Shard:
    """One rank's place in a tensor-parallel sampler group."""
    group: object = None
    rank: int = 0
    world: int = 1
    reduce: PeerAllReduce | None = None

    @staticmethod
    def create(group, device, reduce: bool = True) -> "Shard":
        """``reduce``: also set up the group's activation sum (a tensor-parallel group needs it, pipeline stages do not)."""
        world = dist.get_world_size(group) if group is not None else 1
        rank = dist.get_rank(group) if group is not None else 0
        return Shard(group, rank, world, PeerAllReduce(group, device) if reduce else None)


def local_config(cfg: ModelConfig, world: int) -> ModelConfig:
    """The configuration of one rank's part: heads (and the dense MLP width) divided by the group size."""
    g = cfg.num_key_value_heads
    if cfg.num_attention_heads % world or (g % world and world % g):
        raise ValueError(f"{cfg.num_attention_heads} query / {g} key-value heads do not divide over {world} ranks")
    # more ranks than key / value heads: world / g ranks hold the same head (and keep its cache pages) next to their own query heads
    kw = dict(num_attention_heads=cfg.num_attention_heads // world, num_key_value_heads=max(1, g // world))
    if cfg.num_experts > 0:
        if cfg.num_experts % world:
            raise ValueError(f"{cfg.num_experts} experts do not divide over {world} ranks")
    else:
        if cfg.intermediate_size % world:
            raise ValueError(f"MLP width {cfg.intermediate_size} does not divide over {world} ranks")
        kw["intermediate_size"] = cfg.intermediate_size // world
    return dataclasses.replace(cfg, extra=dict(cfg.extra), **kw)


def local_layout(cfg: ModelConfig, world: int, rank: int):
    """Parameter shapes of one rank, in the full model's parameter order (the order weight-sync plans assume)."""
    return tp_param_layout(cfg, world, rank, ep=world if cfg.num_experts > 0 else 1)


class _ShardedInference:
    """Mixed in front of DenseModel / MoEModel: partial sums after the row-parallel products, weight localisation."""

    def _bind(self, full_cfg: ModelConfig, shard: Shard) -> None:
        self.full_cfg, self.shard = full_cfg, shard
        E = full_cfg.num_experts
        self.expert_range = (shard.rank * E // shard.world, (shard.rank + 1) * E // shard.world) if E else (0, 0)
        self.params.expert_offset = self.expert_range[0]

    def begin_step(self) -> None:
        self.shard.reduce.begin_step()

    def _lin(self, l: int, name: str, x: torch.Tensor) -> torch.Tensor:
        y = super()._lin(l, name, x)
        return self.shard.reduce(y) if name in _ROW_PARALLEL else y

    def forward(self, *a, **k):
        raise NotImplementedError("a sharded sampler model has no training pass; train with the tensor-parallel trainer models")

    backward = forward

    # ------------------------------------------------------------------ weights
    def localize(self, name: str, t: torch.Tensor):
        """This rank's part of the FULL tensor ``name`` (fused in-house name or HF checkpoint name); None when this
        rank holds nothing of it (another rank's expert)."""
        c, W, r = self.full_cfg, self.shard.world, self.shard.rank
        if W == 1:
            return t
        if name in self.params.layout:
            if name.endswith("w13_weight") or name.endswith("w2_weight"):
                return t[self.expert_range[0]:self.expert_range[1]]
            return slice_full_param(c, name, t, W, r)
        m = _EXPERT.search(name)
        if m:
            return t if self.expert_range[0] <= int(m.group(1)) < self.expert_range[1] else None
        leaf = name.rsplit(".", 2)[-2] if name.count(".") >= 2 else ""

        def rows(n):
            return t[r * n // W:(r + 1) * n // W]

        if leaf == "q_proj":
            return rows(c.q_size)
        if leaf in ("k_proj", "v_proj"):
            if c.num_key_value_heads % W:            # one head, shared with the neighbouring ranks
                kv = r * c.num_key_value_heads // W
                return t[kv * c.head_dim:(kv + 1) * c.head_dim]
            return rows(c.kv_size)
        if leaf == "o_proj":
            return t[:, r * c.q_size // W:(r + 1) * c.q_size // W]
        if leaf in ("gate_proj", "up_proj") and ".mlp." in name and c.num_experts == 0:
            return rows(c.intermediate_size)
        if leaf == "down_proj" and ".mlp." in name and c.num_experts == 0:
            return t[:, r * c.intermediate_size // W:(r + 1) * c.intermediate_size // W]
        return t

    def load_full_state(self, full_views: dict) -> None:
        """Copy from an unsharded model's views, keeping this rank's part."""
        for name, dst in self.params.views.items():
            dst.copy_(self.localize(name, full_views[name]).to(dst.device).to(dst.dtype))

    def load_hf_checkpoint(self, path: str, strict: bool = True) -> list[str]:
        """Stream an HF checkpoint directory, keeping only what this rank holds."""
        from ..utils.hf_model import iter_hf_weights
        sd = {}
        for name, t in iter_hf_weights(path):
            part = self.localize(name, t)
            if part is not None:
                sd[name] = part.contiguous()
        return self.params.load_hf_state_dict(sd, strict=strict)

    def share_replicated_from_first_rank(self) -> None:
        """After a random initialisation: the parameters every rank holds in full must be the same everywhere."""
        if self.shard.world == 1:
            return
        full_lay = self.params.layout
        from .params import param_layout
        whole = param_layout(self.full_cfg)
        src = dist.get_global_rank(self.shard.group, 0)
        for name, v in self.params.views.items():
            if tuple(full_lay[name]) == tuple(whole[name]):
                dist.broadcast(v, src=src, group=self.shard.group)


def _own_or_shared_params(cfg: ModelConfig, lc: ModelConfig, shard: Shard, device, dtype, share):
    """Storage of one rank's part. ``share``: the ``FlatParams`` of a tensor-parallel TRAINER model of the same group
    size (``tp_dense.TPDenseModel`` / ``tp_moe.TPMoEModel`` use the very same per-rank layout): the sampler then reads
    the trainer's live shards - also after the trainer moved them to another buffer - and a weight update moves nothing."""
    if share is not None:
        assert dict(share.layout) == dict(local_layout(cfg, shard.world, shard.rank)), \
            "trainer and sampler disagree about the per-rank parameter layout"
        return share
    return FlatParams(lc, torch.device(device), dtype, layout=local_layout(cfg, shard.world, shard.rank))


class ShardedDenseModel(_ShardedInference, DenseModel):
    def __init__(self, cfg: ModelConfig, shard: Shard, device="cuda", dtype=torch.bfloat16, share=None):
        lc = local_config(cfg, shard.world)
        DenseModel.__init__(self, lc, device, dtype, _own_or_shared_params(cfg, lc, shard, device, dtype, share))
        self._bind(cfg, shard)


class ShardedMoEModel(_ShardedInference, MoEModel):
    def __init__(self, cfg: ModelConfig, shard: Shard, device="cuda", dtype=torch.bfloat16, share=None):
        lc = local_config(cfg, shard.world)
        MoEModel.__init__(self, lc, device, dtype, _own_or_shared_params(cfg, lc, shard, device, dtype, share))
        self._bind(cfg, shard)

    def mlp_infer(self, l: int, h2):
        c = self.cfg
        logits = G.gemm_nt(h2, self._p(l, "mlp.gate.weight"), out_dtype=torch.float32)
        ids, w = M.route(logits, c.num_experts_per_tok, c.norm_topk_prob, None)
        if self.capture_routing:
            if self.last_routing is None:
                self.last_routing = []
            self.last_routing.append(ids)
        e0, e1 = self.expert_range
        mine = ids - e0
        mine = torch.where((mine >= 0) & (mine < e1 - e0), mine, torch.full_like(mine, -1))
        lay = M.align(mine, e1 - e0)
        xs = M.gather(h2, lay)
        a = A.swiglu_fwd(M.grouped_fwd(xs, self._p(l, "mlp.experts.w13_weight"), lay))
        ys = M.grouped_fwd(a, self._p(l, "mlp.experts.w2_weight"), lay)
        return self.shard.reduce(M.combine(ys, w, lay))

    def mlp_fwd(self, *a, **k):
        raise NotImplementedError("a sharded sampler model has no training pass")


def share_trainer_shards(trainer_model, shard: Shard):
    """The sampler-side model of one rank over the SAME storage as a tensor-parallel trainer model of the same group
    (zero-copy colocated deployment); None when the trainer's layout is not the sampler's."""
    inner = getattr(trainer_model, "inner", trainer_model)
    tp = getattr(inner, "tp", None)
    if tp is None or not hasattr(inner, "hq") or tp.world != shard.world or tp.rank != shard.rank or getattr(inner, "shard_head", False):
        return None
    cfg = inner.cfg
    if cfg.num_experts > 0 and getattr(inner, "ep_world", 1) != shard.world:
        return None
    if dict(inner.params.layout) != dict(local_layout(cfg, shard.world, shard.rank)):
        return None                          # e.g. a pipeline stage: it holds a slice of the layers only
    cls = ShardedMoEModel if cfg.num_experts > 0 else ShardedDenseModel
    return cls(cfg, shard, device=inner.device, dtype=inner.dtype, share=inner.params)


def build_sharded_model(model_path, shard: Shard, device="cuda", dtype=torch.bfloat16, seed: int = 0, load_weights: bool = True):
    """The sampler's model for one rank of a tensor-parallel group: preset name -> random init (replicated parameters
    taken from the group's first rank), HF directory -> this rank's part of its weights."""
    import os

    from ..utils.hf_model import has_hf_weights
    from .config import get_config
    from .families import FAMILY_TYPES
    cfg = get_config(model_path)
    if cfg.model_type in FAMILY_TYPES:
        raise NotImplementedError(f"tensor-parallel sampling is built for the dense and Qwen3-MoE layouts, not '{cfg.model_type}'")
    model = (ShardedMoEModel if cfg.num_experts > 0 else ShardedDenseModel)(cfg, shard, device=device, dtype=dtype)
    if load_weights and os.path.isdir(str(model_path)) and has_hf_weights(model_path):
        model.load_hf_checkpoint(model_path)
    else:
        model.params.init_random(seed=seed)
        model.share_replicated_from_first_rank()
    return model
