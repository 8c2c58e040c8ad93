"""Sampler-side model cut into pipeline stages (inference only).

A group of P sampler ranks holds a model too large for one of them by layers: rank r keeps a contiguous
slice of the decoder layers, their share of the KV cache, and - whole - the embedding, the final norm
and the vocabulary head. The engines of the group run in lockstep (``sampler.server.Lockstep``): every
rank makes the same prefill / decode call; inside it the residual stream travels rank to rank (one
point-to-point pair per stage boundary), and what leaves the last stage is broadcast, so that every
rank computes the same logits and samples the same tokens without exchanging them. Stages work one
after the other - this layout buys capacity, not speed; a tensor-parallel group (``models/tp_infer.py``)
is the faster way to spread a model.

A stage is the whole model's code on a "local" configuration whose layers are the stage's own, renumbered
from zero, so prefill, decode, paged attention and the KV pool are the single-GPU paths; ``localize``
translates full-model tensor names to the stage's (or says that the stage holds nothing of a tensor).

(reference: ``sampler.pipeline_model_parallel_size`` handed to vLLM, axon/sampler/sampler.py:62-91 and
the step ordering of its pipelined executor, axon/sampler/vllm/engine.py:84-88.)
"""
from __future__ import annotations

import dataclasses
import re

import torch
import torch.distributed as dist

from .config import ModelConfig
from .dense import DenseModel
from .moe import MoEModel
from .pp_dense import stage_layers

_LAYER = re.compile(r"^(.*?\blayers\.)(\d+)(\..*)$")


class _StagedInference:
    supports_cuda_graph = False          # the stage boundaries are point-to-point calls

    def _bind(self, full_cfg: ModelConfig, stage) -> None:
        self.full_cfg, self.stage = full_cfg, stage
        self.layer_range = stage_layers(full_cfg.num_hidden_layers, stage.world, stage.rank)
        self._ranks = dist.get_process_group_ranks(stage.group) if stage.world > 1 else [0]

    def begin_step(self) -> None:
        pass

    # ------------------------------------------------------------------ the stream between stages
    def _stage_in(self, x):
        if self.stage.rank == 0:
            return x, None
        got = torch.empty(2, *x.shape, dtype=x.dtype, device=x.device)
        dist.recv(got, src=self._ranks[self.stage.rank - 1], group=self.stage.group)
        return got[0], got[1]

    def _stage_out(self, x, delta):
        st = self.stage
        if st.world == 1:
            return x, delta
        both = torch.stack([x, delta])
        if st.rank < st.world - 1:
            dist.send(both, dst=self._ranks[st.rank + 1], group=st.group)
        dist.broadcast(both, src=self._ranks[-1], group=st.group)        # what left the last stage, for everybody's head
        return both[0], both[1]

    def forward(self, *a, **k):
        raise NotImplementedError("a sampler stage has no training pass; train with the pipeline-parallel trainer models")

    backward = forward

    # ------------------------------------------------------------------ weights
    def local_name(self, name: str) -> str | None:
        """Full-model tensor name -> this stage's name; None when the stage does not hold the tensor."""
        m = _LAYER.match(name)
        if not m:
            return name                                   # embedding, final norm, head: on every stage
        g = int(m.group(2))
        if g not in self.layer_range:
            return None
        return f"{m.group(1)}{g - self.layer_range.start}{m.group(3)}"

    def localize(self, name: str, t: torch.Tensor):
        local = self.local_name(name)
        return None if local is None else (local, t)

    def load_full_state(self, full_views: dict) -> None:
        for name, src in full_views.items():
            local = self.local_name(name)
            if local is not None and local in self.params.views:
                dst = self.params.views[local]
                dst.copy_(src.to(dst.device).to(dst.dtype))

    def load_hf_checkpoint(self, path: str, strict: bool = True) -> list[str]:
        from ..utils.hf_model import iter_hf_weights
        sd = {}
        for name, t in iter_hf_weights(path):
            local = self.local_name(name)
            if local is not None:
                sd[local] = t
        return self.params.load_hf_state_dict(sd, strict=strict)


def _stage_config(cfg: ModelConfig, stage) -> ModelConfig:
    n = len(stage_layers(cfg.num_hidden_layers, stage.world, stage.rank))
    assert n >= 1, f"{cfg.num_hidden_layers} layers do not give every one of {stage.world} stages a layer"
    # a multi-token-prediction module behind the decoder is a training device: no stage holds it (``local_name`` -> None)
    return dataclasses.replace(cfg, num_hidden_layers=n, num_nextn_predict_layers=0, extra=dict(cfg.extra))


class StagedDenseModel(_StagedInference, DenseModel):
    def __init__(self, cfg: ModelConfig, stage, device="cuda", dtype=torch.bfloat16):
        DenseModel.__init__(self, _stage_config(cfg, stage), device, dtype)
        self._bind(cfg, stage)


class StagedMoEModel(_StagedInference, MoEModel):
    def __init__(self, cfg: ModelConfig, stage, device="cuda", dtype=torch.bfloat16):
        MoEModel.__init__(self, _stage_config(cfg, stage), device, dtype)
        self._bind(cfg, stage)


def build_staged_model(model_path, stage, device="cuda", dtype=torch.bfloat16, seed: int = 0, load_weights: bool = True):
    """One stage of a pipelined sampler group: preset name -> random init (the same full-model draw on every rank, cut
    down to the stage), HF directory -> the stage's part of its weights."""
    import os

    from ..utils.hf_model import has_hf_weights
    from .config import get_config
    from .families import FAMILY_TYPES
    from .params import FlatParams
    cfg = get_config(model_path)
    if cfg.model_type in FAMILY_TYPES:
        raise NotImplementedError(f"pipelined sampling is built for the dense and Qwen3-MoE layouts, not '{cfg.model_type}'")
    model = (StagedMoEModel if cfg.num_experts > 0 else StagedDenseModel)(cfg, stage, device=device, dtype=dtype)
    if load_weights and os.path.isdir(str(model_path)) and has_hf_weights(model_path):
        model.load_hf_checkpoint(model_path)
    elif load_weights:
        ref = FlatParams(cfg, "cpu", dtype)
        ref.init_random(seed=seed)
        model.load_full_state(ref.views)
    return model
