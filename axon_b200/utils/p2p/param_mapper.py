"""Parameter metadata for weight sync: how each side's flat parameter buffer is laid out under
tensor / expert parallelism, and the sampler-side fused names.

``convert_hf_to_vllm_param_name``: q/k/v -> ``qkv_proj``, gate/up -> ``gate_up_proj``, per-expert
gate/up -> ``w13_weight`` and down -> ``w2_weight`` (reference: axon/utils/p2p/param_mapper.py:367-413).
``shard_layout`` describes how one rank of a (tp, ep) layout slices every fused parameter of the
in-house models: column-parallel tensors split rows, row-parallel tensors split columns, QKV is split
per KV-head group so that every rank keeps whole GQA groups (q rows | k rows | v rows of its groups),
gate_up keeps the two halves, experts are distributed over EP ranks.
"""
from __future__ import annotations

import re

import torch

from ...models.config import ModelConfig
from ...models.params import param_layout
from .routing_table import ParameterMetadata, RankMapping

_QKV = re.compile(r"\.(q_proj|k_proj|v_proj)\.")
_GU = re.compile(r"\.(gate_proj|up_proj)\.")
_EXPERT = re.compile(r"\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")


def extract_expert_idx(name: str) -> int:
    m = re.search(r"\.experts\.(\d+)\.", name)
    return int(m.group(1)) if m else -1


def convert_hf_to_vllm_param_name(name: str) -> tuple[str, str | None]:
    """(fused sampler-side name, shard id) for an HF parameter name; shard id is 'q'/'k'/'v',
    'gate'/'up', or for experts ('w1'|'w3'|'w2', expert index) encoded as 'w1:7'."""
    m = _EXPERT.search(name)
    if m:
        e, kind = int(m.group(1)), m.group(2)
        base = name[: m.start()] + ".experts."
        if kind == "down_proj":
            return base + "w2_weight", f"w2:{e}"
        return base + "w13_weight", f"{'w1' if kind == 'gate_proj' else 'w3'}:{e}"
    m = _QKV.search(name)
    if m:
        return name.replace(m.group(0), ".qkv_proj."), m.group(1)[0]
    m = _GU.search(name)
    if m:
        return name.replace(m.group(0), ".gate_up_proj."), m.group(1).split("_")[0]
    return name, None


# split kind of every fused parameter of the in-house layout
def split_kind(name: str) -> str:
    if name.endswith("qkv_proj.weight") or name.endswith("qkv_proj.bias"):
        return "qkv"                       # the bias vector splits like the rows of its matrix
    if name.endswith("gate_up_proj.weight"):
        return "gate_up"
    if name.endswith("o_proj.weight") or name.endswith("down_proj.weight"):
        return "row"                       # row-parallel: split the input (column) dimension
    if name.endswith("embed_tokens.weight") or name.endswith("lm_head.weight"):
        return "vocab"                     # split rows
    if name.endswith("w13_weight") or name.endswith("w2_weight"):
        return "expert"
    return "replicated"


def shard_rows(cfg: ModelConfig, name: str, tp: int, tp_rank: int, ep: int = 1, ep_rank: int = 0, replicated_names=()):
    """The slices of the FULL fused parameter that one rank holds, as a list of
    (row_start, row_end, col_start, col_end) boxes in full-parameter coordinates (experts: dim 0 is the
    expert index and boxes cover whole experts)."""
    shape = param_layout(cfg)[name]
    kind = "replicated" if name in replicated_names else split_kind(name)
    D = cfg.head_dim
    if kind == "replicated" or (tp == 1 and kind != "expert"):
        return [(0, shape[0], 0, shape[1] if len(shape) > 1 else 1)]
    if kind == "qkv":
        g = cfg.num_key_value_heads
        qo, ko, vo = 0, cfg.q_size, cfg.q_size + cfg.kv_size
        H = shape[1] if len(shape) > 1 else 1
        if g % tp != 0:
            # more ranks than key / value heads (a sampler group): every rank takes its share of the query heads and
            # the ONE key / value head they attend to, which tp / g ranks hold alike
            assert tp % g == 0 and cfg.num_attention_heads % tp == 0, f"{cfg.num_attention_heads} query / {g} key-value heads do not divide over tp {tp}"
            hq, kv = cfg.num_attention_heads // tp, tp_rank * g // tp
            return [(qo + tp_rank * hq * D, qo + (tp_rank + 1) * hq * D, 0, H), (ko + kv * D, ko + (kv + 1) * D, 0, H),
                    (vo + kv * D, vo + (kv + 1) * D, 0, H)]
        rep = cfg.num_attention_heads // g
        g0, g1 = tp_rank * g // tp, (tp_rank + 1) * g // tp
        return [(qo + g0 * rep * D, qo + g1 * rep * D, 0, H), (ko + g0 * D, ko + g1 * D, 0, H),
                (vo + g0 * D, vo + g1 * D, 0, H)]
    if kind == "gate_up":
        F = shape[0] // 2
        f0, f1 = tp_rank * F // tp, (tp_rank + 1) * F // tp
        return [(f0, f1, 0, shape[1]), (F + f0, F + f1, 0, shape[1])]
    if kind == "row":
        c0, c1 = tp_rank * shape[1] // tp, (tp_rank + 1) * shape[1] // tp
        return [(0, shape[0], c0, c1)]
    if kind == "vocab":
        r0, r1 = tp_rank * shape[0] // tp, (tp_rank + 1) * shape[0] // tp
        return [(r0, r1, 0, shape[1])]
    if kind == "expert":
        E = shape[0]
        e0, e1 = ep_rank * E // ep, (ep_rank + 1) * E // ep
        return [(e0, e1, 0, shape[1] * shape[2])]
    raise ValueError(kind)


def get_param_metadata(cfg: ModelConfig, rank: int, tp: int = 1, tp_rank: int = 0, ep: int = 1, ep_rank: int = 0,
                       dtype=torch.bfloat16, replicated_names=()) -> RankMapping:
    """One rank's ``RankMapping``: a ``ParameterMetadata`` per fused parameter with its shard shape,
    split dim and split index (tp rank for dense tensors, ep rank for expert tensors).
    ``replicated_names``: parameters this rank holds in full although their kind could be split
    (a tensor-parallel trainer that keeps the embedding and the head whole)."""
    out = []
    replicated_names = set(replicated_names)
    for name, full in param_layout(cfg).items():
        kind = "replicated" if name in replicated_names else split_kind(name)
        boxes = shard_rows(cfg, name, tp, tp_rank, ep, ep_rank, replicated_names)
        if kind == "expert":
            shape = (boxes[0][1] - boxes[0][0], *full[1:])
            out.append(ParameterMetadata(name, name, shape, tuple(full), dtype, split_dim=0, split_idx=ep_rank,
                                         metadata={"kind": kind, "boxes": boxes}))
            continue
        rows = sum(b[1] - b[0] for b in boxes)
        cols = boxes[0][3] - boxes[0][2]
        shape = (rows,) if len(full) == 1 else (rows, cols)
        replicated = kind == "replicated" or tp == 1
        out.append(ParameterMetadata(name, name, shape, tuple(full), dtype, split_dim=-1 if replicated else (1 if kind == "row" else 0),
                                     split_idx=0 if replicated else tp_rank, metadata={"kind": kind, "boxes": boxes}))
    return RankMapping(rank=rank, params=out)
