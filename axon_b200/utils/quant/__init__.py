"""Quantising generators for the weight hand-over to a low-precision sampler.

Each generator takes ``(name, tensor)`` pairs (HF names) and yields the pairs the sampler loads:
quantised weights plus their scale tensors under the names serving engines expect, everything else
unchanged (reference: axon/utils/sglang/fp8.py:117-300, int4.py:309-420, mxfp8.py:51-160 and the
fp8 refit path axon/monkey_patches/vllm/fp8/vllm_fp8_patch.py:1264-1330).

Which parameters are quantised: 2-D ``.weight`` tensors of linear projections (attention q/k/v/o and
their MLA / indexer / linear-attention variants, MLP and expert projections). Embeddings, the output
head, every norm, MoE routers / gates and GLM-5's ``eh_proj`` / ``weights_proj`` stay in bf16.
"""
from __future__ import annotations

import re
from typing import Iterable, Iterator

import torch

from ...ops import quant as Q

_EXCLUDE = ("embed_tokens", "lm_head", "layernorm", "norm", "ln_", "embeddings", "router", "mlp.gate.", "eh_proj",
            "weights_proj")
_INCLUDE = ("q_proj", "k_proj", "v_proj", "o_proj", "qkv_proj", "gate_proj", "up_proj", "gate_up_proj", "down_proj", "fc1",
            "fc2", "experts", "shared_experts", "q_a_proj", "q_b_proj", "kv_a_proj", "kv_b_proj", "wq_b", "wk",
            "in_proj_qkv", "in_proj_z", "out_proj", "w13_weight", "w2_weight")


def should_quantize_param(name: str) -> bool:
    low = name.lower()
    if not (low.endswith(".weight") or low.endswith("_weight")):
        return False
    if any(p in low for p in _EXCLUDE):
        return False
    return any(p in low for p in _INCLUDE)


def _matches_ignore(name: str, rules: Iterable[str]) -> bool:
    """Rules are exact names, name prefixes (module paths) or ``re:<regex>`` patterns."""
    for rule in rules or ():
        if rule.startswith("re:"):
            if re.match(rule[3:], name):
                return True
        elif name == rule or name.startswith(rule + ".") or name == rule + ".weight":
            return True
    return False


def _eligible(name: str, t: torch.Tensor, ignore, multiple: int) -> bool:
    return (t.dim() >= 2 and t.dtype in (torch.bfloat16, torch.float16, torch.float32) and should_quantize_param(name)
            and not _matches_ignore(name, ignore) and t.shape[-1] % multiple == 0)


def _as_2d(t: torch.Tensor) -> torch.Tensor:
    return t.reshape(-1, t.shape[-1]).to(torch.bfloat16)


def fp8_quantize_weight_generator(weights: Iterable, ignore: Iterable[str] = ()) -> Iterator:
    """128x128-block e4m3 weights + ``<name>_scale_inv`` fp32 block scales (dequant = q * scale_inv)."""
    for name, t in weights:
        if not _eligible(name, t, ignore, 1):
            yield name, t
            continue
        if t.dim() == 2:
            q, s = Q.fp8_block_quant(_as_2d(t))
        else:                                                # stacked experts: quantise each matrix
            qs = [Q.fp8_block_quant(_as_2d(m)) for m in t]
            q, s = torch.stack([a for a, _ in qs]), torch.stack([b for _, b in qs])
        yield name, q
        yield name + "_scale_inv", s


def int4_quantize_weight_generator(weights: Iterable, group_size: int = 128, ignore: Iterable[str] = ()) -> Iterator:
    """compressed-tensors pack-quantized layout: ``<base>.weight_packed`` int32 [M, N/8],
    ``<base>.weight_scale`` and ``<base>.weight_shape`` (symmetric: no zero points)."""
    for name, t in weights:
        if not _eligible(name, t, ignore, group_size) or t.dim() != 2:
            yield name, t
            continue
        packed, scales = Q.int4_quant_pack(_as_2d(t), group_size)
        base = name[: -len(".weight")] if name.endswith(".weight") else name
        yield base + ".weight_packed", packed
        yield base + ".weight_scale", scales
        yield base + ".weight_shape", torch.tensor(list(t.shape), dtype=torch.int64, device=t.device)


def mxfp8_quantize_weight_generator(weights: Iterable, ignore: Iterable[str] = ()) -> Iterator:
    """e4m3 weights + ``<name>_scale_inv`` UE8M0 bytes, one per 32 values along the row."""
    for name, t in weights:
        if not _eligible(name, t, ignore, Q.MXFP8_GROUP):
            yield name, t
            continue
        q, s = Q.mxfp8_quant(_as_2d(t))
        yield name, q.reshape(t.shape)
        yield name + "_scale_inv", s.reshape(*t.shape[:-1], t.shape[-1] // Q.MXFP8_GROUP)


QUANT_GENERATORS = {"fp8": fp8_quantize_weight_generator, "fp8_fast": fp8_quantize_weight_generator,
                    "int4": int4_quantize_weight_generator, "mxfp8": mxfp8_quantize_weight_generator}


def quantize_weights(weights: Iterable, method: str | None, **kw) -> Iterator:
    if not method:
        yield from weights
        return
    if method not in QUANT_GENERATORS:
        raise ValueError(f"unknown quantization '{method}' (expected one of {sorted(QUANT_GENERATORS)})")
    yield from QUANT_GENERATORS[method](weights, **kw)
