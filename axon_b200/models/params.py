"""Flat parameter storage for the in-house decoder family.

All parameters of a model live in ONE flat bf16 (or fp32 on CPU) buffer; each named parameter is
a view into it. The fp32 main-gradient buffer and the optimizer state use the same offsets, so
the optimizer is a single fused kernel over a contiguous shard and data-parallel sharding is a
plain range split. Fused projections keep the sampler-side names of the reference
(``qkv_proj``, ``gate_up_proj``: axon/utils/p2p/param_mapper.py:367-413) and are mapped to/from
HF checkpoint names (``q_proj``/``k_proj``/``v_proj``, ``gate_proj``/``up_proj``) on load/save.
"""
from __future__ import annotations

from collections import OrderedDict

import torch

from .config import ModelConfig

ALIGN = 128  # elements; keeps every view 256-byte aligned for TMA


def param_layout(cfg: ModelConfig) -> "OrderedDict[str, tuple[int, ...]]":
    H, D = cfg.hidden_size, cfg.head_dim
    lay: OrderedDict[str, tuple[int, ...]] = OrderedDict()
    lay["model.embed_tokens.weight"] = (cfg.vocab_size, H)
    for l in range(cfg.num_hidden_layers + cfg.num_nextn_predict_layers):
        p = f"model.layers.{l}."
        if l >= cfg.num_hidden_layers:          # multi-token-prediction module: input norms + projection, then a decoder layer
            lay[p + "enorm.weight"] = (H,)
            lay[p + "hnorm.weight"] = (H,)
            lay[p + "eh_proj.weight"] = (H, 2 * H)
            lay[p + "shared_head.norm.weight"] = (H,)
        lay[p + "input_layernorm.weight"] = (H,)
        lay[p + "self_attn.qkv_proj.weight"] = (cfg.qkv_size, H)
        if cfg.attention_bias:
            lay[p + "self_attn.qkv_proj.bias"] = (cfg.qkv_size,)
        if cfg.qk_norm:
            lay[p + "self_attn.q_norm.weight"] = (D,)
            lay[p + "self_attn.k_norm.weight"] = (D,)
        lay[p + "self_attn.o_proj.weight"] = (H, cfg.q_size)
        lay[p + "post_attention_layernorm.weight"] = (H,)
        if cfg.sandwich_norm:
            lay[p + "post_self_attn_layernorm.weight"] = (H,)
            lay[p + "post_mlp_layernorm.weight"] = (H,)
        if cfg.num_experts > 0:
            F = cfg.moe_intermediate_size
            lay[p + "mlp.gate.weight"] = (cfg.num_experts, H)
            lay[p + "mlp.experts.w13_weight"] = (cfg.num_experts, 2 * F, H)
            lay[p + "mlp.experts.w2_weight"] = (cfg.num_experts, H, F)
        else:
            lay[p + "mlp.gate_up_proj.weight"] = (2 * cfg.intermediate_size, H)
            lay[p + "mlp.down_proj.weight"] = (H, cfg.intermediate_size)
    lay["model.norm.weight"] = (H,)
    if not cfg.tie_word_embeddings:
        lay["lm_head.weight"] = (cfg.vocab_size, H)
    if cfg.extra.get("value_head", False):          # critic / reward model: scalar head on the final hidden state
        lay["v_head.weight"] = (1, H)
    return lay


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


def rope_row_perm(cfg: ModelConfig) -> "torch.Tensor | None":
    """Per-head permutation of the q / k output rows between a checkpoint's rotary layout and the layout the
    kernels rotate (pairs (i, i + D/2), rotating pairs first): ``ours[i] = checkpoint[perm[i]]``. None when the
    checkpoint already has that layout (full rotary, half-split pairs)."""
    D, r = cfg.head_dim, cfg.rotary_dim
    if r == D and not cfg.rope_interleaved:
        return None
    half, rh, ph = D // 2, r // 2, (D - r) // 2
    perm = torch.empty(D, dtype=torch.long)
    for p in range(rh):
        a, b = (2 * p, 2 * p + 1) if cfg.rope_interleaved else (p, rh + p)
        perm[p], perm[half + p] = a, b
    for j in range(ph):                      # dims that do not rotate: any fixed pairing works, q and k share it
        perm[rh + j], perm[half + rh + j] = r + j, r + ph + j
    return perm


def _permute_heads(t: torch.Tensor, perm: torch.Tensor, head_dim: int) -> torch.Tensor:
    """Rows of ``t`` ([heads * D, ...]) re-ordered inside every head."""
    heads = t.shape[0] // head_dim
    idx = (torch.arange(heads)[:, None] * head_dim + perm[None, :]).reshape(-1).to(t.device)
    return t[idx]


class FlatParams:
    """Named views over one flat buffer (+ optional fp32 main grads with the same offsets)."""

    def __init__(self, cfg: ModelConfig, device, dtype=torch.bfloat16, flat: torch.Tensor | None = None,
                 layout: "OrderedDict[str, tuple[int, ...]] | None" = None):
        self.cfg = cfg
        self.layout = layout if layout is not None else param_layout(cfg)
        self.offsets: dict[str, tuple[int, int]] = {}
        off = 0
        for name, shape in self.layout.items():
            n = _numel(shape)
            self.offsets[name] = (off, n)
            off += (n + ALIGN - 1) // ALIGN * ALIGN
        self.numel = (off + 8191) // 8192 * 8192   # divisible by any power-of-two data-parallel size <= 64
        self.device = torch.device(device)
        self.dtype = dtype
        self.flat = flat if flat is not None else torch.zeros(self.numel, dtype=dtype, device=self.device)
        assert self.flat.numel() >= self.numel
        self.views = {n: self.flat[o:o + k].view(self.layout[n]) for n, (o, k) in self.offsets.items()}
        self.grad_flat: torch.Tensor | None = None
        self.grads: dict[str, torch.Tensor] = {}
        self.expert_offset = 0         # global index of the first expert held (a rank that holds a slice of the experts)

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.views[name]

    def rebind(self, flat: torch.Tensor) -> None:
        """Point every named view at a new flat buffer (an empty one drops the views: parameters
        parked on the host). Consumers that cached views must fetch them again."""
        self.flat = flat
        if flat.numel() >= self.numel:
            self.views = {n: flat[o:o + k].view(self.layout[n]) for n, (o, k) in self.offsets.items()}
        else:
            self.views = {}

    def names(self):
        return list(self.layout.keys())

    def init_random(self, std: float = 0.02, seed: int = 0) -> None:
        """N(0, std) for matrices, ones for norm weights (random-init weights of the architecture)."""
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        for name, v in self.views.items():
            if v.dim() == 1 and name.endswith(".bias"):
                v.copy_((torch.randn(v.shape, generator=g, device=self.device) * std).to(v.dtype))
            elif v.dim() == 1:
                v.fill_(1.0)
            else:
                # generate in chunks to bound the fp32 temporary
                flat = v.view(-1)
                step = 1 << 26
                for s in range(0, flat.numel(), step):
                    e = min(flat.numel(), s + step)
                    flat[s:e] = (torch.randn(e - s, generator=g, device=self.device, dtype=torch.float32) * std).to(v.dtype)

    def alloc_grads(self, grad_flat: torch.Tensor | None = None) -> None:
        if self.grad_flat is None:
            self.grad_flat = grad_flat if grad_flat is not None else torch.zeros(
                self.numel, dtype=torch.float32, device=self.device)
            self.grads = {n: self.grad_flat[o:o + k].view(self.layout[n]) for n, (o, k) in self.offsets.items()}

    def free_grads(self) -> None:
        if getattr(self, "grads_persistent", False):      # buffer lives in symmetric memory: keep the mapping
            return
        self.grad_flat = None
        self.grads = {}

    def zero_grads(self) -> None:
        if self.grad_flat is not None:
            self.grad_flat.zero_()

    # ------------------------------------------------------------------ HF name mapping
    def to_hf_state_dict(self, export: bool = True) -> "OrderedDict[str, torch.Tensor]":
        """HF-named tensors. With ``export`` they have the checkpoint's values (q / k rows of partial- or
        interleaved-rotary families are re-ordered copies); without it they are views of the buffers in this
        framework's row order, which ``load_hf_state_dict`` fills and then re-orders in place."""
        cfg = self.cfg
        perm = rope_row_perm(cfg)
        inv = None if perm is None else torch.argsort(perm)
        out: OrderedDict[str, torch.Tensor] = OrderedDict()
        for name, v in self.views.items():
            if name.endswith("qkv_proj.weight") or name.endswith("qkv_proj.bias"):
                kind = name.rsplit(".", 1)[1]
                base = name[: -len("qkv_proj." + kind)]
                q, k, vv = v.split([cfg.q_size, cfg.kv_size, cfg.kv_size], 0)
                if export and inv is not None:          # back to the checkpoint's rotary layout (copies, not views)
                    q, k = _permute_heads(q, inv, cfg.head_dim), _permute_heads(k, inv, cfg.head_dim)
                out[base + "q_proj." + kind], out[base + "k_proj." + kind], out[base + "v_proj." + kind] = q, k, vv
            elif name.endswith("gate_up_proj.weight") and cfg.model_type == "glm4":
                out[name] = v                           # GLM-4 checkpoints keep gate and up fused
            elif name.endswith("gate_up_proj.weight"):
                base = name[: -len("gate_up_proj.weight")]
                g, u = v.split(cfg.intermediate_size, 0)
                out[base + "gate_proj.weight"], out[base + "up_proj.weight"] = g, u
            elif name.endswith("experts.w13_weight"):
                base = name[: -len("w13_weight")]
                F = cfg.moe_intermediate_size
                for e in range(v.shape[0]):
                    out[f"{base}{e + self.expert_offset}.gate_proj.weight"] = v[e, :F]
                    out[f"{base}{e + self.expert_offset}.up_proj.weight"] = v[e, F:]
            elif name.endswith("experts.w2_weight"):
                base = name[: -len("w2_weight")]
                for e in range(v.shape[0]):
                    out[f"{base}{e + self.expert_offset}.down_proj.weight"] = v[e]
            else:
                out[name] = v
        return out

    def load_hf_state_dict(self, sd: dict, strict: bool = True) -> list[str]:
        """Copy HF-named tensors into the fused views. Returns the list of missing HF names."""
        missing = []
        perm = rope_row_perm(self.cfg)
        for hf_name, dst in self.to_hf_state_dict(export=False).items():
            src = sd.get(hf_name)
            if src is None:
                if hf_name == "lm_head.weight" and "model.embed_tokens.weight" in sd:
                    src = sd["model.embed_tokens.weight"]
                else:
                    missing.append(hf_name)
                    continue
            src = src.to(dst.dtype)
            if perm is not None and hf_name.rsplit(".", 2)[-2] in ("q_proj", "k_proj"):
                src = _permute_heads(src, perm, self.cfg.head_dim)       # checkpoint rotary layout -> kernel layout
            dst.copy_(src)
        if strict and missing:
            raise KeyError(f"missing tensors in checkpoint: {missing[:5]} ... ({len(missing)} total)")
        return missing
