"""Model FLOPs per step and MFU (reference: axon/utils/profiler/flops_counter.py:47-555).

Training FLOPs are counted as 6 x (matmul parameters) x tokens plus the causal-attention term
12 x sum(seqlen^2) x head_dim x heads x layers (forward + backward, no recompute credit). The device
peak used for MFU is the dense tensor-core rate of the GPU name, bf16 unless another dtype is given.
"""
from __future__ import annotations

import torch

_DEVICE_TFLOPS_BF16 = (("B200", 2250.0), ("B100", 1750.0), ("GB200", 2500.0), ("H200", 989.0), ("H100", 989.0),
                       ("H800", 989.0), ("A100", 312.0), ("A800", 312.0), ("L40", 181.0), ("L20", 119.5), ("H20", 148.0),
                       ("MI300X", 1336.0), ("910B", 354.0))


def _dtype_multiplier(dtype) -> float:
    if dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return 2.0
    if dtype == torch.float32:
        return 0.5
    return 1.0


def get_device_flops(unit: str = "T", dtype=torch.bfloat16, device_name: str | None = None) -> float:
    if device_name is None:
        device_name = torch.cuda.get_device_name() if torch.cuda.is_available() else "cpu"
    tf = next((v for k, v in _DEVICE_TFLOPS_BF16 if k in device_name), float("inf"))
    scale = {"B": 1e3, "K": 1e9, "M": 1e6, "G": 1e3, "T": 1.0, "P": 1e-3}[unit]
    return tf * _dtype_multiplier(dtype) * scale


class FlopsCounter:
    """``estimate_flops(batch_seqlens, delta_time) -> (achieved TFLOP/s, peak TFLOP/s)``."""

    def __init__(self, config, dtype: torch.dtype = torch.bfloat16):
        self.config = getattr(config, "text_config", config)
        self.dtype = dtype
        mt = getattr(self.config, "model_type", "")
        if "deepseek" in mt or "glm5" in mt or "kimi" in mt:
            self._fn = self._mla_moe
        elif "moe" in mt or getattr(self.config, "num_experts", 0):
            self._fn = self._moe
        elif mt in ("", None):
            self._fn = lambda *_: 0.0
        else:
            self._fn = self._dense

    def _c(self, name, default=None):
        return getattr(self.config, name, default)

    def _attn_sizes(self):
        hd = self._c("head_dim") or self._c("hidden_size") // self._c("num_attention_heads")
        return hd, self._c("num_attention_heads") * hd, self._c("num_key_value_heads", self._c("num_attention_heads")) * hd

    def _attention_flops(self, seqlens, head_dim, heads, layers) -> float:
        return 12.0 * sum(s * s for s in seqlens) * head_dim * heads * layers

    def _dense(self, tokens, seqlens) -> float:
        c = self.config
        hd, q, kv = self._attn_sizes()
        per_layer = c.hidden_size * c.intermediate_size * 3 + c.hidden_size * (q + 2 * kv + q)
        n = per_layer * c.num_hidden_layers + 2 * c.vocab_size * c.hidden_size
        return 6.0 * n * tokens + self._attention_flops(seqlens, hd, c.num_attention_heads, c.num_hidden_layers)

    def _moe(self, tokens, seqlens) -> float:
        c = self.config
        hd, q, kv = self._attn_sizes()
        topk = self._c("num_experts_per_tok", 1)
        moe_mlp = c.hidden_size * self._c("moe_intermediate_size", c.intermediate_size) * 3 * topk + c.hidden_size * self._c("num_experts", 1)
        shared = c.hidden_size * self._c("shared_expert_intermediate_size", 0) * 3
        per_layer = moe_mlp + shared + c.hidden_size * (q + 2 * kv + q)
        n = per_layer * c.num_hidden_layers + 2 * c.vocab_size * c.hidden_size
        return 6.0 * n * tokens + self._attention_flops(seqlens, hd, c.num_attention_heads, c.num_hidden_layers)

    def _mla_moe(self, tokens, seqlens) -> float:
        c = self.config
        H, L, heads = c.hidden_size, c.num_hidden_layers, c.num_attention_heads
        qk_nope, qk_rope, v_hd = self._c("qk_nope_head_dim", 128), self._c("qk_rope_head_dim", 64), self._c("v_head_dim", 128)
        q_lora, kv_lora = self._c("q_lora_rank"), self._c("kv_lora_rank", 512)
        q_hd = qk_nope + qk_rope
        attn = (H * q_lora + q_lora * heads * q_hd) if q_lora else H * heads * q_hd
        attn += H * (kv_lora + qk_rope) + kv_lora * heads * (qk_nope + v_hd) + heads * v_hd * H
        first_dense = self._c("first_k_dense_replace", 0)
        moe_layers = max(0, L - first_dense)
        topk, n_shared = self._c("num_experts_per_tok", 8), self._c("n_shared_experts", 1) or 0
        moe_mlp = H * self._c("moe_intermediate_size", 2048) * 3 * (topk + n_shared) + H * self._c("n_routed_experts", 256)
        dense_mlp = H * c.intermediate_size * 3
        n = attn * L + moe_mlp * moe_layers + dense_mlp * first_dense + 2 * c.vocab_size * H
        return 6.0 * n * tokens + 12.0 * sum(s * s for s in seqlens) * (q_hd + v_hd) / 2 * heads * L

    def estimate_flops(self, batch_seqlens, delta_time: float) -> tuple[float, float]:
        seqlens = [int(s) for s in batch_seqlens]
        flops = self._fn(sum(seqlens), seqlens)
        return (flops / max(delta_time, 1e-9) / 1e12, get_device_flops("T", self.dtype))
