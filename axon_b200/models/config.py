"""Model configurations of the in-house decoder family (dense Qwen3 / Llama-3 style).

One definition serves the trainer and the sampler, so their numerics agree by construction.
Field names follow the HF config keys the reference reads through ``AutoConfig``
(axon/trainer/fsdp_trainer.py:186-260, axon/utils/hf_model.py).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path


@dataclass
class ModelConfig:
    model_type: str = "qwen3"
    vocab_size: int = 151936
    hidden_size: int = 4096
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 12288
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    qk_norm: bool = True
    attention_bias: bool = False      # bias on the q / k / v projections (Qwen2 / Qwen2.5 family)
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 40960
    eos_token_id: int = 151645
    pad_token_id: int = 151643
    # MoE (0 experts = dense)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    partial_rotary_factor: float = 1.0    # share of the head dims that rotate (GLM-4: 0.5)
    rope_interleaved: bool = False        # checkpoint pairs rotary dims (2i, 2i+1) instead of (i, i + half): GLM family
    sandwich_norm: bool = False           # extra RMSNorm on the attention and MLP outputs before the residual add (GLM-4)
    num_nextn_predict_layers: int = 0     # multi-token-prediction modules after the decoder (DeepSeek-V3 style, depth 1)
    extra: dict = field(default_factory=dict)

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor) // 2 * 2

    @property
    def qkv_size(self) -> int:
        return self.q_size + 2 * self.kv_size

    def num_params(self) -> int:
        H, F, L, V = self.hidden_size, self.intermediate_size, self.num_hidden_layers, self.vocab_size
        per_layer = self.qkv_size * H + H * self.q_size + 2 * H
        if self.qk_norm:
            per_layer += 2 * self.head_dim
        if self.attention_bias:
            per_layer += self.qkv_size
        if self.num_experts > 0:
            per_layer += self.num_experts * H + self.num_experts * 3 * H * self.moe_intermediate_size
        else:
            per_layer += 3 * H * F
        emb = V * H * (1 if self.tie_word_embeddings else 2)
        return L * per_layer + emb + H

    def to_hf_dict(self) -> dict:
        if "hf_config" in self.extra:            # families described by their own HF config (models/families.py)
            hf = dict(self.extra["hf_config"])
            return dict(hf["_nested_config"]) if "_nested_config" in hf else hf
        d = asdict(self)
        d.pop("extra")
        d.update(self.extra)
        d["architectures"] = [{"qwen3": "Qwen3ForCausalLM", "llama": "LlamaForCausalLM", "qwen2": "Qwen2ForCausalLM",
                               "mistral": "MistralForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM", "glm4": "Glm4ForCausalLM"}.get(self.model_type, "Qwen3ForCausalLM")]
        return d

    @classmethod
    def from_hf_dict(cls, d: dict) -> "ModelConfig":
        from .families import FAMILY_TYPES, TEXT_ONLY_OF, family_config
        if d.get("model_type") in FAMILY_TYPES or (d.get("model_type") in TEXT_ONLY_OF and "text_config" in d):
            return family_config(d)
        known = {f for f in cls.__dataclass_fields__ if f != "extra"}
        kw = {k: v for k, v in d.items() if k in known}
        if "head_dim" not in kw and "hidden_size" in d and "num_attention_heads" in d:
            kw["head_dim"] = d["hidden_size"] // d["num_attention_heads"]
        mt = d.get("model_type", "qwen3")
        if "qk_norm" not in kw:
            kw["qk_norm"] = mt.startswith("qwen3")
        if mt == "glm4":                      # GLM-4 dense: half of each head rotates (interleaved pairs), sandwich norms, q/k/v bias
            kw.setdefault("partial_rotary_factor", 0.5)
            kw["rope_interleaved"], kw["sandwich_norm"], kw["qk_norm"] = True, True, False
            kw.setdefault("attention_bias", True)
        supported = ("qwen3", "qwen3_moe", "qwen2", "llama", "mistral", "glm4")
        if mt not in supported:
            raise NotImplementedError(f"model_type '{mt}' is not among the decoder families built here {supported}")
        if mt == "mistral" and d.get("sliding_window") and d.get("sliding_window") < d.get("max_position_embeddings", 0):
            kw.setdefault("max_position_embeddings", d["sliding_window"])
            kw["max_position_embeddings"] = min(kw["max_position_embeddings"], d["sliding_window"])      # full attention inside the window only
        if "attention_bias" not in d and mt == "qwen2":      # Qwen2 checkpoints carry q/k/v biases without a config flag
            kw["attention_bias"] = True
        if isinstance(kw.get("eos_token_id"), list):
            kw["eos_token_id"] = kw["eos_token_id"][0]
        if kw.get("pad_token_id") is None:
            kw["pad_token_id"] = kw.get("eos_token_id", 0)
        return cls(**kw)

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        return cls.from_hf_dict(json.loads((Path(path) / "config.json").read_text()))

    def save_pretrained(self, path: str) -> None:
        Path(path).mkdir(parents=True, exist_ok=True)
        (Path(path) / "config.json").write_text(json.dumps(self.to_hf_dict(), indent=2))


def qwen3_8b() -> ModelConfig:
    return ModelConfig()


def llama3_8b() -> ModelConfig:
    return ModelConfig(model_type="llama", vocab_size=128256, hidden_size=4096, num_hidden_layers=32,
                       num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336,
                       rms_norm_eps=1e-5, rope_theta=5e5, qk_norm=False, max_position_embeddings=131072,
                       eos_token_id=128009, pad_token_id=128009)


def qwen2_5_7b() -> ModelConfig:
    return ModelConfig(model_type="qwen2", vocab_size=152064, hidden_size=3584, num_hidden_layers=28, num_attention_heads=28,
                       num_key_value_heads=4, head_dim=128, intermediate_size=18944, qk_norm=False, attention_bias=True,
                       max_position_embeddings=32768)


def qwen3_30b_a3b() -> ModelConfig:
    return ModelConfig(model_type="qwen3_moe", hidden_size=2048, num_hidden_layers=48, num_attention_heads=32,
                       num_key_value_heads=4, head_dim=128, intermediate_size=6144, num_experts=128,
                       num_experts_per_tok=8, moe_intermediate_size=768)


def tiny_qwen3() -> ModelConfig:
    """The 2-layer CPU/gloo configuration: d_model 256, 4 q / 2 kv heads of 64, FFN 688, vocab 4096, tied."""
    return ModelConfig(vocab_size=4096, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, intermediate_size=688, tie_word_embeddings=True,
                       max_position_embeddings=4096, eos_token_id=1, pad_token_id=0)


def tiny_gpu() -> ModelConfig:
    """A small head-dim-128 model for GPU smoke tests."""
    return ModelConfig(vocab_size=8192, hidden_size=512, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=128, intermediate_size=1024, tie_word_embeddings=False,
                       max_position_embeddings=8192, eos_token_id=1, pad_token_id=0)


def tiny_moe() -> ModelConfig:
    """A small sparse model (8 experts, top-2, head dim 64) for CPU tests."""
    return ModelConfig(model_type="qwen3_moe", vocab_size=2048, hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, intermediate_size=256, tie_word_embeddings=False,
                       max_position_embeddings=2048, eos_token_id=1, pad_token_id=0, num_experts=8,
                       num_experts_per_tok=2, moe_intermediate_size=128, norm_topk_prob=True)


def tiny_moe_gpu() -> ModelConfig:
    """Sparse GPU smoke model: head dim 128, 16 experts top-4, expert FFN 256."""
    return ModelConfig(model_type="qwen3_moe", vocab_size=8192, hidden_size=512, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=128, intermediate_size=1024, tie_word_embeddings=False,
                       max_position_embeddings=8192, eos_token_id=1, pad_token_id=0, num_experts=16,
                       num_experts_per_tok=4, moe_intermediate_size=256, norm_topk_prob=True)


PRESETS = {"qwen3-8b": qwen3_8b, "llama3-8b": llama3_8b, "qwen2.5-7b": qwen2_5_7b,
           "tiny-qwen2": lambda: _with(tiny_qwen3(), model_type="qwen2", qk_norm=False, attention_bias=True), "qwen3-30b-a3b": qwen3_30b_a3b,
           "tiny-qwen3": tiny_qwen3, "tiny-qwen3-untied": lambda: _untied(tiny_qwen3()),
           "tiny-glm4": lambda: _with(tiny_qwen3(), model_type="glm4", qk_norm=False, attention_bias=True, partial_rotary_factor=0.5,
                                    rope_interleaved=True, sandwich_norm=True, tie_word_embeddings=False),
           "tiny-qwen3-mtp": lambda: _with(tiny_qwen3(), num_nextn_predict_layers=1),
           "tiny-qwen3-untied-mtp": lambda: _with(_untied(tiny_qwen3()), num_nextn_predict_layers=1),
           "tiny-moe-mtp": lambda: _with(tiny_moe(), num_nextn_predict_layers=1),
           "tiny-qwen3-5l": lambda: _with(tiny_qwen3(), num_hidden_layers=5),
           "tiny-qwen3-untied-5l": lambda: _with(_untied(tiny_qwen3()), num_hidden_layers=5), "tiny-gpu": tiny_gpu, "tiny-moe": tiny_moe, "tiny-moe-gpu": tiny_moe_gpu}


def _with(cfg: ModelConfig, **kw) -> ModelConfig:
    for k, v in kw.items():
        setattr(cfg, k, v)
    return cfg


def _untied(cfg: ModelConfig) -> ModelConfig:
    cfg.tie_word_embeddings = False
    return cfg


def _tiny_family(kind: str) -> ModelConfig:
    """Small random-init members of the families of ``models/families.py`` (tests, dry runs)."""
    from .families import family_config
    base = dict(vocab_size=4096, hidden_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                intermediate_size=256, rms_norm_eps=1e-6, max_position_embeddings=4096, tie_word_embeddings=False, eos_token_id=1,
                pad_token_id=0, rope_parameters={"rope_type": "default", "rope_theta": 10000.0})
    extra = {
        "deepseek_v3": dict(model_type="deepseek_v3", num_key_value_heads=4, q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=32,
                            qk_rope_head_dim=16, v_head_dim=32, n_routed_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1,
                            first_k_dense_replace=1, moe_intermediate_size=64, n_shared_experts=1, routed_scaling_factor=2.5,
                            norm_topk_prob=True, rope_interleave=True),
        "gpt_oss": dict(model_type="gpt_oss", num_local_experts=4, num_experts_per_tok=2, intermediate_size=64, sliding_window=64,
                        attention_bias=True),
        "gemma3": dict(model_type="gemma3_text", sliding_window=64, query_pre_attn_scalar=32, tie_word_embeddings=True, num_hidden_layers=6,
                       rope_parameters={"full_attention": {"rope_type": "default", "rope_theta": 1000000.0},
                                        "sliding_attention": {"rope_type": "default", "rope_theta": 10000.0}}),
        "qwen3_next": dict(model_type="qwen3_next", partial_rotary_factor=0.25, linear_num_value_heads=4, linear_num_key_heads=2,
                           linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4, num_experts=4, num_experts_per_tok=2,
                           moe_intermediate_size=64, shared_expert_intermediate_size=64, decoder_sparse_step=1, norm_topk_prob=True),
        "glm4_moe": dict(model_type="glm4_moe", partial_rotary_factor=0.5, use_qk_norm=True, attention_bias=True, n_routed_experts=8,
                         num_experts_per_tok=2, n_group=1, topk_group=1, first_k_dense_replace=1, moe_intermediate_size=64, n_shared_experts=1,
                         routed_scaling_factor=1.0, norm_topk_prob=True),
    }[kind]
    return family_config({**base, **extra})


for _k in ("deepseek_v3", "gpt_oss", "gemma3", "qwen3_next", "glm4_moe"):
    PRESETS["tiny-" + _k.replace("_", "-")] = (lambda k=_k: _tiny_family(k))


def get_config(name_or_path: str) -> ModelConfig:
    key = name_or_path.lower()
    if key in PRESETS:
        return PRESETS[key]()
    return ModelConfig.from_pretrained(name_or_path)
