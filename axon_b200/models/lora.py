"""Low-rank adapters (LoRA) on the dense decoder.

The reference wraps the HF module with PEFT (``apply_lora_to_module``, axon/utils/hf_model.py:732-767;
config block ``lora:`` in axon/config/trainer/trainer.yaml:156-189) and trains only the adapters. Here
the base weights stay in the model's flat bf16 buffer, frozen, and the adapters live in a second,
small flat buffer that is the model's ``params`` - so the optimizer, its sharding, gradient clipping
and checkpoints see only the adapters, exactly like a PEFT run.

For a fused linear with sub-modules (q/k/v or gate/up) every HF sub-module keeps its own adapter pair,
stored side by side so that the low-rank path costs two GEMMs plus one small GEMM per sub-module:

    t  = x @ A_cat^T                       A_cat [n*r, in]   (the n sub-modules' A matrices stacked)
    y  = x @ W^T ; y[:, rows_i] += s * t[:, i*r:(i+1)*r] @ B[rows_i]^T        B [out, r]

with ``s = alpha / r``. Backward never forms a gradient of W (a third of the GEMM work of full
fine-tuning disappears):

    u[:, i] = dy[:, rows_i] @ B[rows_i]              dx = dy @ W + s * u @ A_cat
    dB[rows_i] += s * dy[:, rows_i]^T @ t[:, i]      dA_cat += s * u^T @ x

The sampler paths (``prefill`` / ``decode``) go through the same ``_lin`` and therefore sample from
exactly the adapted model - no merge / un-merge round trip through bf16. ``merged_weight`` gives
``W + s * B A`` per linear for exporting to an engine that cannot apply adapters.

Adapters load and save in the PEFT layout (``adapter_config.json`` + ``adapter_model.safetensors``
with ``base_model.model.<hf module>.lora_A.weight`` keys), so ``lora.adapter_path`` of the reference
works unchanged.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field

import torch

from ..ops import gemm as G
from .config import ModelConfig
from .dense import DenseModel, PackedBatch
from .params import FlatParams

# fused linear -> HF sub-modules it is made of, in row order
_SUBMODULES = {
    "self_attn.qkv_proj.weight": ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"),
    "self_attn.o_proj.weight": ("self_attn.o_proj",),
    "mlp.gate_up_proj.weight": ("mlp.gate_proj", "mlp.up_proj"),
    "mlp.down_proj.weight": ("mlp.down_proj",),
}


@dataclass
class LoRAConfig:
    rank: int = 8
    alpha: float = 16.0
    target_modules: object = "all-linear"          # "all-linear" or a list of HF module names (q_proj, up_proj, ...)
    exclude_modules: list = field(default_factory=list)
    adapter_path: str | None = None

    @classmethod
    def from_dict(cls, d) -> "LoRAConfig":
        get = (lambda k, dv: d.get(k, dv)) if hasattr(d, "get") else (lambda k, dv: getattr(d, k, dv))
        tm = get("target_modules", "all-linear")
        if not isinstance(tm, str):
            tm = list(tm)
            if tm == ["all-linear"]:
                tm = "all-linear"
        return cls(rank=int(get("rank", 8)), alpha=float(get("alpha", 16)), target_modules=tm,
                   exclude_modules=list(get("exclude_modules", None) or []), adapter_path=get("adapter_path", None))

    def targets(self, module: str) -> bool:
        leaf = module.rsplit(".", 1)[-1]
        if leaf in self.exclude_modules or module in self.exclude_modules:
            return False
        return self.target_modules == "all-linear" or leaf in self.target_modules or module in self.target_modules


def _rows(cfg: ModelConfig, fused: str) -> list[tuple[int, int]]:
    """Row range of every sub-module inside the fused weight."""
    if fused == "self_attn.qkv_proj.weight":
        q, kv = cfg.q_size, cfg.kv_size
        return [(0, q), (q, q + kv), (q + kv, q + 2 * kv)]
    if fused == "mlp.gate_up_proj.weight":
        return [(0, cfg.intermediate_size), (cfg.intermediate_size, 2 * cfg.intermediate_size)]
    if fused == "self_attn.o_proj.weight":
        return [(0, cfg.hidden_size)]
    return [(0, cfg.hidden_size)]


def _in_features(cfg: ModelConfig, fused: str) -> int:
    return {"self_attn.qkv_proj.weight": cfg.hidden_size, "self_attn.o_proj.weight": cfg.q_size,
            "mlp.gate_up_proj.weight": cfg.hidden_size, "mlp.down_proj.weight": cfg.intermediate_size}[fused]


def lora_layout(cfg: ModelConfig, lc: LoRAConfig) -> dict:
    """Adapter parameter layout: ``model.layers.L.<fused linear sans .weight>.lora_A`` [n*r, in] and
    ``.lora_B`` [out, r] for every fused linear with at least one targeted sub-module."""
    lay = {}
    for l in range(cfg.num_hidden_layers):
        for fused, subs in _SUBMODULES.items():
            if not any(lc.targets(m) for m in subs):
                continue
            base = f"model.layers.{l}.{fused[:-len('.weight')]}"
            lay[base + ".lora_A"] = (len(subs) * lc.rank, _in_features(cfg, fused))
            lay[base + ".lora_B"] = (_rows(cfg, fused)[-1][1], lc.rank)
    return lay


class LoRADenseModel(DenseModel):
    def __init__(self, cfg: ModelConfig, lora: LoRAConfig, device="cuda", dtype=torch.bfloat16, base: FlatParams | None = None):
        assert lora.rank > 0 and lora.rank % 8 == 0, "LoRA rank must be a positive multiple of 8 (16-byte rows for TMA)"
        super().__init__(cfg, device, dtype, params=base)
        self.base = self.params                     # frozen
        self.lora = lora
        self.scale = lora.alpha / lora.rank
        self.params = FlatParams(cfg, self.device, dtype, layout=lora_layout(cfg, lora))
        self._sinks: dict = {}
        self.init_adapters()
        if lora.adapter_path:
            self.load_adapter(lora.adapter_path)

    # ------------------------------------------------------------------ parameters
    @property
    def weights(self) -> FlatParams:
        return self.base

    def _wgrad(self, name: str):
        """Gradients of frozen tensors: small vectors (norm weights) go to a scratch sink that nobody
        reads, matrices are not computed at all."""
        w = self.base[name]
        if w.dim() > 1 or name.endswith(".bias"):
            return None
        key = tuple(w.shape)
        if key not in self._sinks:
            self._sinks[key] = torch.zeros(key, dtype=torch.float32, device=self.device)
        return self._sinks[key]

    def _embed_bwd(self, batch: PackedBatch, dx: torch.Tensor) -> None:
        return None

    def init_adapters(self, seed: int = 0) -> None:
        """A ~ U(-1/sqrt(in), 1/sqrt(in)) (PEFT's kaiming-uniform with a = sqrt(5)), B = 0; the A rows and
        B rows of sub-modules that are not targeted stay zero (and receive zero gradients)."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        for name, v in self.params.views.items():
            if name.endswith(".lora_A"):
                bound = 1.0 / math.sqrt(v.shape[1])
                v.copy_(((torch.rand(v.shape, generator=g) * 2 - 1) * bound).to(v.dtype))
            else:
                v.zero_()
        self._apply_target_mask(self.params.views)

    def _apply_target_mask(self, tensors: dict) -> None:
        r = self.lora.rank
        for l in range(self.cfg.num_hidden_layers):
            for fused, subs in _SUBMODULES.items():
                base = f"model.layers.{l}.{fused[:-len('.weight')]}"
                if base + ".lora_A" not in tensors:
                    continue
                for i, (m, (r0, r1)) in enumerate(zip(subs, _rows(self.cfg, fused))):
                    if not self.lora.targets(m):
                        tensors[base + ".lora_A"][i * r:(i + 1) * r].zero_()
                        tensors[base + ".lora_B"][r0:r1].zero_()

    def finalize_grads(self) -> None:
        """Called before the optimizer step: sub-modules outside ``target_modules`` keep zero adapters."""
        if self.params.grad_flat is not None and (self.lora.target_modules != "all-linear" or self.lora.exclude_modules):
            self._apply_target_mask(self.params.grads)

    def _ab(self, l: int, fused: str):
        base = f"model.layers.{l}.{fused[:-len('.weight')]}"
        if base + ".lora_A" not in self.params.layout:
            return None, None, base
        return self.params[base + ".lora_A"], self.params[base + ".lora_B"], base

    # ------------------------------------------------------------------ linear hooks
    def _lin(self, l: int, name: str, x: torch.Tensor) -> torch.Tensor:
        y = self._bias_fwd(l, name, G.gemm_nt(x, self._p(l, name)))
        A, B, _ = self._ab(l, name)
        if A is None:
            return y
        r = self.lora.rank
        t = G.gemm_nt(x, A)                                          # [T, n*r]
        for i, (r0, r1) in enumerate(_rows(self.cfg, name)):
            G.gemm_nt(t[:, i * r:(i + 1) * r], B[r0:r1], out=y[:, r0:r1], accumulate=True, alpha=self.scale)
        return y

    def _lin_bwd(self, l: int, name: str, dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        dx = G.gemm_nn(dy, self._p(l, name))
        A, B, base = self._ab(l, name)
        if A is None:
            return dx
        r, s = self.lora.rank, self.scale
        gA, gB = self.params.grads[base + ".lora_A"], self.params.grads[base + ".lora_B"]
        t = G.gemm_nt(x, A)                                          # recomputed: [T, n*r] is cheap
        u = torch.empty_like(t)
        for i, (r0, r1) in enumerate(_rows(self.cfg, name)):
            sl = slice(i * r, (i + 1) * r)
            G.gemm_nn(dy[:, r0:r1], B[r0:r1], out=u[:, sl])
            G.gemm_tn(dy[:, r0:r1], t[:, sl], out=gB[r0:r1], accumulate=True, alpha=s)
        G.gemm_tn(u, x, out=gA, accumulate=True, alpha=s)
        G.gemm_nn(u, A, out=dx, accumulate=True, alpha=s)
        return dx

    def head_grad(self):
        return None

    # ------------------------------------------------------------------ export
    @torch.no_grad()
    def merged_weight(self, l: int, fused: str) -> torch.Tensor:
        """``W + s * B A`` of one fused linear (fp32 accumulate, model dtype out)."""
        W = self._p(l, fused).float().clone()
        A, B, _ = self._ab(l, fused)
        if A is not None:
            r = self.lora.rank
            for i, (r0, r1) in enumerate(_rows(self.cfg, fused)):
                W[r0:r1] += self.scale * (B[r0:r1].float() @ A[i * r:(i + 1) * r].float())
        return W.to(self.dtype)

    def peft_state_dict(self) -> dict:
        """Adapters under PEFT's key names, one pair per HF sub-module."""
        out, r = {}, self.lora.rank
        for l in range(self.cfg.num_hidden_layers):
            for fused, subs in _SUBMODULES.items():
                A, B, _ = self._ab(l, fused)
                if A is None:
                    continue
                for i, (m, (r0, r1)) in enumerate(zip(subs, _rows(self.cfg, fused))):
                    if not self.lora.targets(m):
                        continue
                    k = f"base_model.model.model.layers.{l}.{m}"
                    out[k + ".lora_A.weight"] = A[i * r:(i + 1) * r].detach().clone().contiguous()
                    out[k + ".lora_B.weight"] = B[r0:r1].detach().clone().contiguous()
        return out

    def save_adapter(self, path: str) -> None:
        from safetensors.torch import save_file
        os.makedirs(path, exist_ok=True)
        save_file({k: v.cpu() for k, v in self.peft_state_dict().items()}, os.path.join(path, "adapter_model.safetensors"))
        mods = sorted({m.rsplit(".", 1)[-1] for subs in _SUBMODULES.values() for m in subs if self.lora.targets(m)})
        with open(os.path.join(path, "adapter_config.json"), "w") as f:
            json.dump({"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": self.lora.rank, "lora_alpha": self.lora.alpha,
                       "target_modules": mods, "bias": "none", "lora_dropout": 0.0, "fan_in_fan_out": False}, f, indent=1)

    def load_adapter(self, path: str) -> None:
        from safetensors.torch import load_file
        with open(os.path.join(path, "adapter_config.json")) as f:
            ac = json.load(f)
        assert int(ac["r"]) == self.lora.rank, f"adapter rank {ac['r']} != configured rank {self.lora.rank}"
        self.lora.alpha = float(ac.get("lora_alpha", self.lora.alpha))
        self.scale = self.lora.alpha / self.lora.rank
        sd = load_file(os.path.join(path, "adapter_model.safetensors"))
        r = self.lora.rank
        for l in range(self.cfg.num_hidden_layers):
            for fused, subs in _SUBMODULES.items():
                A, B, _ = self._ab(l, fused)
                if A is None:
                    continue
                for i, (m, (r0, r1)) in enumerate(zip(subs, _rows(self.cfg, fused))):
                    k = f"base_model.model.model.layers.{l}.{m}"
                    if k + ".lora_A.weight" in sd:
                        A[i * r:(i + 1) * r].copy_(sd[k + ".lora_A.weight"].to(A.dtype))
                        B[r0:r1].copy_(sd[k + ".lora_B.weight"].to(B.dtype))

    def flops_per_token(self, seqlen: int) -> float:
        """Forward + input-gradient GEMMs of the frozen base (4 x params) plus attention; the adapters' own
        work is below a percent at the usual ranks."""
        full = DenseModel.flops_per_token(self, seqlen)
        c = self.cfg
        dense = c.num_hidden_layers * (c.qkv_size * c.hidden_size + c.hidden_size * c.q_size
                                       + 3 * c.hidden_size * c.intermediate_size) + c.vocab_size * c.hidden_size
        return full - 2 * dense
