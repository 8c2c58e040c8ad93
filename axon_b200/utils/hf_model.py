"""Model construction and HuggingFace-format weight IO.

``build_model`` resolves a preset name or a HuggingFace directory (``config.json`` plus
``*.safetensors`` shards, optionally indexed by ``model.safetensors.index.json``) into a
``DenseModel`` whose parameters live in one flat buffer; weights stream shard by shard straight into
that buffer. ``save_hf_model`` writes the same layout back (bf16 safetensors shards, index,
``config.json``) so any HF-compatible consumer can load the result
(reference: axon/utils/hf_model.py:400-455,566-775 for name normalisation and factories).
"""
from __future__ import annotations

import json
import os
import re
from collections import OrderedDict

import torch

from ..models.config import ModelConfig, get_config

_SHARD_BYTES = 5 * (1 << 30)
_PREFIXES = ("base_model.model.", "_fsdp_wrapped_module.", "module.", "_orig_mod.")


def normalize_param_name(name: str) -> str:
    """Strip wrapper prefixes (FSDP / DDP / compile / PEFT) and LoRA's ``base_layer`` infix."""
    changed = True
    while changed:
        changed = False
        for p in _PREFIXES:
            if name.startswith(p):
                name, changed = name[len(p):], True
    return name.replace("._fsdp_wrapped_module", "").replace(".base_layer", "").replace("._checkpoint_wrapped_module", "")


def has_hf_weights(path: str) -> bool:
    return os.path.isdir(path) and any(f.endswith(".safetensors") or f == "pytorch_model.bin" for f in os.listdir(path))


def iter_hf_weights(path: str):
    """Yields ``(name, tensor)`` from every weight file of an HF directory (CPU tensors)."""
    files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
    if files:
        from safetensors import safe_open
        for fn in files:
            with safe_open(os.path.join(path, fn), framework="pt", device="cpu") as f:
                for k in f.keys():
                    yield normalize_param_name(k), f.get_tensor(k)
        return
    bin_path = os.path.join(path, "pytorch_model.bin")
    if os.path.exists(bin_path):
        for k, v in torch.load(bin_path, map_location="cpu", weights_only=True).items():
            yield normalize_param_name(k), v
        return
    raise FileNotFoundError(f"no *.safetensors or pytorch_model.bin under {path}")


def load_hf_weights(model, path: str, strict: bool = True) -> list[str]:
    """Stream an HF checkpoint into the model's flat parameter buffer. Returns missing names."""
    return model.params.load_hf_state_dict(OrderedDict(iter_hf_weights(path)), strict=strict)


def build_model(model_path: str, device="cuda", dtype=torch.bfloat16, seed: int = 0, load_weights: bool = True,
                model_cls=None):
    """Preset name -> random init (seeded); HF directory -> its config, and its weights when present."""
    from ..models.moe import build_model_for
    cfg = get_config(model_path)
    model = model_cls(cfg, device=device, dtype=dtype) if model_cls is not None else build_model_for(cfg, device, dtype)
    if load_weights and os.path.isdir(str(model_path)) and has_hf_weights(model_path):
        load_hf_weights(model, model_path)
    else:
        model.params.init_random(seed=seed)
    return model


def save_hf_model(model_or_params, path: str, cfg: ModelConfig | None = None, tokenizer=None,
                  state_dict: "OrderedDict[str, torch.Tensor] | None" = None) -> None:
    """bf16 safetensors shards (<= 5 GiB each) + index + config.json (+ tokenizer files)."""
    from safetensors.torch import save_file
    params = getattr(model_or_params, "params", model_or_params)
    cfg = cfg or params.cfg
    os.makedirs(path, exist_ok=True)
    sd = state_dict if state_dict is not None else params.to_hf_state_dict()
    shards: list[OrderedDict] = [OrderedDict()]
    size = 0
    for k, v in sd.items():
        nbytes = v.numel() * v.element_size()
        if size + nbytes > _SHARD_BYTES and shards[-1]:
            shards.append(OrderedDict())
            size = 0
        shards[-1][k] = v.detach().to("cpu").contiguous()
        size += nbytes
    weight_map, total = {}, 0
    n = len(shards)
    for i, shard in enumerate(shards):
        fn = "model.safetensors" if n == 1 else f"model-{i + 1:05d}-of-{n:05d}.safetensors"
        save_file(shard, os.path.join(path, fn), metadata={"format": "pt"})
        for k, v in shard.items():
            weight_map[k] = fn
            total += v.numel() * v.element_size()
    if n > 1:
        with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
    cfg.save_pretrained(path)
    if tokenizer is not None and hasattr(tokenizer, "save_pretrained"):
        tokenizer.save_pretrained(path)


def layer_index(name: str) -> int | None:
    m = re.search(r"\blayers\.(\d+)\.", name)
    return int(m.group(1)) if m else None
