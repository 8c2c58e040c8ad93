"""Explicit forward/backward of the dense decoder vs an independent autograd implementation."""
import math

import pytest
import torch
import torch.nn.functional as F

from axon_b200.models.config import ModelConfig, tiny_gpu, tiny_qwen3
from axon_b200.models.dense import DenseModel, PackedBatch


def autograd_reference(cfg: ModelConfig, sd: dict, seqs, temperature, g_lp, g_ent):
    """Plain PyTorch fp32 implementation with autograd; returns (lp, ent, grads by fused name)."""
    P = {k: v.detach().double().requires_grad_(True) for k, v in sd.items()}
    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads

    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w

    def rope(x, pos):  # [L,h,D]
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
        ang = pos.double()[:, None] * inv[None]
        c, s = ang.cos()[:, None], ang.sin()[:, None]
        x1, x2 = x[..., : D // 2], x[..., D // 2:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)

    lps, ents = [], []
    for seq in seqs:
        L = seq.numel()
        pos = torch.arange(L)
        x = P["model.embed_tokens.weight"][seq.long()]
        for l in range(cfg.num_hidden_layers):
            p = f"model.layers.{l}."
            h = rms(x, P[p + "input_layernorm.weight"])
            qkv = h @ P[p + "self_attn.qkv_proj.weight"].t()
            if cfg.attention_bias:
                qkv = qkv + P[p + "self_attn.qkv_proj.bias"]
            qkv = qkv.view(L, Hq + 2 * Hkv, D)
            q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hkv], qkv[:, Hq + Hkv:]
            if cfg.qk_norm:
                q = rms(q, P[p + "self_attn.q_norm.weight"])
                k = rms(k, P[p + "self_attn.k_norm.weight"])
            q, k = rope(q, pos), rope(k, pos)
            rep = Hq // Hkv
            k = k.repeat_interleave(rep, 1)
            v = v.repeat_interleave(rep, 1)
            sc = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D)
            sc = sc.masked_fill(torch.ones(L, L, dtype=torch.bool).triu(1), float("-inf"))
            o = torch.einsum("hqk,khd->qhd", sc.softmax(-1), v).reshape(L, Hq * D)
            x = x + o @ P[p + "self_attn.o_proj.weight"].t()
            h2 = rms(x, P[p + "post_attention_layernorm.weight"])
            gu = h2 @ P[p + "mlp.gate_up_proj.weight"].t()
            g, u = gu.chunk(2, -1)
            x = x + (F.silu(g) * u) @ P[p + "mlp.down_proj.weight"].t()
        hf = rms(x, P["model.norm.weight"])
        W = P["model.embed_tokens.weight"] if cfg.tie_word_embeddings else P["lm_head.weight"]
        z = hf @ W.t() / temperature
        lsm = z.log_softmax(-1)
        lp = torch.cat([lsm[:-1].gather(1, seq[1:].long()[:, None])[:, 0], torch.zeros(1, dtype=torch.float64)])
        ent = -(lsm.exp() * lsm).sum(-1)
        lps.append(lp)
        ents.append(ent)
    lp, ent = torch.cat(lps), torch.cat(ents)
    (lp * g_lp.double()).sum().add((ent * g_ent.double()).sum()).backward()
    return lp.detach(), ent.detach(), {k: v.grad for k, v in P.items()}


def _run(cfg, device, dtype, seqs, temperature=0.9):
    torch.manual_seed(0)
    model = DenseModel(cfg, device=device, dtype=dtype)
    model.params.init_random(std=0.05, seed=1)
    for n, v in model.params.views.items():  # non-trivial norm weights
        if v.dim() == 1:
            v.copy_((1 + 0.1 * torch.randn(v.shape)).to(dtype))
    batch = PackedBatch.from_sequences(seqs, device)
    T = batch.input_ids.numel()
    g_lp, g_ent = torch.randn(T), 0.1 * torch.randn(T)
    lp, ent = model.forward(batch, temperature, save_for_backward=True)
    model.params.alloc_grads()
    model.params.zero_grads()
    model.backward(g_lp.to(device), g_ent.to(device))
    sd = {k: v.detach().float().cpu() for k, v in model.params.views.items()}
    lp_r, ent_r, grads_r = autograd_reference(cfg, sd, seqs, temperature, g_lp, g_ent)
    return model, lp.cpu(), ent.cpu(), lp_r, ent_r, grads_r


@pytest.mark.parametrize("preset", ["tiny-qwen3", "tiny-qwen2"])
def test_dense_model_cpu_matches_autograd(preset):
    from axon_b200.models.config import get_config
    cfg = get_config(preset)
    seqs = [torch.randint(0, cfg.vocab_size, (n,)) for n in (17, 5, 33)]
    model, lp, ent, lp_r, ent_r, grads_r = _run(cfg, "cpu", torch.float32, seqs)
    assert torch.allclose(lp.double(), lp_r, atol=1e-4), (lp.double() - lp_r).abs().max()
    assert torch.allclose(ent.double(), ent_r, atol=1e-4)
    for name, g in model.params.grads.items():
        ref = grads_r[name]
        err = (g.double() - ref).abs().max().item()
        assert err < 1e-3 * max(1.0, ref.abs().max().item()), (name, err)


@pytest.mark.gpu
def test_dense_model_gpu_matches_autograd():
    cfg = tiny_gpu()
    seqs = [torch.randint(0, cfg.vocab_size, (n,)) for n in (150, 260, 31)]
    model, lp, ent, lp_r, ent_r, grads_r = _run(cfg, "cuda", torch.bfloat16, seqs)
    from axon_b200.ops import _common as C
    C.check_status()
    assert (lp.double() - lp_r).abs().max() < 0.15, (lp.double() - lp_r).abs().max()
    assert (lp.double() - lp_r).abs().mean() < 0.02
    assert (ent.double() - ent_r).abs().max() < 0.1
    for name, g in model.params.grads.items():
        ref = grads_r[name]
        g = g.double().cpu()
        rel = (g - ref).norm() / (ref.norm() + 1e-12)
        assert rel < 0.08, (name, rel.item())


def test_qwen2_family_bias_round_trips_through_hf_names(tmp_path):
    """Qwen2-style checkpoints: q/k/v biases fuse into one vector and split back under their HF names."""
    from axon_b200.models.config import ModelConfig, get_config
    from axon_b200.utils.hf_model import load_hf_weights, save_hf_model
    cfg = get_config("tiny-qwen2")
    assert cfg.attention_bias and not cfg.qk_norm
    m = DenseModel(cfg, device="cpu", dtype=torch.float32)
    m.params.init_random(std=0.05, seed=2)
    sd = m.params.to_hf_state_dict()
    b = "model.layers.0.self_attn."
    assert tuple(sd[b + "k_proj.bias"].shape) == (cfg.kv_size,) and b + "qkv_proj.bias" not in sd
    save_hf_model(m, str(tmp_path / "hf"), cfg=cfg)
    cfg2 = ModelConfig.from_pretrained(str(tmp_path / "hf"))
    assert cfg2.attention_bias and cfg2.model_type == "qwen2"
    m2 = DenseModel(cfg2, device="cpu", dtype=torch.float32)
    load_hf_weights(m2, str(tmp_path / "hf"))
    torch.testing.assert_close(m2.params.flat, m.params.flat, rtol=0, atol=4e-3)      # bf16 on disk
    # a config.json without the flag (as Qwen2 ships it) still turns the biases on
    assert ModelConfig.from_hf_dict({"model_type": "qwen2", "hidden_size": 256, "num_attention_heads": 4}).attention_bias
