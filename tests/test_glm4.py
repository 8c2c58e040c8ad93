"""GLM-4 dense family: partial interleaved rotary embeddings, sandwich norms and q/k/v biases against the
HF implementation (random tiny model), explicit backward against autograd, and the checkpoint round trip."""
import pytest
import torch

from axon_b200.models.config import ModelConfig, get_config
from axon_b200.models.dense import DenseModel, PackedBatch


def _hf_model(tmp_path):
    tr = pytest.importorskip("transformers")
    if not hasattr(tr, "Glm4ForCausalLM"):
        pytest.skip("transformers without Glm4")
    c = get_config("tiny-glm4")
    hf_cfg = tr.Glm4Config(vocab_size=c.vocab_size, hidden_size=c.hidden_size, intermediate_size=c.intermediate_size,
                           num_hidden_layers=c.num_hidden_layers, num_attention_heads=c.num_attention_heads,
                           num_key_value_heads=c.num_key_value_heads, head_dim=c.head_dim, partial_rotary_factor=0.5,
                           attention_bias=True, rms_norm_eps=c.rms_norm_eps, rope_theta=c.rope_theta,
                           max_position_embeddings=c.max_position_embeddings, tie_word_embeddings=False,
                           pad_token_id=0, eos_token_id=1)
    torch.manual_seed(0)
    m = tr.Glm4ForCausalLM(hf_cfg).float().eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() == 1:
                p.copy_(1 + 0.1 * torch.randn_like(p) if "norm" in n else 0.1 * torch.randn_like(p))
    d = str(tmp_path / "hf")
    m.save_pretrained(d, safe_serialization=True)
    return m, d


def test_matches_hf_glm4_and_round_trips(tmp_path):
    from axon_b200.utils.hf_model import load_hf_weights, save_hf_model
    hf, d = _hf_model(tmp_path)
    cfg = ModelConfig.from_pretrained(d)
    assert cfg.model_type == "glm4" and cfg.sandwich_norm and cfg.rope_interleaved and cfg.rotary_dim == cfg.head_dim // 2 and cfg.attention_bias
    ours = DenseModel(cfg, device="cpu", dtype=torch.float32)
    load_hf_weights(ours, d)
    seqs = [torch.randint(2, cfg.vocab_size, (n,)) for n in (19, 7)]
    lp, _ = ours.forward(PackedBatch.from_sequences(seqs, "cpu"), 1.0)
    off = 0
    for s in seqs:
        with torch.no_grad():
            logits = hf(s[None].long()).logits[0]
        ref = logits.log_softmax(-1)[:-1].gather(1, s[1:].long()[:, None])[:, 0]
        torch.testing.assert_close(lp[off:off + s.numel() - 1], ref, rtol=2e-4, atol=2e-4)
        off += s.numel()
    # export goes back to the checkpoint's layout: the HF model loads it and agrees
    save_hf_model(ours, str(tmp_path / "out"), cfg=cfg)
    import transformers as tr
    again = tr.Glm4ForCausalLM.from_pretrained(str(tmp_path / "out")).float().eval()
    with torch.no_grad():
        torch.testing.assert_close(again(seqs[0][None].long()).logits, hf(seqs[0][None].long()).logits, rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("recompute", ["full", "selective", "none"])
def test_backward_matches_hf_autograd(tmp_path, recompute):
    from axon_b200.models.params import _permute_heads, rope_row_perm
    from axon_b200.utils.hf_model import load_hf_weights
    hf, d = _hf_model(tmp_path)
    cfg = ModelConfig.from_pretrained(d)
    m = DenseModel(cfg, device="cpu", dtype=torch.float32)
    load_hf_weights(m, d)
    m.recompute = recompute
    seqs = [torch.randint(2, cfg.vocab_size, (n,)) for n in (13, 6)]
    batch = PackedBatch.from_sequences(seqs, "cpu")
    g = torch.randn(batch.input_ids.numel()) * (batch.labels >= 0)
    m.params.alloc_grads()
    m.params.zero_grads()
    m.forward(batch, 1.0, save_for_backward=True)
    m.backward(g, None)
    off, loss = 0, 0.0
    for s in seqs:
        lsm = hf(s[None].long()).logits[0].log_softmax(-1)
        loss = loss + (lsm[:-1].gather(1, s[1:].long()[:, None])[:, 0] * g[off:off + s.numel() - 1]).sum()
        off += s.numel()
    hf.zero_grad()
    loss.backward()
    ref = {n: p.grad for n, p in hf.named_parameters()}
    inv = torch.argsort(rope_row_perm(cfg))
    checked = 0
    for name, gr in m.params.grads.items():
        if name.endswith("qkv_proj.weight") or name.endswith("qkv_proj.bias"):
            kind = name.rsplit(".", 1)[1]
            base = name[: -len("qkv_proj." + kind)]
            q, k, v = gr.split([cfg.q_size, cfg.kv_size, cfg.kv_size], 0)
            pairs = [(_permute_heads(q, inv, cfg.head_dim), ref[base + "q_proj." + kind]),
                     (_permute_heads(k, inv, cfg.head_dim), ref[base + "k_proj." + kind]), (v, ref[base + "v_proj." + kind])]
        else:
            pairs = [(gr, ref[name])]
        for a, b in pairs:
            err = (a.double() - b.double()).abs().max().item()
            assert err < 2e-3 * max(1.0, b.abs().max().item()), (name, err)
            checked += 1
    assert checked > 20


@pytest.mark.gpu
def test_gpu_kernels_match_the_cpu_model():
    """Same GLM-4-style model (head dim 128) in bf16 on the native kernels and in fp32 on CPU."""
    from axon_b200.models.config import tiny_gpu
    from axon_b200.ops import _common as C
    cfg = tiny_gpu()
    cfg.model_type, cfg.qk_norm, cfg.attention_bias = "glm4", False, True
    cfg.partial_rotary_factor, cfg.rope_interleaved, cfg.sandwich_norm = 0.5, True, True
    ref = DenseModel(cfg, device="cpu", dtype=torch.float32)
    ref.params.init_random(std=0.05, seed=1)
    for v in ref.params.views.values():
        if v.dim() == 1:
            v.copy_(1 + 0.1 * torch.randn(v.shape))
    gpu = DenseModel(cfg, device="cuda", dtype=torch.bfloat16)
    gpu.params.flat.copy_(ref.params.flat.to(torch.bfloat16))
    ref.params.flat.copy_(gpu.params.flat.float().cpu())            # both start from the bf16-rounded values
    seqs = [torch.randint(0, cfg.vocab_size, (n,)) for n in (150, 260, 31)]
    g = torch.randn(sum(s.numel() for s in seqs))
    out = {}
    for name, m, dev in (("ref", ref, "cpu"), ("gpu", gpu, "cuda")):
        b = PackedBatch.from_sequences(seqs, dev)
        m.params.alloc_grads()
        m.params.zero_grads()
        lp, ent = m.forward(b, 1.0, save_for_backward=True)
        m.backward((g * (b.labels.cpu() >= 0)).to(dev), None)
        out[name] = (lp.float().cpu(), {k: v.float().cpu() for k, v in m.params.grads.items()})
    C.check_status()
    assert (out["gpu"][0] - out["ref"][0]).abs().max() < 0.15 and (out["gpu"][0] - out["ref"][0]).abs().mean() < 0.02
    for name, gr in out["ref"][1].items():
        rel = (out["gpu"][1][name] - gr).norm() / (gr.norm() + 1e-12)
        assert rel < 0.08, (name, float(rel))
