"""Multi-token-prediction module: loss value and every gradient (module, shared embedding / head, trunk)
against an autograd implementation; the engine reports the loss and scales it by mini-batch counts."""
import math

import pytest
import torch
import torch.nn.functional as F

from axon_b200.models.config import get_config
from axon_b200.models.dense import DenseModel, PackedBatch


def _reference(cfg, sd, seqs, g_lp, scale):
    P = {k: v.detach().double().requires_grad_(True) for k, v in sd.items()}
    D, Hq, Hkv, L0 = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.num_hidden_layers

    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w

    def rope(x, pos):
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
        ang = pos.double()[:, None] * inv[None]
        c, s = ang.cos()[:, None], ang.sin()[:, None]
        x1, x2 = x[..., : D // 2], x[..., D // 2:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)

    def layer(l, x):
        n, p = x.shape[0], f"model.layers.{l}."
        pos = torch.arange(n)
        qkv = (rms(x, P[p + "input_layernorm.weight"]) @ P[p + "self_attn.qkv_proj.weight"].t()).view(n, Hq + 2 * Hkv, D)
        q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hkv], qkv[:, Hq + Hkv:]
        q, k = rms(q, P[p + "self_attn.q_norm.weight"]), rms(k, P[p + "self_attn.k_norm.weight"])
        q, k = rope(q, pos), rope(k, pos)
        k, v = k.repeat_interleave(Hq // Hkv, 1), v.repeat_interleave(Hq // Hkv, 1)
        sc = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D)
        sc = sc.masked_fill(torch.ones(n, n, dtype=torch.bool).triu(1), float("-inf"))
        x = x + torch.einsum("hqk,khd->qhd", sc.softmax(-1), v).reshape(n, Hq * D) @ P[p + "self_attn.o_proj.weight"].t()
        g, u = (rms(x, P[p + "post_attention_layernorm.weight"]) @ P[p + "mlp.gate_up_proj.weight"].t()).chunk(2, -1)
        return x + (F.silu(g) * u) @ P[p + "mlp.down_proj.weight"].t()

    emb = P["model.embed_tokens.weight"]
    head = emb if cfg.tie_word_embeddings else P["lm_head.weight"]
    total, nll, off = 0.0, 0.0, 0
    for seq in seqs:
        n = seq.numel()
        x = emb[seq.long()]
        for l in range(L0):
            x = layer(l, x)
        lsm = (rms(x, P["model.norm.weight"]) @ head.t()).log_softmax(-1)
        lp = lsm[:-1].gather(1, seq[1:].long()[:, None])[:, 0]
        total = total + (lp * g_lp[off:off + n - 1].double()).sum()
        if n > 2:        # position t sees h_t and token t+1, predicts token t+2
            p = f"model.layers.{L0}."
            z = torch.cat([rms(emb[seq[1:-1].long()], P[p + "enorm.weight"]), rms(x[:-2], P[p + "hnorm.weight"])], -1) @ P[p + "eh_proj.weight"].t()
            # the module's layer runs over whole packed sequences (positions 0 .. n-1); the last two
            # positions have no target and, being last, influence no earlier one
            h2 = layer(L0, z)
            lsm2 = (rms(h2, P[p + "shared_head.norm.weight"]) @ head.t()).log_softmax(-1)
            nll = nll - lsm2.gather(1, seq[2:].long()[:, None]).sum()
        off += n
    (total + scale * nll).backward()
    return float(nll.detach()), {k: v.grad for k, v in P.items()}


def test_mtp_loss_and_gradients_match_autograd():
    cfg = get_config("tiny-qwen3-mtp")
    torch.manual_seed(0)
    model = DenseModel(cfg, device="cpu", dtype=torch.float32)
    model.params.init_random(std=0.05, seed=1)
    for v in model.params.views.values():
        if v.dim() == 1:
            v.copy_(1 + 0.1 * torch.randn(v.shape))
    seqs = [torch.randint(0, cfg.vocab_size, (n,)) for n in (17, 2, 5, 33)]
    batch = PackedBatch.from_sequences(seqs, "cpu")
    g_lp = torch.randn(batch.input_ids.numel()) * (batch.labels >= 0)
    model.mtp_scale = 0.3
    model.params.alloc_grads()
    model.params.zero_grads()
    model.forward(batch, 1.0, save_for_backward=True)
    nll, count = model.mtp_last
    model.backward(g_lp, None)
    sd = {k: v.detach().clone() for k, v in model.params.views.items()}
    nll_ref, grads = _reference(cfg, sd, seqs, g_lp, 0.3)
    assert int(count) == sum(max(0, s.numel() - 2) for s in seqs)
    assert abs(float(nll) - nll_ref) < 1e-3 * abs(nll_ref)
    for name, g in model.params.grads.items():
        ref = grads[name]
        err = (g.double() - ref).abs().max().item()
        assert err < 1e-3 * max(1.0, ref.abs().max().item()), (name, err)


def test_mtp_idle_without_scale():
    cfg = get_config("tiny-qwen3-mtp")
    model = DenseModel(cfg, device="cpu", dtype=torch.float32)
    model.params.init_random(std=0.05, seed=1)
    batch = PackedBatch.from_sequences([torch.randint(0, cfg.vocab_size, (9,))], "cpu")
    model.params.alloc_grads()
    model.params.zero_grads()
    lp, _ = model.forward(batch, 1.0, save_for_backward=True)
    model.backward(torch.ones_like(lp), None)
    assert model.mtp_last is None
    assert float(model.params.grads[f"model.layers.{cfg.num_hidden_layers}.eh_proj.weight"].abs().max()) == 0.0


def test_engine_adds_the_mtp_loss_and_reports_it():
    """The module's weights move only when the factor is set; the loss is reported per micro-batch and its
    gradient does not depend on how the mini-batch is cut into micro-batches."""
    from axon_b200.protocol import DataProto
    from axon_b200.trainer.policy import OptimConfig, PolicyEngine
    cfg = get_config("tiny-qwen3-mtp")
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab_size, (4, 24), generator=g)
    att = torch.ones(4, 24, dtype=torch.long)
    att[1, 15:] = 0
    rm = att.clone().float()
    rm[:, :5] = 0

    def run(cap, coef):
        model = DenseModel(cfg, device="cpu", dtype=torch.float32)
        model.params.init_random(std=0.05, seed=1)
        eng = PolicyEngine(model, OptimConfig(lr=1e-3), max_token_len_per_gpu=cap)
        eng.mtp_loss_coef = coef
        d = DataProto.from_dict({"input_ids": ids, "attention_mask": att, "position_ids": (att.cumsum(1) - 1) * att,
                                 "response_mask": rm, "advantages": torch.randn(4, 24, generator=torch.Generator().manual_seed(5)) * rm,
                                 "old_log_probs": torch.zeros(4, 24)})
        d.meta_info["temperature"] = 1.0
        from axon_b200.driver.driver_utils import process_mini_batch
        process_mini_batch(d)
        m = eng.forward_backward(d, "ppo", {"clip_ratio": 0.2})
        return m, model.params.grad_flat.clone(), model.params.grads[f"model.layers.{cfg.num_hidden_layers}.eh_proj.weight"].clone()

    m0, _, g_mod0 = run(512, 0.0)
    assert "mtp_loss" not in m0 and float(g_mod0.abs().max()) == 0.0
    m1, flat1, g_mod1 = run(512, 0.3)
    assert len(m1["mtp_loss"]) == 1 and m1["mtp_loss"][0] > 1.0 and float(g_mod1.abs().max()) > 0.0
    m4, flat4, _ = run(24, 0.3)                     # one row per micro-batch
    assert len(m4["mtp_loss"]) == 4
    torch.testing.assert_close(flat4, flat1, rtol=1e-3, atol=1e-6)


def test_mtp_weights_round_trip_through_hf_names(tmp_path):
    from axon_b200.models.config import ModelConfig
    from axon_b200.utils.hf_model import load_hf_weights, save_hf_model
    cfg = get_config("tiny-qwen3-mtp")
    m = DenseModel(cfg, device="cpu", dtype=torch.float32)
    m.params.init_random(std=0.05, seed=2)
    sd = m.params.to_hf_state_dict()
    p = f"model.layers.{cfg.num_hidden_layers}."
    assert tuple(sd[p + "eh_proj.weight"].shape) == (cfg.hidden_size, 2 * cfg.hidden_size)
    assert p + "self_attn.q_proj.weight" in sd and p + "shared_head.norm.weight" in sd
    save_hf_model(m, str(tmp_path / "hf"), cfg=cfg)
    cfg2 = ModelConfig.from_pretrained(str(tmp_path / "hf"))
    assert cfg2.num_nextn_predict_layers == 1
    m2 = DenseModel(cfg2, device="cpu", dtype=torch.float32)
    load_hf_weights(m2, str(tmp_path / "hf"))
    torch.testing.assert_close(m2.params.flat, m.params.flat, rtol=0, atol=4e-3)


def test_sparse_model_replays_the_decoder_layers_and_routes_the_module_itself():
    """A routing record from the sampler covers the decoder layers only; the prediction module behind them is a sparse
    layer too and picks its own experts while the decoder layers replay theirs."""
    from axon_b200.models.moe import MoEModel
    cfg = get_config("tiny-moe-mtp")
    model = MoEModel(cfg, device="cpu", dtype=torch.float32)
    model.params.init_random(std=0.05, seed=1)
    batch = PackedBatch.from_sequences([torch.randint(0, cfg.vocab_size, (n,)) for n in (19, 6)], "cpu")
    T = batch.input_ids.numel()
    g = torch.Generator().manual_seed(2)
    rm = torch.stack([torch.stack([torch.randperm(cfg.num_experts, generator=g)[:cfg.num_experts_per_tok] for _ in range(cfg.num_hidden_layers)])
                      for _ in range(T)])                                   # [T, decoder layers, top-k]
    batch.routermap = rm
    model.mtp_scale = 0.3
    model.capture_routing, model.last_routing = True, None
    model.params.alloc_grads()
    model.params.zero_grads()
    lp, _ = model.forward(batch, 1.0, save_for_backward=True)
    routed = model.last_routing
    assert len(routed) == cfg.num_hidden_layers + 1
    for l in range(cfg.num_hidden_layers):
        assert torch.equal(routed[l].sort(1).values.long(), rm[:, l].sort(1).values)
    model.backward(torch.ones_like(lp), None)
    L = cfg.num_hidden_layers
    assert float(model.params.grads[f"model.layers.{L}.mlp.experts.w13_weight"].abs().max()) > 0
    assert float(model.params.grads[f"model.layers.{L}.mlp.gate.weight"].abs().max()) > 0


@pytest.mark.timeout(900)
@pytest.mark.parametrize("kind", ["ulysses", "context", "param-shards", "tensor-context"])
def test_module_on_ranks_that_hold_a_slice_of_the_tokens_matches_single_process(monkeypatch, kind):
    """Sequence-parallel (Ulysses) and context-parallel (zigzag) ranks hold a slice of every sequence: the next tokens and
    the second-next labels are shifted within whole sequences before the cut, the module's attention is the group's, its
    targets are counted once; reported loss, gradient norm and update equal the single-process trainer. Parameter-sharding
    ranks are the opposite case: data-parallel peers outside the optimizer's group, whose targets have to be added."""
    import numpy as np
    from test_megatron_trainer import _cfg, _run
    monkeypatch.setenv("AXON_ENABLE_MTP", "1")
    name = "tiny-qwen3-mtp"
    ref_cfg = _cfg(1, name)
    if kind == "ulysses":
        got_cfg, cls = _cfg(1, name), "axon_b200.trainer.fsdp_trainer.TrainerWorker"
        got_cfg["fsdp"] = {"ulysses_sequence_parallel_size": 2}
    elif kind == "tensor-context":          # world = 4: two context-parallel members, each a tensor-parallel pair
        got_cfg, cls = _cfg(2, name, cp=2), "axon_b200.trainer.megatron_trainer.TrainerWorker"
    elif kind == "param-shards":
        got_cfg, cls = _cfg(1, name), "axon_b200.trainer.fsdp_trainer.TrainerWorker"
        got_cfg["fsdp"] = {"param_sharding": True}
    else:
        got_cfg, cls = _cfg(1, name, cp=2), "axon_b200.trainer.megatron_trainer.TrainerWorker"
    ref_cfg["mtp_loss_scaling_factor"] = got_cfg["mtp_loss_scaling_factor"] = 0.3
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", ref_cfg, 1)
    got = _run(cls, got_cfg, 4 if kind == "tensor-context" else 2)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    # data-parallel ranks report the mean over their own micro-batches: close to, not equal to, the single process's
    tol = 5e-3 if kind == "param-shards" else 1e-3
    assert "actor/mtp_loss" in got[1] and abs(np.mean(got[1]["actor/mtp_loss"]) - np.mean(ref[1]["actor/mtp_loss"])) < tol
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
