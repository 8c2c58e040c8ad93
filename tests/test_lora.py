"""LoRA adapters on the dense model: forward equals the merged-weight model, adapter gradients equal the
chain rule through the merged weights' gradients, only adapters train, PEFT-layout save / load round trip."""
import torch

from axon_b200.models.config import tiny_qwen3
from axon_b200.models.dense import DenseModel, PackedBatch
from axon_b200.models.lora import LoRAConfig, LoRADenseModel, _SUBMODULES, _rows


def _models(target="all-linear", exclude=()):
    cfg = tiny_qwen3()
    torch.manual_seed(0)
    lm = LoRADenseModel(cfg, LoRAConfig(rank=8, alpha=16, target_modules=target, exclude_modules=list(exclude)), device="cpu", dtype=torch.float32)
    lm.base.init_random(std=0.05, seed=1)
    g = torch.Generator().manual_seed(2)
    for n, v in lm.params.views.items():
        if n.endswith("lora_B"):
            v.copy_(torch.randn(v.shape, generator=g) * 0.05)
    lm._apply_target_mask(lm.params.views)
    full = DenseModel(cfg, device="cpu", dtype=torch.float32)
    full.params.flat.copy_(lm.base.flat)
    for l in range(cfg.num_hidden_layers):
        for fused in _SUBMODULES:
            full.params[f"model.layers.{l}.{fused}"].copy_(lm.merged_weight(l, fused))
    return cfg, lm, full


def _batch(cfg):
    g = torch.Generator().manual_seed(3)
    return PackedBatch.from_sequences([torch.randint(0, cfg.vocab_size, (n,), generator=g, dtype=torch.int32) for n in (37, 20)], "cpu")


def test_forward_and_gradients_match_merged_weights():
    cfg, lm, full = _models()
    b = _batch(cfg)
    lp1, e1 = lm.forward(b, 1.0, save_for_backward=True)
    lp2, e2 = full.forward(b, 1.0, save_for_backward=True)
    torch.testing.assert_close(lp1, lp2, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(e1, e2, rtol=1e-4, atol=1e-5)
    g = torch.randn(lp1.shape, generator=torch.Generator().manual_seed(4))
    lm.params.alloc_grads()
    lm.backward(g, 0.1 * g)
    full.backward(g, 0.1 * g)
    r, s = 8, lm.scale
    for l in range(cfg.num_hidden_layers):
        for fused in _SUBMODULES:
            A, B, base = lm._ab(l, fused)
            G = full.params.grads[f"model.layers.{l}.{fused}"]
            for i, (r0, r1) in enumerate(_rows(cfg, fused)):
                torch.testing.assert_close(lm.params.grads[base + ".lora_A"][i * r:(i + 1) * r], s * B[r0:r1].t() @ G[r0:r1], rtol=2e-3, atol=2e-5)
                torch.testing.assert_close(lm.params.grads[base + ".lora_B"][r0:r1], s * G[r0:r1] @ A[i * r:(i + 1) * r].t(), rtol=2e-3, atol=2e-5)
    assert lm.base.grad_flat is None                     # the frozen base never allocates gradients
    assert lm.params.numel < 0.2 * lm.base.numel


def test_target_modules_subset_and_policy_engine_step():
    from axon_b200.protocol import DataProto
    from axon_b200.trainer.policy import OptimConfig, PolicyEngine
    cfg, lm, _ = _models(target=["q_proj", "v_proj", "down_proj"])
    assert not any("o_proj" in n or "gate_up" in n for n in lm.params.layout)
    base_before = lm.base.flat.clone()
    k_rows = slice(cfg.q_size, cfg.q_size + cfg.kv_size)
    assert float(lm.params["model.layers.0.self_attn.qkv_proj.lora_B"][k_rows].abs().sum()) == 0.0
    eng = PolicyEngine(lm, OptimConfig(lr=1e-2, weight_decay=0.0), max_token_len_per_gpu=256)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, cfg.vocab_size, (4, 24), generator=g)
    att = torch.ones(4, 24, dtype=torch.long)
    rm = att.clone().float(); rm[:, :6] = 0
    d = DataProto.from_dict({"input_ids": ids, "attention_mask": att, "position_ids": att.cumsum(1) - 1, "response_mask": rm,
                             "advantages": torch.randn(4, 24, generator=g) * rm})
    d.meta_info["temperature"] = 1.0
    before = eng.forward(d).batch["log_probs"].clone()
    d.batch["old_log_probs"] = before
    eng.forward_backward(d, "ppo", {"clip_ratio": 0.2})
    m = eng.optim_step()
    assert m["grad_norm"] > 0
    after = eng.forward(d).batch["log_probs"]
    assert (after - before).abs().max() > 1e-5                       # the adapters moved the policy
    assert torch.equal(lm.base.flat, base_before)                    # the base did not move
    assert float(lm.params["model.layers.0.self_attn.qkv_proj.lora_B"][k_rows].abs().sum()) == 0.0   # k_proj is not a target
    assert float(lm.params["model.layers.0.self_attn.qkv_proj.lora_A"][8:16].abs().sum()) == 0.0


def test_peft_layout_round_trip(tmp_path):
    cfg, lm, _ = _models()
    lm.save_adapter(str(tmp_path / "ad"))
    sd = lm.peft_state_dict()
    assert "base_model.model.model.layers.0.self_attn.k_proj.lora_A.weight" in sd
    assert tuple(sd["base_model.model.model.layers.1.mlp.up_proj.lora_B.weight"].shape) == (cfg.intermediate_size, 8)
    other = LoRADenseModel(cfg, LoRAConfig(rank=8, alpha=4, adapter_path=str(tmp_path / "ad")), device="cpu", dtype=torch.float32)
    assert other.scale == lm.scale
    torch.testing.assert_close(other.params.flat, lm.params.flat)
    b = _batch(cfg)
    other.base.flat.copy_(lm.base.flat)
    torch.testing.assert_close(other.forward(b)[0], lm.forward(b)[0])
    # sampler path samples from the adapted model: decode logits differ from the bare base
    from axon_b200.sampler.engine import GenerationEngine
    from axon_b200.sampler.params import SamplingParams
    eng = GenerationEngine(lm, num_pages=8, max_num_seqs=2)
    out = eng.generate([[5, 6, 7, 8]], SamplingParams(temperature=1.0, max_tokens=4, ignore_eos=True))[0]
    seq = torch.tensor([5, 6, 7, 8] + out.token_ids)
    lp, _ = lm.forward(PackedBatch.from_sequences([seq], "cpu"))
    torch.testing.assert_close(torch.tensor(out.logprobs), lp[3:7], rtol=1e-4, atol=1e-4)


def test_trainer_worker_with_lora_config(tmp_path):
    """`lora.rank` in the trainer config builds the adapter model; checkpoints carry a PEFT adapter directory."""
    import os
    from axon_b200.protocol import DataProto
    from axon_b200.trainer.fsdp_trainer import TrainerWorker
    w = TrainerWorker({"model_path": "tiny-qwen3", "force_cpu": True, "seed": 1, "max_token_len_per_gpu": 256,
                       "optimizer_args": {"lr": 1e-2, "weight_decay": 0.0}, "lora": {"rank": 8, "alpha": 16, "target_modules": "all-linear"}},
                      name="actor")
    w.init_model()
    assert type(w.model).__name__ == "LoRADenseModel" and w.engine.model.params.numel < w.model.base.numel
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 4096, (2, 20), generator=g)
    att = torch.ones(2, 20, dtype=torch.long)
    rm = att.clone().float(); rm[:, :5] = 0
    d = DataProto.from_dict({"input_ids": ids, "attention_mask": att, "position_ids": att.cumsum(1) - 1, "response_mask": rm,
                             "advantages": torch.randn(2, 20, generator=g) * rm})
    d.meta_info["temperature"] = 1.0
    d.batch["old_log_probs"] = w.forward(d).batch["log_probs"]
    w.forward_backward(d, loss_fn="ppo", loss_fn_args={"clip_ratio": 0.2})
    w.optim_step()
    w.save_state(str(tmp_path / "ck"), global_step=1)
    w.wait_for_save()
    assert os.path.exists(tmp_path / "ck" / "lora_adapter" / "adapter_model.safetensors")
    assert os.path.exists(tmp_path / "ck" / "lora_adapter" / "adapter_config.json")
