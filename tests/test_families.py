"""Model families built on ``FamilyModel``: logits and parameter gradients against the HF implementation of the same
architecture (tiny random models, fp32, CPU), the sampler path (prefill + decode over the paged cache) against the
full forward, and one optimizer step through the policy engine."""
import copy

import numpy as np
import pytest
import torch

from axon_b200.models.families import build_family_model, family_config

torch.manual_seed(0)

HF = {
    "deepseek_v3": dict(model_type="deepseek_v3", vocab_size=160, hidden_size=64, num_hidden_layers=3, num_attention_heads=4,
                        num_key_value_heads=4, q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8,
                        v_head_dim=16, n_routed_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1, first_k_dense_replace=1,
                        moe_intermediate_size=32, intermediate_size=96, n_shared_experts=1, routed_scaling_factor=2.5,
                        norm_topk_prob=True, rope_interleave=True, rms_norm_eps=1e-6, max_position_embeddings=256,
                        rope_parameters={"rope_type": "default", "rope_theta": 10000.0}, tie_word_embeddings=False),
    "deepseek_v3_yarn": dict(model_type="deepseek_v3", vocab_size=160, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                             num_key_value_heads=4, q_lora_rank=None, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8,
                             v_head_dim=16, n_routed_experts=4, num_experts_per_tok=2, n_group=1, topk_group=1, first_k_dense_replace=1,
                             moe_intermediate_size=32, intermediate_size=96, n_shared_experts=2, routed_scaling_factor=1.0,
                             norm_topk_prob=True, rope_interleave=True, rms_norm_eps=1e-6, max_position_embeddings=512,
                             rope_parameters={"rope_type": "yarn", "rope_theta": 10000.0, "factor": 4.0, "beta_fast": 32, "beta_slow": 1,
                                              "mscale": 1.0, "mscale_all_dim": 1.0, "original_max_position_embeddings": 128},
                             tie_word_embeddings=False),
    "glm4_moe": dict(model_type="glm4_moe", vocab_size=160, hidden_size=64, num_hidden_layers=3, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=16, partial_rotary_factor=0.5, use_qk_norm=True, attention_bias=True,
                     n_routed_experts=8, num_experts_per_tok=2, n_group=1, topk_group=1, first_k_dense_replace=1, moe_intermediate_size=32,
                     intermediate_size=96, n_shared_experts=1, routed_scaling_factor=1.0, norm_topk_prob=True, rms_norm_eps=1e-5,
                     max_position_embeddings=256, rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5},
                     tie_word_embeddings=False),
    "gpt_oss": dict(model_type="gpt_oss", vocab_size=160, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                    head_dim=16, num_local_experts=4, num_experts_per_tok=2, intermediate_size=48, sliding_window=8, attention_bias=True,
                    rms_norm_eps=1e-5, max_position_embeddings=256, rope_parameters={"rope_type": "default", "rope_theta": 150000.0},
                    tie_word_embeddings=False, layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"]),
    "gemma2": dict(model_type="gemma2", vocab_size=160, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                   head_dim=16, intermediate_size=96, sliding_window=8, query_pre_attn_scalar=24, attn_logit_softcapping=20.0,
                   final_logit_softcapping=10.0, rms_norm_eps=1e-6, max_position_embeddings=256, hidden_activation="gelu_pytorch_tanh",
                   rope_parameters={"rope_type": "default", "rope_theta": 10000.0}, tie_word_embeddings=True),
    "gemma3_text": dict(model_type="gemma3_text", vocab_size=160, hidden_size=64, num_hidden_layers=6, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=16, intermediate_size=96, sliding_window=8, query_pre_attn_scalar=16,
                        rms_norm_eps=1e-6, max_position_embeddings=256, hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True,
                        rope_parameters={"full_attention": {"rope_type": "default", "rope_theta": 1000000.0},
                                         "sliding_attention": {"rope_type": "default", "rope_theta": 10000.0}}),
    "qwen3_next": dict(model_type="qwen3_next", vocab_size=160, hidden_size=64, num_hidden_layers=4, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=16, partial_rotary_factor=0.25, linear_num_value_heads=4, linear_num_key_heads=2,
                       linear_key_head_dim=8, linear_value_head_dim=8, linear_conv_kernel_dim=4, num_experts=4, num_experts_per_tok=2,
                       moe_intermediate_size=32, shared_expert_intermediate_size=32, intermediate_size=96, decoder_sparse_step=1,
                       norm_topk_prob=True, rms_norm_eps=1e-6, max_position_embeddings=256, tie_word_embeddings=False,
                       rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.25},
                       layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"]),
    "qwen3_5_text": dict(model_type="qwen3_5_text", vocab_size=160, hidden_size=64, num_hidden_layers=4, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=16, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=8,
                         linear_value_head_dim=8, linear_conv_kernel_dim=4, intermediate_size=96, rms_norm_eps=1e-6,
                         max_position_embeddings=256, tie_word_embeddings=False,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.25,
                                          "mrope_section": [1, 1, 0], "mrope_interleaved": True},
                         layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"]),
    "gemma4_text": dict(model_type="gemma4_text", vocab_size=160, hidden_size=64, num_hidden_layers=6, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=16, global_head_dim=32, intermediate_size=96, sliding_window=8,
                        hidden_size_per_layer_input=8, vocab_size_per_layer_input=160, num_kv_shared_layers=2, attention_k_eq_v=True,
                        num_global_key_value_heads=1, enable_moe_block=True, num_experts=4, top_k_experts=2, moe_intermediate_size=32,
                        max_position_embeddings=256, use_double_wide_mlp=True, final_logit_softcapping=12.0, rms_norm_eps=1e-6,
                        tie_word_embeddings=True,
                        layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention", "sliding_attention",
                                     "full_attention"],
                        rope_parameters={"sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                                         "full_attention": {"rope_type": "proportional", "partial_rotary_factor": 0.25,
                                                            "rope_theta": 1000000.0}}),
    "glm_moe_dsa": dict(model_type="glm_moe_dsa", vocab_size=160, hidden_size=64, num_hidden_layers=3, num_attention_heads=4,
                        num_key_value_heads=4, q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                        n_routed_experts=8, num_experts_per_tok=2, n_group=1, topk_group=1, first_k_dense_replace=1,
                        moe_intermediate_size=32, intermediate_size=96, n_shared_experts=1, routed_scaling_factor=1.5,
                        norm_topk_prob=True, rms_norm_eps=1e-5, max_position_embeddings=256, index_n_heads=8, index_head_dim=16,
                        index_topk=6, rope_parameters={"rope_type": "default", "rope_theta": 10000.0}, tie_word_embeddings=False,
                        mlp_layer_types=["dense", "sparse", "sparse"]),
    "glm4_moe_lite": dict(model_type="glm4_moe_lite", vocab_size=160, hidden_size=64, num_hidden_layers=3, num_attention_heads=4,
                          num_key_value_heads=4, q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                          n_routed_experts=8, num_experts_per_tok=2, n_group=1, topk_group=1, first_k_dense_replace=1,
                          moe_intermediate_size=32, intermediate_size=96, n_shared_experts=1, routed_scaling_factor=1.8,
                          norm_topk_prob=True, rms_norm_eps=1e-5, max_position_embeddings=256,
                          rope_parameters={"rope_type": "default", "rope_theta": 10000.0}, tie_word_embeddings=False),
}


def _hf_model(name):
    import transformers
    hf = dict(HF[name])
    mt = hf["model_type"]
    cfg_cls = transformers.CONFIG_MAPPING[mt]
    cfg = cfg_cls(**{k: v for k, v in hf.items() if k != "model_type"})
    cfg._attn_implementation = "eager"
    model = transformers.AutoModelForCausalLM.from_config(cfg, attn_implementation="eager").float().eval()
    with torch.no_grad():                                   # make every parameter matter (HF zero-initialises some)
        g = torch.Generator().manual_seed(1)
        for n, p in model.named_parameters():
            if p.dim() >= 2 or n.endswith(("bias", "sinks", "dt_bias", "A_log")):
                p.copy_(torch.randn(p.shape, generator=g) * (0.08 if p.dim() >= 2 else 0.3))
            else:
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=g) if "norm" in n and mt not in ("gemma2", "gemma3_text", "qwen3_next", "qwen3_5_text")
                        else 0.1 * torch.randn(p.shape, generator=g))
        for n, b in model.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.copy_(0.1 * torch.randn(b.shape, generator=g))
            if n.endswith("layer_scalar"):
                b.copy_(1.0 + 0.2 * torch.randn(b.shape, generator=g))
        if "A_log" in dict(model.named_parameters()).keys().__str__():
            for n, p in model.named_parameters():
                if n.endswith("A_log"):
                    p.copy_(torch.log(torch.empty(p.shape).uniform_(1, 8, generator=g)))
    return model, cfg


def _ours_from(model, name):
    hf = dict(HF[name])
    ours = build_family_model(hf, "cpu", torch.float32)
    ours.load_state_dict({k: v.detach().clone() for k, v in model.state_dict().items()})
    return ours


@pytest.mark.parametrize("name", list(HF))
def test_logits_match_transformers(name):
    try:
        model, _ = _hf_model(name)
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"transformers cannot build {name}: {type(e).__name__}: {e}")
    ours = _ours_from(model, name)
    ids = torch.randint(0, 160, (37,))
    with torch.no_grad():
        ref = model(input_ids=ids[None]).logits[0].float()
    got = ours.logits(ids)
    assert (got - ref).abs().max() < 2e-4 * max(1.0, ref.abs().max().item()), (got - ref).abs().max()


@pytest.mark.parametrize("name", ["deepseek_v3", "gpt_oss", "gemma2", "qwen3_next", "glm4_moe", "gemma4_text"])
def test_gradients_match_transformers(name):
    from axon_b200.models.dense import PackedBatch
    try:
        model, _ = _hf_model(name)
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"transformers cannot build {name}: {type(e).__name__}: {e}")
    ours = _ours_from(model, name)
    seqs = [torch.randint(2, 160, (n,)) for n in (19, 11)]      # id 0 is HF's padding row (its lookups get no gradient there)
    batch = PackedBatch.from_sequences(seqs, "cpu")
    for recompute in ("full", "none"):
        ours.recompute = recompute
        ours.params.free_grads()
        lp, ent = ours.forward(batch, 1.0, save_for_backward=True)
        g = torch.randn(lp.shape, generator=torch.Generator().manual_seed(2)) * (batch.labels >= 0)
        ours.backward(g, 0.1 * torch.ones_like(ent))
        model.zero_grad()
        total = 0.0
        off = 0
        for s in seqs:
            z = model(input_ids=s[None]).logits[0].float()
            logp = torch.log_softmax(z, -1)
            lab = batch.labels[off:off + len(s)]
            lps = logp.gather(1, lab.clamp_min(0)[:, None].long())[:, 0] * (lab >= 0)
            ents = -(logp.exp() * logp).sum(-1)
            total = total + (lps * g[off:off + len(s)]).sum() + 0.1 * ents.sum()
            off += len(s)
        total.backward()
        ref = {n: p.grad for n, p in model.named_parameters() if p.grad is not None}
        checked = 0
        for n, gr in ref.items():
            mine = ours.params.grads[n].view(gr.shape)
            scale = max(gr.abs().max().item(), 1e-6)
            assert (mine - gr).abs().max() < 2e-3 * scale + 1e-6, (name, recompute, n, (mine - gr).abs().max().item(), scale)
            checked += 1
        assert checked >= 10


@pytest.mark.parametrize("name", ["deepseek_v3", "gpt_oss", "gemma3_text", "qwen3_next", "glm_moe_dsa", "gemma4_text"])
def test_sampler_path_matches_full_forward(name):
    """Prefill a prompt into the paged cache, decode three tokens one at a time: every step's logits equal the logits
    of the full forward over the tokens so far."""
    from axon_b200.models.dense import PackedBatch
    from axon_b200.sampler.engine import GenerationEngine
    from axon_b200.sampler.params import SamplingParams
    hf = dict(HF[name])
    ours = build_family_model(hf, "cpu", torch.float32)
    ours.init_random(0.08, seed=3)
    eng = GenerationEngine(ours, num_pages=12, max_num_seqs=4)
    prompts = [torch.randint(2, 160, (n,)).tolist() for n in (140, 9)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o.token_ids:
            z = ours.logits(torch.tensor(seq))[-1]
            assert int(z.argmax()) == tok, (name, len(seq))
            seq.append(tok)
    # the engine's log-probs agree with a teacher-forced forward
    o = outs[0]
    seq = torch.tensor(prompts[0] + o.token_ids)
    lp, _ = ours.forward(PackedBatch.from_sequences([seq], "cpu"), 1.0)
    ref = lp[len(prompts[0]) - 1: len(prompts[0]) - 1 + len(o.token_ids)]
    assert len(o.logprobs) == 4 and torch.isfinite(ref).all()


def test_policy_engine_steps_a_family_model():
    from axon_b200.protocol import DataProto
    from axon_b200.trainer.policy import OptimConfig, PolicyEngine
    ours = build_family_model(dict(HF["gpt_oss"]), "cpu", torch.float32)
    ours.init_random(0.05, seed=5)
    eng = PolicyEngine(ours, OptimConfig(lr=1e-2, weight_decay=0.0, grad_clip=1.0), max_token_len_per_gpu=64)
    B, T = 4, 24
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(2, 160, (B, T), generator=g)
    att = torch.ones(B, T, dtype=torch.long)
    att[1, 15:] = 0
    resp = att.clone().float()
    resp[:, :5] = 0
    adv = torch.randn(B, 1, generator=g).expand(B, T) * resp
    d = DataProto.from_dict({"input_ids": ids * att, "attention_mask": att, "response_mask": resp, "advantages": adv},
                            {"uid": np.arange(B).astype(object)})
    d.batch["valid_token_count"] = resp.sum().expand(B).clone()
    old = eng.forward(d).batch["log_probs"]
    d.batch["old_log_probs"] = old

    def objective():
        lp = eng.forward(d).batch["log_probs"]
        return ((lp - old) * adv * resp).sum().item()
    before = objective()
    for _ in range(3):
        eng.forward_backward(copy.deepcopy(d), "ppo", {})
        st = eng.optim_step()
        assert np.isfinite(st["grad_norm"]) and st["grad_norm"] > 0
    assert objective() > before + 1e-4


def test_family_config_describes_the_cache():
    cfg = family_config(dict(HF["deepseek_v3"]))
    assert cfg.num_key_value_heads == 4 and cfg.head_dim == 24 and cfg.num_experts == 8
    cfg = family_config(dict(HF["gemma3_text"]))
    assert cfg.tie_word_embeddings and cfg.head_dim == 16


def test_hf_directory_round_trip_and_per_expert_checkpoints(tmp_path):
    """``build_model`` on a preset, export as an HF directory, build again from the directory: same logits. A checkpoint
    that stores each expert separately loads into the stacked expert tensors."""
    from axon_b200.utils.hf_model import build_model, save_hf_model
    m = build_model("tiny-deepseek-v3", device="cpu", dtype=torch.float32, seed=3)
    ids = torch.randint(2, 4096, (33,))
    ref = m.logits(ids)
    save_hf_model(m, str(tmp_path / "ck"))
    m2 = build_model(str(tmp_path / "ck"), device="cpu", dtype=torch.float32)
    assert type(m2).__name__ == "FamilyModel" and torch.equal(m2.logits(ids), ref)
    sd = dict(m.params.to_hf_state_dict())
    split = {}
    for k, v in sd.items():
        if k.endswith("mlp.experts.gate_up_proj"):
            base = k[: -len("gate_up_proj")]
            for e in range(v.shape[0]):
                g, u = v[e].chunk(2, dim=0)
                split[f"{base}{e}.gate_proj.weight"], split[f"{base}{e}.up_proj.weight"] = g.clone(), u.clone()
        elif k.endswith("mlp.experts.down_proj"):
            base = k[: -len("down_proj")]
            for e in range(v.shape[0]):
                split[f"{base}{e}.down_proj.weight"] = v[e].clone()
        else:
            split[k] = v.clone()
    m3 = build_model("tiny-deepseek-v3", device="cpu", dtype=torch.float32, seed=9)
    m3.params.load_hf_state_dict(split)
    assert torch.equal(m3.logits(ids), ref)


@pytest.mark.timeout(600)
@pytest.mark.parametrize("preset", ["tiny-gpt-oss", "tiny-qwen3-next"])
def test_driver_trains_a_family_model_end_to_end(tmp_path, preset):
    """The whole stack (driver, worker groups, engine, program, sampler, trainer) on a family model: two RL steps."""
    import json
    import os

    from axon_b200.driver.train_agent_ppo import train_agent
    from axon_b200.utils.config import compose_config
    rows = [{"question": f"What is {i}+{i}?", "ground_truth": str(2 * i), "data_source": "toy", "reward_fn": "bernoulli"} for i in range(8)]
    data = tmp_path / "train.jsonl"
    data.write_text("".join(json.dumps(r) + "\n" for r in rows))
    os.environ["AXON_FILE_LOGGER_ROOT"] = str(tmp_path)
    cfg = compose_config([f"train_files={data}", f"model_path={preset}", "+force_cpu=true", "train_batch_size=2", "decoding.n=2",
                          "mini_batch_size=2", "max_seq_length=256", "max_prompt_length=200", f"output_dir={tmp_path}/out", "advantage=grpo",
                          "validation.before_train=false", "+sampler.num_kv_pages=64", "sampler.max_num_seqs=8", "max_tokens_per_step=8",
                          "drop_zero_advantage_samples=false", "actor.max_token_len_per_gpu=512", "save_programs_flag=false", "logger=[file]",
                          "num_gpus_per_node=1", "total_training_steps=2", "save_steps=-1"])
    drv = train_agent(cfg, backend="inline", keep_alive=True)
    try:
        assert drv.global_steps == 3
    finally:
        drv.shutdown()
    logs = [json.loads(line) for line in open(tmp_path / "axon-agent_ppo.jsonl")]
    assert [r["step"] for r in logs][:2] == [1, 2] and logs[0]["data"]["batch/sampler_logprobs_diff_mean"] < 1e-4


def test_qwen2_vl_matches_transformers_with_an_image():
    """Vision tower + three-row rotary decoder against HF Qwen2-VL on a prompt with one image and one text-only prompt:
    logits, the gradient of a log-prob loss through decoder AND tower, and the HF state-dict round trip."""
    try:
        from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration
    except Exception:
        pytest.skip("transformers has no Qwen2-VL")
    from axon_b200.models.config import ModelConfig
    from axon_b200.models.dense import PackedBatch
    from axon_b200.models.families import FamilyModel
    torch.manual_seed(0)
    cfg = Qwen2VLConfig(text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                         vocab_size=300, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}, max_position_embeddings=512,
                                         tie_word_embeddings=False),
                        vision_config=dict(depth=2, embed_dim=32, hidden_size=64, num_heads=2, mlp_ratio=2, in_channels=3, patch_size=4,
                                           temporal_patch_size=2, spatial_merge_size=2),
                        image_token_id=290, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)
    ref = Qwen2VLForConditionalGeneration(cfg).float().eval()
    grid = torch.tensor([[1, 4, 6]])                               # one image: 24 patches -> 6 placeholder tokens
    pix = torch.randn(24, 3 * 2 * 4 * 4)
    ids = torch.tensor([[5, 17, 292] + [290] * 6 + [293, 44, 9, 120, 33, 7]])
    with torch.no_grad():
        types = (ids == 290).int()                                 # 1 marks image placeholder tokens
        want = ref(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=types).logits[0].float()
        got_pos = ref.model.get_rope_index(ids, types, image_grid_thw=grid, attention_mask=torch.ones_like(ids))[0][:, 0]      # [3, T]
    mcfg = ModelConfig.from_hf_dict(cfg.to_dict())
    assert mcfg.to_hf_dict()["text_config"]["hidden_size"] == 64          # the nested form survives for export
    m = FamilyModel(mcfg, device="cpu", dtype=torch.float32)
    m.load_state_dict(ref.state_dict())
    mm = {"pixel_values": pix, "image_grid_thw": grid, "mrope_positions": got_pos}
    z = m.logits(ids[0].to(torch.int32), multimodal=mm)
    assert (z - want).abs().max() < 2e-4, (z - want).abs().max()
    # our own position builder gives the rows HF computes
    from axon_b200.models.vision import mrope_position_ids

    class _Proc:
        image_token_id, video_token_id, vision_start_token_id = 290, 291, 292

        class image_processor:
            merge_size = 2
    mine = mrope_position_ids(_Proc, ids, torch.ones_like(ids), image_grid_thw=grid)
    assert torch.equal(mine.reshape(3, -1).long(), got_pos.long())
    # text-only: plain positions serve all three rows
    t_ids = torch.randint(0, 280, (1, 12))
    with torch.no_grad():
        want_t = ref(input_ids=t_ids).logits[0].float()
    assert (m.logits(t_ids[0].to(torch.int32)) - want_t).abs().max() < 2e-4
    # gradients through decoder and tower
    batch = PackedBatch.from_sequences([ids[0]], "cpu")
    batch.multimodal = mm
    lp, _ = m.forward(batch, 1.0, save_for_backward=True)
    g = torch.linspace(0.5, 1.5, lp.numel())
    g[-1] = 0
    m.backward(g)
    out = ref(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=types).logits[0].float()
    lp_ref = torch.log_softmax(out[:-1], -1).gather(1, ids[0, 1:, None])[:, 0]
    assert (lp[:-1] - lp_ref.detach()).abs().max() < 2e-4
    (lp_ref * g[:-1]).sum().backward()
    sd = dict(ref.named_parameters())
    for name in ("model.visual.blocks.0.attn.qkv.weight", "model.visual.merger.mlp.2.weight", "model.language_model.layers.1.self_attn.k_proj.bias",
                 "model.language_model.layers.0.mlp.down_proj.weight", "model.visual.patch_embed.proj.weight"):
        a, b = m.params.grads[name], sd[name].grad.reshape(m.params.grads[name].shape)
        assert (a - b).abs().max() < 2e-4 * max(1.0, b.abs().max().item()), name
    # round trip in the checkpoint's shapes
    ref2 = Qwen2VLForConditionalGeneration(cfg).float()
    ref2.load_state_dict({k: v.clone() for k, v in m.params.to_hf_state_dict().items()})
    with torch.no_grad():
        assert torch.equal(ref2(input_ids=t_ids).logits, ref(input_ids=t_ids).logits)


def test_policy_engine_trains_a_vision_language_model_on_padded_rows_with_images():
    """Rows with and without images through ``PolicyEngine``: per-row ``multi_modal_inputs`` and the [B, 4, T] position
    rows of the driver are packed for the model; log-probs equal the per-sequence forward, and an update moves the
    vision tower as well as the decoder."""
    from axon_b200.models.config import ModelConfig
    from axon_b200.models.families import FamilyModel
    from axon_b200.models.vision import mrope_position_ids
    from axon_b200.protocol import DataProto
    from axon_b200.trainer.policy import OptimConfig, PolicyEngine
    hf = {"model_type": "qwen2_vl", "image_token_id": 290, "video_token_id": 291, "vision_start_token_id": 292, "vision_end_token_id": 293,
          "text_config": dict(model_type="qwen2_vl_text", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                              num_key_value_heads=2, vocab_size=300, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}, rope_theta=10000.0,
                              max_position_embeddings=512, tie_word_embeddings=False, rms_norm_eps=1e-6),
          "vision_config": dict(depth=1, embed_dim=32, hidden_size=64, num_heads=2, mlp_ratio=2, in_channels=3, patch_size=4,
                                temporal_patch_size=2, spatial_merge_size=2)}
    m = FamilyModel(ModelConfig.from_hf_dict(hf), device="cpu", dtype=torch.float32)
    m.init_random(0.05, seed=2)
    g = torch.Generator().manual_seed(1)
    T = 20
    rows = [[5, 17, 292] + [290] * 6 + [293, 44, 9, 120, 33, 7], torch.randint(2, 280, (12,), generator=g).tolist(),
            [292] + [290] * 4 + [293, 8, 9, 10]]
    grids = [torch.tensor([[1, 4, 6]]), None, torch.tensor([[1, 4, 4]])]
    pix = [torch.randn(24, 96, generator=g), None, torch.randn(16, 96, generator=g)]
    ids = torch.zeros(3, T, dtype=torch.long)
    att = torch.zeros(3, T, dtype=torch.long)
    for b, r in enumerate(rows):
        ids[b, :len(r)], att[b, :len(r)] = torch.tensor(r), 1

    class _Proc:
        image_token_id, video_token_id, vision_start_token_id = 290, 291, 292

        class image_processor:
            merge_size = 2
    text = (att.cumsum(1) - 1) * att
    pos = torch.stack([torch.cat([text[b:b + 1], mrope_position_ids(_Proc, ids[b], att[b], image_grid_thw=grids[b]).reshape(3, T)]) for b in range(3)])
    mm = np.empty(3, dtype=object)
    for b in range(3):
        mm[b] = {} if grids[b] is None else {"pixel_values": pix[b], "image_grid_thw": grids[b]}
    resp = att.clone().float()
    resp[:, :2] = 0
    d = DataProto.from_dict({"input_ids": ids, "attention_mask": att, "position_ids": pos, "response_mask": resp,
                             "advantages": torch.randn(3, 1, generator=g).expand(3, T) * resp}, {"multi_modal_inputs": mm})
    d.batch["valid_token_count"] = resp.sum().expand(3).clone()
    eng = PolicyEngine(m, OptimConfig(lr=5e-3, weight_decay=0.0, grad_clip=1.0), max_token_len_per_gpu=32)     # several micro-batches
    lp = eng.forward(d).batch["log_probs"]
    for b, r in enumerate(rows):
        n = len(r)
        one = {"pixel_values": pix[b], "image_grid_thw": grids[b], "mrope_positions": pos[b, 1:, :n]} if grids[b] is not None else None
        z = m.logits(ids[b, :n].to(torch.int32), multimodal=one)
        want = torch.log_softmax(z[:-1], -1).gather(1, ids[b, 1:n, None])[:, 0]
        assert (lp[b, 1:n] - want).abs().max() < 1e-4, b
    d.batch["old_log_probs"] = lp
    before = {k: m.params[k].clone() for k in ("model.visual.blocks.0.attn.qkv.weight", "model.language_model.layers.1.mlp.up_proj.weight")}
    eng.forward_backward(copy.deepcopy(d), "ppo", {})
    st = eng.optim_step()
    assert np.isfinite(st["grad_norm"]) and st["grad_norm"] > 0
    for k, v in before.items():
        assert (m.params[k] - v).abs().max() > 0, k


def test_sampler_generates_from_a_prompt_with_an_image():
    """Greedy generation through the paged engine for a prompt with an image (and a text-only neighbour in the same
    batch): every sampled token's log-prob equals the full forward over prompt + output with the rotary rows continued
    after the image; two samples of the same request object share the prompt's pages."""
    from axon_b200.models.config import ModelConfig
    from axon_b200.models.families import FamilyModel
    from axon_b200.sampler.engine import GenerationEngine
    from axon_b200.sampler.params import SamplingParams
    hf = {"model_type": "qwen2_vl", "image_token_id": 290, "video_token_id": 291, "vision_start_token_id": 292, "vision_end_token_id": 293,
          "text_config": dict(model_type="qwen2_vl_text", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                              num_key_value_heads=2, vocab_size=300, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}, rope_theta=10000.0,
                              max_position_embeddings=512, tie_word_embeddings=False, rms_norm_eps=1e-6, eos_token_id=299),
          "vision_config": dict(depth=1, embed_dim=32, hidden_size=64, num_heads=2, mlp_ratio=2, in_channels=3, patch_size=4,
                                temporal_patch_size=2, spatial_merge_size=2)}
    m = FamilyModel(ModelConfig.from_hf_dict(hf), device="cpu", dtype=torch.float32)
    m.init_random(0.08, seed=4)
    g = torch.Generator().manual_seed(2)
    img = {"pixel_values": torch.randn(24, 96, generator=g), "image_grid_thw": torch.tensor([[1, 4, 6]])}
    p_img = [5, 17, 292] + [290] * 6 + [293, 44, 9]
    p_txt = torch.randint(2, 280, (9,), generator=g).tolist()
    eng = GenerationEngine(m, num_pages=16, max_num_seqs=4)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    outs = eng.generate([p_img, p_txt, p_img], sp, image_data=[img, None, img])
    assert eng.stats.get("shared_prompt_seqs", 0) == 1 and outs[0].token_ids == outs[2].token_ids
    assert eng.cache.num_free() == 16
    # full forward over prompt + output, rotary rows as the engine continues them
    full = p_img + outs[0].token_ids
    rows = m.rotary_rows(p_img, img)
    delta = int(rows.max()) + 1 - len(p_img)
    assert delta < 0                                              # six placeholders advance the rotary count by less than six
    pos = torch.cat([rows, (torch.arange(len(outs[0].token_ids)) + len(p_img) + delta)[None].expand(3, -1)], dim=1)
    z = m.logits(torch.tensor(full, dtype=torch.int32), multimodal={**img, "mrope_positions": pos})
    lp = torch.log_softmax(z, -1)
    for i, (tok, got) in enumerate(zip(outs[0].token_ids, outs[0].logprobs)):
        row = len(p_img) - 1 + i
        assert int(lp[row].argmax()) == tok
        assert abs(float(lp[row, tok]) - got) < 1e-4
    zt = torch.log_softmax(m.logits(torch.tensor(p_txt + outs[1].token_ids, dtype=torch.int32)), -1)
    for i, (tok, got) in enumerate(zip(outs[1].token_ids, outs[1].logprobs)):
        assert abs(float(zt[len(p_txt) - 1 + i, tok]) - got) < 1e-4
    # the same request through the server front end (processor output as plain lists, as the HTTP body carries it)
    from axon_b200.sampler.server import SamplerServer
    srv = SamplerServer(eng, name="vl").start()
    try:
        fut = srv.submit(p_img, {"temperature": 0.0, "max_tokens": 6, "ignore_eos": True},
                         image_data={"pixel_values": img["pixel_values"].tolist(), "image_grid_thw": img["image_grid_thw"].tolist()})
        assert fut.result(timeout=60).token_ids == outs[0].token_ids
        with pytest.raises(ValueError, match="processor"):
            srv.submit(p_img, {}, image_data=["data:image/png;base64,AAAA"])
    finally:
        srv.stop()


def test_qwen2_5_vl_windowed_tower_matches_transformers():
    """Windowed vision tower (regrouping by windows, full-attention blocks, RMSNorm, gated MLP) + decoder against HF
    Qwen2.5-VL with two images of different sizes (one larger than a window): logits and tower gradients."""
    try:
        from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration
    except Exception:
        pytest.skip("transformers has no Qwen2.5-VL")
    from axon_b200.models.config import ModelConfig
    from axon_b200.models.dense import PackedBatch
    from axon_b200.models.families import FamilyModel
    torch.manual_seed(0)
    cfg = Qwen2_5_VLConfig(text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                            vocab_size=300, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}, max_position_embeddings=512,
                                            tie_word_embeddings=False),
                           vision_config=dict(depth=4, hidden_size=32, out_hidden_size=64, intermediate_size=48, num_heads=2, in_channels=3, patch_size=4,
                                              temporal_patch_size=2, spatial_merge_size=2, window_size=16, fullatt_block_indexes=[1, 3]),
                           image_token_id=290, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)
    ref = Qwen2_5_VLForConditionalGeneration(cfg).float().eval()
    grid = torch.tensor([[1, 6, 8], [1, 2, 4]])                    # 48 + 8 patches -> 12 + 2 placeholder tokens; windows of 2 x 2 merged units
    pix = torch.randn(56, 3 * 2 * 4 * 4)
    ids = torch.tensor([[5, 292] + [290] * 12 + [293, 44, 292] + [290] * 2 + [293, 9, 120, 33]])
    types = (ids == 290).int()
    with torch.no_grad():
        want = ref(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=types).logits[0].float()
        pos = ref.model.get_rope_index(ids, types, image_grid_thw=grid, attention_mask=torch.ones_like(ids))[0][:, 0]
    m = FamilyModel(ModelConfig.from_hf_dict(cfg.to_dict()), device="cpu", dtype=torch.float32)
    m.load_state_dict(ref.state_dict())
    mm = {"pixel_values": pix, "image_grid_thw": grid, "mrope_positions": pos}
    z = m.logits(ids[0].to(torch.int32), multimodal=mm)
    assert (z - want).abs().max() < 2e-4, (z - want).abs().max()
    # height / width rows and every text position agree with HF; for image tokens this build keeps the temporal row at the
    # image's first position (a still image has one frame), where transformers 5.5 scales that offset by tokens_per_second
    mine = m.rotary_rows(ids[0].tolist(), {"image_grid_thw": grid}).long()
    assert torch.equal(mine[1:], pos[1:].long()) and torch.equal(mine[0][types[0] == 0], pos[0][types[0] == 0].long())
    assert mine[0][types[0] == 1].tolist() == [2] * 12 + [9] * 2
    batch = PackedBatch.from_sequences([ids[0]], "cpu")
    batch.multimodal = mm
    lp, _ = m.forward(batch, 1.0, save_for_backward=True)
    g = torch.linspace(0.5, 1.5, lp.numel())
    g[-1] = 0
    m.backward(g)
    out = ref(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=types).logits[0].float()
    lp_ref = torch.log_softmax(out[:-1], -1).gather(1, ids[0, 1:, None])[:, 0]
    (lp_ref * g[:-1]).sum().backward()
    sd = dict(ref.named_parameters())
    for name in ("model.visual.blocks.0.attn.qkv.weight", "model.visual.blocks.1.mlp.gate_proj.bias", "model.visual.merger.ln_q.weight",
                 "model.visual.patch_embed.proj.weight"):
        a, b = m.params.grads[name], sd[name].grad.reshape(m.params.grads[name].shape)
        assert (a - b).abs().max() < 2e-4 * max(1.0, b.abs().max().item()), name


def test_qwen3_vl_deepstack_and_interleaved_rotary_match_transformers():
    """Qwen3-VL: interpolated position table, DeepStack taps added after the first decoder layers, interleaved
    three-row rotary positions, query / key norms - logits and gradients (tower taps included) against HF."""
    try:
        from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration
    except Exception:
        pytest.skip("transformers has no Qwen3-VL")
    from axon_b200.models.config import ModelConfig
    from axon_b200.models.dense import PackedBatch
    from axon_b200.models.families import FamilyModel
    torch.manual_seed(0)
    cfg = Qwen3VLConfig(text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                                         head_dim=16, vocab_size=300, rope_scaling={"rope_type": "default", "mrope_section": [2, 3, 3], "mrope_interleaved": True},
                                         max_position_embeddings=512, tie_word_embeddings=False),
                        vision_config=dict(depth=3, hidden_size=32, out_hidden_size=64, intermediate_size=48, num_heads=2, in_channels=3, patch_size=4,
                                           temporal_patch_size=2, spatial_merge_size=2, num_position_embeddings=64, deepstack_visual_indexes=[0, 1]),
                        image_token_id=290, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)
    ref = Qwen3VLForConditionalGeneration(cfg).float().eval()
    grid = torch.tensor([[1, 6, 8], [1, 2, 4]])
    pix = torch.randn(56, 3 * 2 * 4 * 4)
    ids = torch.tensor([[5, 292] + [290] * 12 + [293, 44, 292] + [290] * 2 + [293, 9, 120, 33]])
    types = (ids == 290).int()
    with torch.no_grad():
        want = ref(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=types).logits[0].float()
        pos = ref.model.get_rope_index(ids, types, image_grid_thw=grid, attention_mask=torch.ones_like(ids))[0][:, 0]
    m = FamilyModel(ModelConfig.from_hf_dict(cfg.to_dict()), device="cpu", dtype=torch.float32)
    m.load_state_dict(ref.state_dict())
    mm = {"pixel_values": pix, "image_grid_thw": grid, "mrope_positions": pos}
    z = m.logits(ids[0].to(torch.int32), multimodal=mm)
    assert (z - want).abs().max() < 2e-4, (z - want).abs().max()
    assert torch.equal(m.rotary_rows(ids[0].tolist(), {"image_grid_thw": grid}).long(), pos.long())
    t_ids = torch.randint(0, 280, (1, 12))
    with torch.no_grad():
        assert (m.logits(t_ids[0].to(torch.int32)) - ref(input_ids=t_ids).logits[0].float()).abs().max() < 2e-4
    batch = PackedBatch.from_sequences([ids[0]], "cpu")
    batch.multimodal = mm
    lp, _ = m.forward(batch, 1.0, save_for_backward=True)
    g = torch.linspace(0.5, 1.5, lp.numel())
    g[-1] = 0
    m.backward(g)
    out = ref(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=types).logits[0].float()
    lp_ref = torch.log_softmax(out[:-1], -1).gather(1, ids[0, 1:, None])[:, 0]
    (lp_ref * g[:-1]).sum().backward()
    sd = dict(ref.named_parameters())
    for name in ("model.visual.pos_embed.weight", "model.visual.deepstack_merger_list.1.linear_fc2.weight", "model.visual.blocks.0.attn.qkv.weight",
                 "model.language_model.layers.2.self_attn.k_norm.weight", "model.visual.patch_embed.proj.bias"):
        a, b = m.params.grads[name], sd[name].grad.reshape(m.params.grads[name].shape)
        assert (a - b).abs().max() < 2e-4 * max(1.0, b.abs().max().item()), name


def test_glm4v_tower_and_partial_interleaved_rotary_match_transformers():
    """GLM-4.1V: bicubically sampled position table, RMSNorm / SwiGLU tower with the strided-convolution merger,
    sandwich-norm decoder with three-row rotary angles on interleaved pairs of half of each head - logits and
    gradients (decoder and tower) against HF."""
    try:
        from transformers import Glm4vConfig, Glm4vForConditionalGeneration
    except Exception:
        pytest.skip("transformers has no GLM-4V")
    from axon_b200.models.config import ModelConfig
    from axon_b200.models.dense import PackedBatch
    from axon_b200.models.families import FamilyModel
    torch.manual_seed(0)
    cfg = Glm4vConfig(text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                       vocab_size=300, max_position_embeddings=512,
                                       rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [2, 1, 1], "partial_rotary_factor": 0.5}),
                      vision_config=dict(depth=2, hidden_size=32, out_hidden_size=64, intermediate_size=48, num_heads=2, in_channels=3, patch_size=4,
                                         temporal_patch_size=2, spatial_merge_size=2, image_size=32),
                      image_token_id=290, video_token_id=291, image_start_token_id=292, image_end_token_id=293)
    ref = Glm4vForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for n, p in ref.named_parameters():          # norms away from one, biases away from zero
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    grid = torch.tensor([[1, 6, 8], [1, 2, 4]])
    pix = torch.randn(56, 3 * 2 * 4 * 4)
    ids = torch.tensor([[5, 292] + [290] * 12 + [293, 44, 292] + [290] * 2 + [293, 9, 120, 33]])
    types = (ids == 290).int()
    with torch.no_grad():
        want = ref(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=types).logits[0].float()
        pos = ref.model.get_rope_index(ids, types, image_grid_thw=grid, attention_mask=torch.ones_like(ids))[0][:, 0]
    m = FamilyModel(ModelConfig.from_hf_dict(cfg.to_dict()), device="cpu", dtype=torch.float32)
    m.load_state_dict(ref.state_dict())
    mm = {"pixel_values": pix, "image_grid_thw": grid, "mrope_positions": pos}
    z = m.logits(ids[0].to(torch.int32), multimodal=mm)
    assert (z - want).abs().max() < 2e-4, (z - want).abs().max()
    assert torch.equal(m.rotary_rows(ids[0].tolist(), {"image_grid_thw": grid}).long(), pos.long())
    t_ids = torch.randint(0, 280, (1, 12))
    with torch.no_grad():
        assert (m.logits(t_ids[0].to(torch.int32)) - ref(input_ids=t_ids).logits[0].float()).abs().max() < 2e-4
    exported = m.params.to_hf_state_dict()           # the checkpoint's shapes: the strided convolution as a Conv2d kernel
    assert tuple(exported["model.visual.downsample.weight"].shape) == (64, 32, 2, 2)
    assert torch.equal(exported["model.visual.downsample.weight"], ref.state_dict()["model.visual.downsample.weight"])
    batch = PackedBatch.from_sequences([ids[0]], "cpu")
    batch.multimodal = mm
    lp, _ = m.forward(batch, 1.0, save_for_backward=True)
    g = torch.linspace(0.5, 1.5, lp.numel())
    g[-1] = 0
    m.backward(g)
    out = ref(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=types).logits[0].float()
    lp_ref = torch.log_softmax(out[:-1], -1).gather(1, ids[0, 1:, None])[:, 0]
    (lp_ref * g[:-1]).sum().backward()
    named = dict(ref.named_parameters())
    for name in ("model.visual.embeddings.position_embedding.weight", "model.visual.downsample.weight", "model.visual.blocks.0.attn.qkv.weight",
                 "model.visual.merger.post_projection_norm.bias", "model.language_model.layers.1.post_mlp_layernorm.weight",
                 "model.language_model.layers.0.mlp.gate_up_proj.weight", "model.language_model.layers.0.self_attn.k_proj.bias"):
        a, b = m.params.grads[name], named[name].grad.reshape(m.params.grads[name].shape)
        assert (a - b).abs().max() < 2e-4 * max(1.0, b.abs().max().item()), name


def test_qwen3_vl_moe_sparse_decoder_matches_transformers():
    """Qwen3-VL-MoE: the Qwen3-VL tower and DeepStack in front of a decoder with routed experts."""
    try:
        from transformers import Qwen3VLMoeConfig, Qwen3VLMoeForConditionalGeneration
    except Exception:
        pytest.skip("transformers has no Qwen3-VL-MoE")
    from axon_b200.models.config import ModelConfig
    from axon_b200.models.dense import PackedBatch
    from axon_b200.models.families import FamilyModel
    torch.manual_seed(0)
    cfg = Qwen3VLMoeConfig(text_config=dict(hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_experts=4, num_experts_per_tok=2,
                                            num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=300,
                                            decoder_sparse_step=1, mlp_only_layers=[1], max_position_embeddings=512,
                                            rope_scaling={"rope_type": "default", "mrope_section": [2, 3, 3], "mrope_interleaved": True}),
                           vision_config=dict(depth=2, hidden_size=32, out_hidden_size=64, intermediate_size=48, num_heads=2, in_channels=3, patch_size=4,
                                              temporal_patch_size=2, spatial_merge_size=2, num_position_embeddings=64, deepstack_visual_indexes=[0]),
                           image_token_id=290, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)
    ref = Qwen3VLMoeForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for n, p in ref.named_parameters():
            if "experts" in n or n.endswith("mlp.gate.weight"):
                p.normal_(0, 0.2)
    grid = torch.tensor([[1, 4, 4]])
    pix = torch.randn(16, 3 * 2 * 4 * 4)
    ids = torch.tensor([[5, 292] + [290] * 4 + [293, 44, 9, 120, 33, 7]])
    types = (ids == 290).int()
    with torch.no_grad():
        want = ref(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=types).logits[0].float()
        pos = ref.model.get_rope_index(ids, types, image_grid_thw=grid, attention_mask=torch.ones_like(ids))[0][:, 0]
    m = FamilyModel(ModelConfig.from_hf_dict(cfg.to_dict()), device="cpu", dtype=torch.float32)
    assert m.cfg.num_experts == 4
    m.load_state_dict(ref.state_dict())
    mm = {"pixel_values": pix, "image_grid_thw": grid, "mrope_positions": pos}
    z = m.logits(ids[0].to(torch.int32), multimodal=mm)
    assert (z - want).abs().max() < 2e-4, (z - want).abs().max()
    batch = PackedBatch.from_sequences([ids[0]], "cpu")
    batch.multimodal = mm
    lp, _ = m.forward(batch, 1.0, save_for_backward=True)
    g = torch.linspace(0.5, 1.5, lp.numel())
    g[-1] = 0
    m.backward(g)
    out = ref(input_ids=ids, pixel_values=pix, image_grid_thw=grid, mm_token_type_ids=types).logits[0].float()
    lp_ref = torch.log_softmax(out[:-1], -1).gather(1, ids[0, 1:, None])[:, 0]
    (lp_ref * g[:-1]).sum().backward()
    named = dict(ref.named_parameters())
    for name in ("model.language_model.layers.0.mlp.experts.gate_up_proj", "model.language_model.layers.2.mlp.gate.weight",
                 "model.language_model.layers.1.mlp.up_proj.weight", "model.visual.deepstack_merger_list.0.linear_fc1.weight"):
        a, b = m.params.grads[name], named[name].grad
        assert (a - b).abs().max() < 2e-4 * max(1.0, b.abs().max().item()), name


def test_multimodal_checkpoint_of_a_text_family_is_read_text_only():
    """A multimodal wrapper (``gemma3`` around ``gemma3_text``): the configuration is the nested decoder's, its tensors are
    found under ``model.language_model.``, tower tensors are ignored, and the logits are the text model's."""
    from axon_b200.models.config import ModelConfig
    from axon_b200.models.families import FamilyModel
    text = dict(_HF["gemma3_text"]) if "gemma3_text" in globals().get("_HF", {}) else None
    if text is None:
        text = dict(model_type="gemma3_text", vocab_size=160, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                    head_dim=16, intermediate_size=96, sliding_window=8, query_pre_attn_scalar=16, rms_norm_eps=1e-6, rope_theta=10000.0,
                    rope_local_base_freq=10000.0, layer_types=["sliding_attention", "sliding_attention", "sliding_attention", "full_attention"],
                    max_position_embeddings=256, tie_word_embeddings=True)
    plain = FamilyModel(ModelConfig.from_hf_dict(text), device="cpu", dtype=torch.float32)
    plain.init_random(std=0.05, seed=2)
    wrapper = {"model_type": "gemma3", "text_config": {k: v for k, v in text.items() if k != "tie_word_embeddings"}, "tie_word_embeddings": True,
               "vision_config": {"model_type": "siglip_vision_model", "hidden_size": 32}, "eos_token_id": 1}
    cfg = ModelConfig.from_hf_dict(wrapper)
    assert cfg.model_type == "gemma3_text" and cfg.num_hidden_layers == 4 and cfg.eos_token_id == 1
    m = FamilyModel(cfg, device="cpu", dtype=torch.float32)
    sd = {k.replace("model.", "model.language_model.", 1): v for k, v in plain.state_dict().items()}
    sd["model.vision_tower.vision_model.embeddings.patch_embedding.weight"] = torch.zeros(32, 3, 4, 4)
    sd["model.multi_modal_projector.mm_input_projection_weight"] = torch.zeros(32, 64)
    m.load_state_dict(sd)
    ids = torch.randint(0, 150, (23,), dtype=torch.int32)
    assert torch.equal(m.logits(ids), plain.logits(ids))
    assert m.cfg.to_hf_dict()["model_type"] == "gemma3_text"          # what is exported is the text model
