"""PolicyEngine: padded DataProto -> packed micro-batches -> loss registry -> explicit backward -> AdamW."""
import copy

import numpy as np
import pytest
import torch

from axon_b200.models.config import tiny_gpu, tiny_qwen3
from axon_b200.models.dense import DenseModel
from axon_b200.protocol import DataProto
from axon_b200.trainer.policy import OptimConfig, PolicyEngine, lr_at


def make_batch(cfg, B=6, T=40, seed=0):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(8, T + 1, (B,), generator=g)
    ids = torch.randint(2, cfg.vocab_size, (B, T), generator=g)
    att = (torch.arange(T)[None] < lens[:, None]).long()
    ids = ids * att
    resp = att.clone().float()
    resp[:, :4] = 0
    adv = torch.randn(B, 1, generator=g).expand(B, T) * resp
    d = DataProto.from_dict({"input_ids": ids, "attention_mask": att, "response_mask": resp, "advantages": adv},
                            {"uid": np.arange(B).astype(object)})
    d.batch["valid_token_count"] = resp.sum().expand(B).clone()
    return d


def _engine(cfg, device, dtype, max_tokens, lr=1e-2):
    m = DenseModel(cfg, device=device, dtype=dtype)
    m.params.init_random(0.05, seed=2)
    return PolicyEngine(m, OptimConfig(lr=lr, weight_decay=0.0, grad_clip=1.0), max_token_len_per_gpu=max_tokens)


def test_forward_convention_and_microbatch_invariance_cpu():
    cfg = tiny_qwen3()
    d = make_batch(cfg)
    e1 = _engine(cfg, "cpu", torch.float32, 10_000)
    e2 = _engine(cfg, "cpu", torch.float32, 64)      # forces several micro-batches
    o1, o2 = e1.forward(d), e2.forward(d)
    assert torch.allclose(o1.batch["log_probs"], o2.batch["log_probs"], atol=1e-5)
    lp = o1.batch["log_probs"]
    att = d.batch["attention_mask"]
    assert torch.all(lp[:, 0] == 0) and torch.all(lp[att == 0] == 0) and torch.all(lp[:, 1:][att[:, 1:] == 1] < 0)
    # gradient accumulated over micro-batches equals the single-batch gradient
    d.batch["old_log_probs"] = lp.clone()
    e1.forward_backward(copy.deepcopy(d), "ppo", {})
    e2.forward_backward(copy.deepcopy(d), "ppo", {})
    g1, g2 = e1.model.params.grad_flat, e2.model.params.grad_flat
    assert torch.allclose(g1, g2, atol=1e-6) and g1.abs().sum() > 0


def test_training_improves_objective_cpu():
    cfg = tiny_qwen3()
    d = make_batch(cfg)
    e = _engine(cfg, "cpu", torch.float32, 128)
    old = e.forward(d).batch["log_probs"]
    d.batch["old_log_probs"] = old

    def objective():
        lp = e.forward(d).batch["log_probs"]
        return ((lp - old) * d.batch["advantages"] * d.batch["response_mask"]).sum().item()

    before = objective()
    for _ in range(3):
        m = e.forward_backward(copy.deepcopy(d), "ppo", {"entropy_coef": 0.001})
        s = e.optim_step()
        assert np.isfinite(s["grad_norm"]) and s["skipped"] == 0.0 and "entropy_loss" in m
    assert objective() > before + 1e-3
    assert e.opt_step == 3 and torch.all(e.model.params.grad_flat == 0)


def test_lr_schedule():
    c = OptimConfig(lr=1.0, warmup_steps=4, total_steps=12, schedule="cosine", min_lr_ratio=0.1)
    assert lr_at(c, 2) == 0.5 and lr_at(c, 4) == 1.0 and abs(lr_at(c, 12) - 0.1) < 1e-9
    assert lr_at(OptimConfig(lr=3.0), 100) == 3.0


@pytest.mark.gpu
def test_policy_engine_gpu_step():
    cfg = tiny_gpu()
    d = make_batch(cfg, B=8, T=300)
    e = _engine(cfg, "cuda", torch.bfloat16, 700, lr=1e-3)
    old = e.forward(d).batch["log_probs"]
    d.batch["old_log_probs"] = old.cpu()
    w0 = e.model.params.flat.clone()
    m = e.forward_backward(copy.deepcopy(d), "ppo", {})
    s = e.optim_step()
    from axon_b200.ops import _common as C
    C.check_status()
    assert np.isfinite(s["grad_norm"]) and s["grad_norm"] > 0 and len(m["loss"]) >= 2
    assert not torch.equal(w0, e.model.params.flat)
    e.offload_optimizer()
    assert e.master is None
    e.load_optimizer()
    assert e.master is not None and e.master.is_cuda


def test_lr_schedules_and_both_config_forms():
    """Warm-up from a start value, cosine to the larger of the two floors, warm-up / stable / decay, and the two
    accepted spellings of the schedule block."""
    from axon_b200.trainer.policy import OptimConfig, lr_at, schedule_from_config
    c = OptimConfig(lr=1.0, warmup_steps=4, warmup_init=0.2, total_steps=24, schedule="cosine", min_lr_ratio=0.1, min_lr=0.05)
    assert abs(lr_at(c, 2) - 0.6) < 1e-9 and abs(lr_at(c, 4) - 1.0) < 1e-9
    assert abs(lr_at(c, 14) - (0.1 + 0.9 * 0.5)) < 1e-9 and abs(lr_at(c, 24) - 0.1) < 1e-9 and abs(lr_at(c, 99) - 0.1) < 1e-9
    w = OptimConfig(lr=1.0, warmup_steps=2, total_steps=20, schedule="wsd", wsd_decay_steps=10, wsd_decay_style="linear")
    assert lr_at(w, 10) == 1.0 and abs(lr_at(w, 15) - 0.5) < 1e-9 and abs(lr_at(w, 20)) < 1e-9
    e = OptimConfig(lr=1.0, total_steps=10, schedule="wsd", wsd_decay_steps=10, wsd_decay_style="exponential")
    assert lr_at(e, 0) == 1.0 and 0 < lr_at(e, 5) < 0.5 and abs(lr_at(e, 10)) < 1e-9
    a = schedule_from_config("cosine", {"total_training_steps": 100, "lr_warmup_steps": -1, "lr_warmup_steps_ratio": 0.1,
                                        "min_lr_ratio": 0.2, "num_cycles": 0.5}, 1e-5)
    assert a["schedule"] == "cosine" and a["warmup_steps"] == 10 and a["total_steps"] == 100 and a["min_lr_ratio"] == 0.2
    b = schedule_from_config({"type": "cosine", "warmup_ratio": 0.1, "total_steps": 100, "min_lr_ratio": 0.2}, None, 1e-5)
    assert (b["schedule"], b["warmup_steps"], b["total_steps"]) == ("cosine", 10, 100)
    assert schedule_from_config("constant", {"total_training_steps": -1}, 1e-5, fallback_total=7)["total_steps"] == 7
