"""One colocated RL step end to end (rollout -> batch -> advantages -> train -> hand-over)."""
import numpy as np
import pytest
import torch

from axon_b200.driver.colocated import ColocatedRLRunner, RLStepConfig, build_training_batch
from axon_b200.models.config import tiny_gpu, tiny_qwen3
from axon_b200.models.dense import DenseModel
from axon_b200.sampler.params import TokenOutput
from axon_b200.trainer.policy import OptimConfig


def test_training_batch_schema():
    outs = [TokenOutput(token_ids=[5, 6, 7], logprobs=[-1.0, -2.0, -3.0]), TokenOutput(token_ids=[9], logprobs=[-0.5])]
    d = build_training_batch([[1, 2], [3, 4, 8]], outs, [1.0, 0.0], ["g", "g"], pad_id=0, max_len=16)
    b = d.batch
    assert b["input_ids"].tolist() == [[1, 2, 5, 6, 7], [3, 4, 8, 9, 0]]
    assert torch.equal(b["responses"], b["input_ids"])
    assert b["attention_mask"].tolist() == [[1, 1, 1, 1, 1], [1, 1, 1, 1, 0]]
    assert b["response_mask"].tolist() == [[0, 0, 1, 1, 1], [0, 0, 0, 1, 0]]
    assert b["token_level_scores"][0].tolist() == [0, 0, 0, 0, 1.0]
    assert b["sampler_log_probs"][1].tolist() == [0, 0, 0, -0.5, 0]
    assert d.non_tensor_batch["uid"].tolist() == ["g", "g"]


def _run(cfg, device, dtype, lr):
    model = DenseModel(cfg, device=device, dtype=dtype)
    model.params.init_random(0.05, seed=0)
    rl = RLStepConfig(n_samples=4, max_prompt_length=16, max_response_length=140, mini_batch_size=2,
                      max_token_len_per_gpu=512, max_num_seqs=8, optim=OptimConfig(lr=lr, weight_decay=0.0))
    runner = ColocatedRLRunner(model, rl, seed=0)
    prompts = torch.randint(2, cfg.vocab_size, (3, 16), dtype=torch.int32)
    caps = np.array([5, 130, 20, 9] * 3)
    rewards = np.array([1, 0, 0, 1, 0, 0, 1, 1, 0, 1, 0, 0], dtype=np.float32)
    w0 = model.params.flat.clone()
    out = runner.step(prompts, response_caps=caps, rewards=rewards)
    assert out["sequences"] == 12 and out["response_tokens"] == int(caps.sum())
    assert np.isfinite(out["loss"]) and out["grad_norm"] > 0
    assert not torch.equal(w0, model.params.flat)
    assert runner.policy.opt_step == 2          # 3 prompts, 2 per mini-batch
    return out, runner


def test_rl_step_cpu():
    out, runner = _run(tiny_qwen3(), "cpu", torch.float32, 1e-3)
    assert out["sampler_probs_diff_mean"] < 1e-5       # trainer and sampler share kernels and weights
    out2 = runner.step(torch.randint(2, 4096, (2, 16), dtype=torch.int32))   # EOS-terminated path, default rewards
    assert out2["sequences"] == 8


@pytest.mark.gpu
def test_rl_step_gpu():
    out, _ = _run(tiny_gpu(), "cuda", torch.bfloat16, 1e-4)
    from axon_b200.ops import _common as C
    C.check_status()
    assert out["sampler_probs_diff_mean"] < 0.02
