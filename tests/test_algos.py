"""Loss / advantage registries: closed-form expectations on tiny tensors, and the invariant that the
multi-rank gradient equals the single-process gradient for every reduce mode."""
import itertools

import numpy as np
import pytest
import torch

from axon_b200.protocol import DataProto
from axon_b200.trainer.algos import (AdvantageFn, LossFn, agg_loss, compute_advantage, compute_loss_fn,
                                     register_advantage, register_loss)
from axon_b200.trainer.algos.advantages.advantage import _chunked_gae_core


def adv_batch(scores, uids, T=4, lens=None):
    B = len(scores)
    mask = torch.zeros(B, T)
    rew = torch.zeros(B, T)
    for i, s in enumerate(scores):
        n = lens[i] if lens else T
        mask[i, :n] = 1
        rew[i, n - 1] = s
    return DataProto.from_dict({"token_level_rewards": rew, "response_mask": mask},
                               {"uid": np.array(uids, dtype=object)})


def test_grpo_matches_hand_computation():
    d = adv_batch([1.0, 0.0, 0.0, 1.0, 5.0], ["a", "a", "a", "a", "solo"])
    compute_advantage(d, {"advantage": "grpo", "advantage_args": {}})
    a = d.batch["advantages"]
    s = torch.tensor([1.0, 0, 0, 1])
    exp = (s - s.mean()) / (s.std(unbiased=True) + 1e-6)
    assert torch.allclose(a[:4, 0], exp, atol=1e-5)
    assert torch.all(a[4] == 0)                       # singleton group -> zero
    assert torch.equal(d.batch["returns"], a)
    d2 = adv_batch([1.0, 0.0], ["a", "a"])
    compute_advantage(d2, {"advantage": AdvantageFn.GRPO, "advantage_args": {"norm_adv_by_std": False}})
    assert torch.allclose(d2.batch["advantages"][:, 0], torch.tensor([0.5, -0.5]))


def test_rloo_opo_gpg_passk_identity():
    d = adv_batch([3.0, 1.0, 2.0], ["g", "g", "g"])
    compute_advantage(d, {"advantage": "rloo"})
    assert torch.allclose(d.batch["advantages"][:, 0], torch.tensor([1.5, -1.5, 0.0]))
    compute_advantage(d, {"advantage": "loop"})
    d = adv_batch([1.0, 0.0], ["g", "g"], lens=[1, 3])
    compute_advantage(d, {"advantage": "opo"})
    assert torch.allclose(d.batch["advantages"][:, 0], torch.tensor([0.75, -0.25]))
    d = adv_batch([1.0, 0.0, 0.0, 0.0], ["g", "g", "h", "h"])
    compute_advantage(d, {"advantage": "gpg"})
    assert torch.allclose(d.batch["advantages"][:, 0], torch.tensor([2.0, -2.0, 0.0, 0.0]))
    d = adv_batch([3.0, 1.0, 2.0], ["g", "g", "g"])
    compute_advantage(d, {"advantage": "grpo_passk", "advantage_args": {"norm_adv_by_std": False}})
    assert torch.allclose(d.batch["advantages"][:, 0], torch.tensor([1.0, 0.0, 0.0]))
    with pytest.raises(ValueError):
        compute_advantage(adv_batch([1.0], ["x"]), {"advantage": "grpo_passk"})
    d = adv_batch([2.0], ["x"])
    compute_advantage(d, {"advantage": "identity", "advantage_args": {"clip_advantages": True}})
    assert d.batch["advantages"].max() == 1.0


def test_gae_and_chunked_gae_agree():
    torch.manual_seed(0)
    B, T = 3, 37
    r, v = torch.randn(B, T), torch.randn(B, T)
    mask = torch.ones(B, T)
    d = DataProto.from_dict({"token_level_rewards": r, "values": v, "response_mask": mask})
    compute_advantage(d, {"advantage": "gae", "advantage_args": {"gamma": 0.97, "lam": 0.9}})
    a1, r1 = d.batch["advantages"].clone(), d.batch["returns"].clone()
    compute_advantage(d, {"advantage": "chunked_gae", "advantage_args": {"gamma": 0.97, "lam": 0.9, "chunk_size": 8}})
    assert torch.allclose(a1, d.batch["advantages"], atol=1e-4) and torch.allclose(r1, d.batch["returns"], atol=1e-4)
    # direct recursion check of the scan core
    adv, _ = _chunked_gae_core(r, v, 0.97, 0.9, chunk_size=5)
    ref = torch.zeros(B, T)
    run = torch.zeros(B)
    for t in reversed(range(T)):
        nv = v[:, t + 1] if t + 1 < T else torch.zeros(B)
        run = r[:, t] + 0.97 * nv - v[:, t] + 0.97 * 0.9 * run
        ref[:, t] = run
    assert torch.allclose(adv, ref, atol=1e-4)
    # non-contiguous mask is compacted
    mask2 = mask.clone()
    mask2[:, 5:9] = 0
    d2 = DataProto.from_dict({"token_level_rewards": r * mask2, "values": v, "response_mask": mask2})
    compute_advantage(d2, {"advantage": "gae", "advantage_args": {}})
    g = d2.batch["advantages"].clone()
    compute_advantage(d2, {"advantage": "chunked_gae", "advantage_args": {}})
    assert torch.allclose(g * mask2, d2.batch["advantages"] * mask2, atol=1e-4)


def test_rpp_remax_kimi():
    d = adv_batch([1.0, 0.0], ["a", "a"], T=3)
    compute_advantage(d, {"advantage": "reinforce_plus_plus"})
    assert torch.allclose(d.batch["returns"], torch.tensor([[1.0, 1, 1], [0, 0, 0]]))
    compute_advantage(d, {"advantage": "reinforce_plus_plus_baseline"})
    assert abs(d.batch["advantages"].mean().item()) < 1e-6
    d.batch["reward_baselines"] = torch.tensor([0.5, 0.5])
    compute_advantage(d, {"advantage": "remax"})
    assert torch.allclose(d.batch["advantages"][0], torch.tensor([0.5, 0.5, 0.5]))
    d = adv_batch([1.0, 1.0, 0.0], ["a", "a", "a"], T=6, lens=[2, 6, 4])
    d.meta_info["global_steps"] = 10
    compute_advantage(d, {"advantage": "kimi_k1_5", "advantage_args": {"length_coef": 1.0, "norm_adv_by_std": False}})
    shaped = torch.tensor([1.5, 0.5, 0.0])      # +0.5 short correct, -0.5 long correct, min(0, 0)=0 wrong
    assert torch.allclose(d.batch["advantages"][:, 0], shaped - shaped.mean(), atol=1e-5)


def loss_batch(B=4, T=6, seed=0):
    g = torch.Generator().manual_seed(seed)
    old = -torch.rand(B, T, generator=g)
    new = (old + 0.3 * torch.randn(B, T, generator=g)).requires_grad_(True)
    adv = torch.randn(B, T, generator=g)
    mask = (torch.rand(B, T, generator=g) > 0.3).float()
    mask[:, 0] = 1
    return DataProto.from_dict({"old_log_probs": old, "log_probs": new, "advantages": adv, "response_mask": mask})


def test_ppo_closed_form_and_metrics():
    d = loss_batch()
    b = d.batch
    loss, m = compute_loss_fn(d, "ppo", {"clip_ratio": 0.2, "clip_ratio_high": 0.3})
    ratio = torch.exp((b["log_probs"] - b["old_log_probs"]).clamp(-20, 20))
    l1, l2 = -b["advantages"] * ratio, -b["advantages"] * ratio.clamp(0.8, 1.3)
    pess = torch.maximum(l1, l2)
    exp = torch.where(b["advantages"] < 0, torch.minimum(-b["advantages"] * 3.0, pess), pess)
    exp = (exp * b["response_mask"]).sum() / b["response_mask"].sum()
    assert torch.allclose(loss, exp, atol=1e-6)
    assert set(m) == {"pg_clipfrac", "ppo_kl", "pg_clipfrac_lower"}
    loss.backward()
    assert torch.isfinite(b["log_probs"].grad).all()


@pytest.mark.parametrize("name", [e.value for e in LossFn if e != LossFn.VALUE])
def test_all_policy_losses_run_and_on_policy_gradient(name):
    d = loss_batch()
    loss, metrics = compute_loss_fn(d, name, {})
    loss.backward()
    assert torch.isfinite(loss) and all(np.isfinite(v) for v in metrics.values())
    # on-policy (ratio 1): clipped surrogates reduce to -A * grad log pi under token-mean
    if name in ("ppo", "reinforce", "gpg", "cispo", "kl_cov"):
        d2 = loss_batch()
        d2.batch["log_probs"] = d2.batch["old_log_probs"].clone().requires_grad_(True)
        l2, _ = compute_loss_fn(d2, name, {})
        l2.backward()
        exp = -(d2.batch["advantages"] * d2.batch["response_mask"]) / d2.batch["response_mask"].sum()
        got = d2.batch["log_probs"].grad
        if name == "kl_cov":   # one token carries the extra |log ratio| term whose subgradient at 0 is 0
            assert torch.allclose(got, exp, atol=1e-6)
        else:
            assert torch.allclose(got, exp, atol=1e-6)


def test_value_loss_and_sampler_correction():
    B, T = 2, 3
    d = DataProto.from_dict({"vpreds": torch.tensor([[1.0, 2, 3], [0, 0, 0]]), "values": torch.zeros(B, T),
                             "returns": torch.ones(B, T), "response_mask": torch.ones(B, T)})
    loss, m = compute_loss_fn(d, "value", {"cliprange_value": 0.5})
    l1 = (d.batch["vpreds"] - 1) ** 2
    l2 = (d.batch["vpreds"].clamp(-0.5, 0.5) - 1) ** 2
    assert torch.allclose(loss, 0.5 * torch.maximum(l1, l2).mean())
    d = loss_batch()
    d.batch["sampler_log_probs"] = d.batch["old_log_probs"] - torch.tensor(1.0)   # ratio e > 2 -> truncated
    _, m = compute_loss_fn(d, "ppo", {"sampler_is": "token", "sampler_is_threshold": 2.0, "sampler_rs": "token",
                                      "sampler_rs_threshold": 2.0, "sampler_token_veto_threshold": 1e-4})
    assert "sampler_is_weights" in d.batch and d.batch["sampler_is_weights"].max() <= 2.0
    assert d.batch["response_mask"].sum() == 0 and m["sampler_corr/sampler_rs_masked_fraction"] == 1.0


def test_agg_loss_modes():
    mat = torch.arange(12.0).view(3, 4)
    mask = torch.tensor([[1.0, 1, 0, 0], [1, 1, 1, 1], [0, 0, 0, 0]])
    assert agg_loss(mat, mask, token_reduce="sum", batch_reduce="token-mean") == (1 + 4 + 5 + 6 + 7) / 6
    assert agg_loss(mat, mask, token_reduce="mean", batch_reduce="step-mean") == (0.5 + 5.5) / 2
    assert agg_loss(mat, mask, token_reduce="mean-norm", batch_reduce="step-mean", valid_batch_size=4) == (0.25 + 5.5) / 4
    npt, nps = torch.tensor([6.0, 6, 1]), torch.tensor([2.0, 2, 1])
    v = agg_loss(mat, mask, token_reduce="mean-program", batch_reduce="program-mean", num_program_tokens=npt,
                 num_program_steps=nps, valid_program_count=1)
    assert torch.isclose(v, torch.tensor((1 / 6 + 22 / 6) / 2))
    with pytest.raises(ValueError):
        agg_loss(mat, mask, token_reduce="bogus")


@pytest.mark.parametrize("token_reduce,batch_reduce,dp", list(itertools.product(
    ["sum", "mean", "mean-norm", "mean-program"], ["token-mean", "step-mean", "program-mean"], [2, 4])))
def test_multi_rank_gradient_equals_single_process(token_reduce, batch_reduce, dp):
    """Simulate ``dp`` data-parallel ranks on CPU. With mini-batch-global valid counts, SUM-reduced rank
    gradients (or AVG-reduced ones pre-multiplied by dp, the FSDP convention) equal the 1-process gradient."""
    torch.manual_seed(1)
    B, T = 8, 5
    theta = torch.randn(T, requires_grad=True)
    feats = torch.randn(B, T)
    mask = (torch.rand(B, T) > 0.4).float()
    mask[:, 0] = 1
    prog = torch.tensor([0, 0, 1, 2, 2, 2, 3, 4])
    n_prog_tokens = torch.stack([mask[prog == p].sum() for p in prog])
    n_prog_steps = torch.stack([(prog == p).sum() for p in prog]).float()
    counts = dict(valid_token_count=mask.sum(), valid_batch_size=torch.tensor(float(B)),
                  valid_program_count=torch.tensor(float(len(prog.unique()))))

    def loss_of(rows):
        lm = feats[rows] * theta
        return agg_loss(lm, mask[rows], token_reduce=token_reduce, batch_reduce=batch_reduce,
                        num_program_tokens=n_prog_tokens[rows], num_program_steps=n_prog_steps[rows], **counts)

    full, = torch.autograd.grad(loss_of(torch.arange(B)), theta)
    shards = torch.arange(B).chunk(dp)
    summed = sum(torch.autograd.grad(loss_of(r), theta)[0] for r in shards)
    assert torch.allclose(summed, full, atol=1e-6)
    averaged = sum(torch.autograd.grad(loss_of(r) * dp, theta)[0] for r in shards) / dp
    assert torch.allclose(averaged, full, atol=1e-6)


def test_registration_of_custom_plugins():
    @register_loss("my_loss")
    def my_loss(data, config):
        return (data.batch["log_probs"] * 0).sum(), {"x": 1.0}

    @register_advantage("my_adv")
    def my_adv(data, config):
        z = torch.zeros_like(data.batch["response_mask"])
        return z, z

    assert compute_loss_fn(loss_batch(), "my_loss")[1] == {"x": 1.0}
    d = adv_batch([1.0], ["a"])
    compute_advantage(d, {"advantage": "my_adv"})
    with pytest.raises(ValueError):
        compute_loss_fn(loss_batch(), "nope")
