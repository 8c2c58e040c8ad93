"""Driver plumbing: program -> batch transformation, advantages over multi-step programs, padding,
balancing, mini-batch splitting and the metrics reducers."""
import numpy as np
import pytest
import torch

from axon_b200.driver.components.advantage_component import compute_advantage_component, stepwise_advantage_broadcast
from axon_b200.driver.components.program_component import (ProgramProcessor, ProgramTransformConfig, compute_score_placement,
                                                           prepare_program_metadata)
from axon_b200.driver.driver_utils import (ValidationResult, balance_batch, convert_batch_dict_to_dataproto,
                                           pad_dataproto_to_world_size, process_mini_batch, split_mini_batches_by_programs,
                                           update_trainer)
from axon_b200.engine.state.program_state import ProgramState, Step
from axon_b200.protocol import DataProto
from axon_b200.utils import metrics as M
from axon_b200.utils.tokenizer import ByteTokenizer


def _program(gid, uid, reward, steps, step_rewards=None):
    ps = ProgramState(group_id=gid, uid=uid, session_id=uid, done=True, reward=reward)
    ps.training_steps = []
    for k, (n_prompt, n_resp, n_tail) in enumerate(steps):
        st = Step(uid=f"{uid}-s{k}", session_id=uid, order_idx=k)
        n = n_prompt + n_resp + n_tail
        st.tokens = list(range(10, 10 + n))
        st.masks = [0] * n_prompt + [1] * n_resp + [0] * n_tail
        st.logprobs = [0.0] * n_prompt + [-0.5] * n_resp + [0.0] * n_tail
        ps.training_steps.append(st)
    if step_rewards:
        ps.step_rewards = step_rewards
    return ps


def _batch():
    tok = ByteTokenizer()
    pp = ProgramProcessor(ProgramTransformConfig(max_seq_length=16, max_prompt_length=8), tok)
    progs = [_program("g0", "p0", 1.0, [(3, 4, 2), (5, 3, 0)]), _program("g0", "p1", 0.0, [(3, 5, 0)]),
             _program("g1", "p2", 1.0, [(2, 2, 0)]), _program("g1", "p3", 1.0, [(2, 6, 1)])]
    batch, metrics = pp.transform_programs(progs, uid_to_index={"g0": 7, "g1": 9})
    return batch, tok


def test_transform_programs_schema():
    batch, tok = _batch()
    b, nt = batch.batch, batch.non_tensor_batch
    assert b["input_ids"].shape == (5, 16) and torch.equal(b["input_ids"], b["responses"])
    assert b["attention_mask"].sum(-1).tolist() == [7, 8, 8, 4, 8]          # trailing masked tokens are cut
    assert b["response_mask"].sum(-1).tolist() == [4, 3, 5, 2, 6]
    assert b["input_ids"][0, 7:].eq(tok.pad_token_id).all()
    assert torch.equal(b["position_ids"][1, :8], torch.arange(8)) and b["position_ids"][1, 8:].eq(0).all()
    assert b["token_level_scores"][0, 6] == 1.0 and b["token_level_scores"][1, 7] == 1.0 and b["token_level_scores"][2].sum() == 0
    assert b["sampler_log_probs"][0, 3:7].eq(-0.5).all() and b["sampler_log_probs"][0, :3].eq(0).all()
    assert nt["uid"].tolist() == ["g0", "g0", "g0", "g1", "g1"] and nt["program_uids"].tolist() == ["p0", "p0", "p1", "p2", "p3"]
    assert nt["is_last_step"].tolist() == [False, True, True, True, True] and nt["num_program_steps"].tolist() == [2, 2, 1, 1, 1]
    assert nt["program_step_ids"][1] == "g0_step1" and nt["index"].tolist() == [7, 7, 7, 9, 9]
    assert b["num_program_tokens"].tolist() == [7, 7, 5, 2, 6] and b["num_program_steps"].tolist() == [2.0, 2.0, 1.0, 1.0, 1.0]
    assert not any(nt["is_padding"])


def test_step_rewards_and_score_placement():
    tok = ByteTokenizer()
    pp = ProgramProcessor(ProgramTransformConfig(max_seq_length=12, max_prompt_length=8), tok)
    batch, _ = pp.transform_programs([_program("g", "p", 0.25, [(2, 2, 0), (2, 3, 0)], step_rewards={0: 0.5})])
    assert batch.batch["token_level_scores"].sum(-1).tolist() == [0.5, 0.25]
    assert all(batch.non_tensor_batch["has_step_rewards"])
    am = torch.tensor([[1, 1, 1, 0], [1, 0, 0, 0], [0, 0, 0, 0]])
    s = compute_score_placement([[1.0, 2.0], 3.0], [2, 1], am)
    assert s[0, 2] == 1.0 and s[1, 0] == 2.0 and s[2].sum() == 0


def test_advantage_component_broadcasts_to_earlier_steps():
    batch, _ = _batch()
    metrics = {}
    out = compute_advantage_component(batch, {"advantage": "grpo", "advantage_args": {"norm_adv_by_std": True},
                                              "drop_zero_advantage_samples": True}, metrics)
    # group g1: both rewards 1 -> zero advantage -> dropped; group g0: p0 (+), p1 (-)
    assert metrics["batch/filtered_zero_adv_count"] == 2 and len(out) == 3
    uids = out.non_tensor_batch["program_uids"].tolist()
    adv = out.batch["advantages"]
    rows_p0 = [i for i, u in enumerate(uids) if u == "p0"]
    vals = [adv[i][out.batch["response_mask"][i].bool()] for i in rows_p0]
    assert all(torch.allclose(v, vals[0][:1].expand_as(v)) for v in vals) and vals[0][0] > 0
    assert torch.allclose(vals[0][0], vals[1][0])                # the earlier step got the last step's advantage
    assert adv[uids.index("p1")][out.batch["response_mask"][uids.index("p1")].bool()][0] < 0
    assert metrics["batch/solve/partial"] == 1 and metrics["batch/solve/all"] == 1 and metrics["batch/reward/mean"] == 0.75
    assert out.non_tensor_batch["pass_rate"].tolist() == [0.5, 0.5, 0.5]


def test_padding_balancing_and_mini_batches():
    batch, _ = _batch()
    batch.batch["advantages"] = torch.ones(5, 16) * batch.batch["response_mask"]
    padded = pad_dataproto_to_world_size(batch, [2, 4])
    assert len(padded) == 8 and padded.non_tensor_batch["is_padding"].tolist() == [False] * 5 + [True] * 3
    assert padded.batch["response_mask"][5:].sum() == 0 and len(set(padded.non_tensor_batch["uid"].tolist())) == 5
    assert padded.non_tensor_batch["index"][5:].tolist() == [-1, -1, -1]
    metrics = {}
    bal = balance_batch(padded, 2, metrics)
    halves = bal.chunk(2)
    sets = [set(h.non_tensor_batch["program_uids"][~h.non_tensor_batch["is_padding"].astype(bool)].tolist()) for h in halves]
    assert sets[0].isdisjoint(sets[1]) and sets[0] | sets[1] == {"p0", "p1", "p2", "p3"}      # programs stay whole
    assert len(halves[0]) == len(halves[1]) and any(k.endswith("balanced_max") or "minmax" in k or "max" in k for k in metrics)
    mbs = split_mini_batches_by_programs(batch, mini_batch_size=2, world_size=2)
    assert [len(m) % 2 for m in mbs] == [0, 0] and sum((~m.non_tensor_batch["is_padding"].astype(bool)).sum() for m in mbs) == 5
    process_mini_batch(mbs[0])
    b0 = mbs[0].batch
    real = ~mbs[0].non_tensor_batch["is_padding"].astype(bool)
    assert b0["valid_batch_size"][0] == real.sum() and b0["valid_token_count"][0] == b0["response_mask"].sum()
    assert b0["valid_program_count"][0] == 2 and torch.equal(b0["per_row_token_count"], b0["response_mask"].sum(-1))


def test_update_trainer_loop_and_lr_stepping():
    batch, _ = _batch()
    calls = []

    class Client:
        def forward_backward(self, mb, loss_fn, loss_fn_args):
            calls.append(("fb", len(mb), int(mb.batch["valid_token_count"][0])))
            return DataProto(meta_info={"metrics": {"actor/loss": 1.0, "actor/grad_norm/max": len(calls)}})

        def optim_step(self, step_lr):
            calls.append(("opt", step_lr))
            return DataProto(meta_info={"metrics": {"actor/lr": 0.1}})
    out = update_trainer(batch, Client(), "ppo", {}, epochs=2, mini_batch_size=2, world_size=1)
    assert [c[0] for c in calls] == ["fb", "opt"] * 4 and [c[1] for c in calls if c[0] == "opt"] == [False, False, False, True]
    assert out["actor/loss"] == 1.0 and out["actor/grad_norm/max"] == 7


def test_convert_batch_and_validation_result():
    bd = {"env_args": [{"q": 1}, {"q": 2}], "index": torch.tensor([4, 5])}

    class Sched:
        def get_temperature(self, s):
            return 1.0 + s
    dp = convert_batch_dict_to_dataproto(bd, global_steps=3, n_samples=2, temperature_scheduler=Sched(), temperature_config={"enable": True})
    assert len(dp) == 4 and dp.non_tensor_batch["uid"][0] == dp.non_tensor_batch["uid"][1] != dp.non_tensor_batch["uid"][2]
    assert dp.non_tensor_batch["index"].tolist() == [4, 4, 5, 5] and dp.meta_info["sample_params"]["temperature"] == 3.0
    vr = ValidationResult(n_samples=2)
    for r, u in ((0.0, "a"), (1.0, "a"), (0.0, "b"), (0.5, "b")):
        vr.add(r, u)
    m = vr.compute_metrics()
    assert m["val/pass@2"] == 0.5 and m["val/reward"] == 0.375


def test_metric_reducers_match_single_shard():
    batch, _ = _batch()
    n = len(batch)
    g = torch.Generator().manual_seed(0)
    batch.batch["token_level_rewards"] = batch.batch["token_level_scores"]
    batch.batch["advantages"] = torch.randn(n, 16, generator=g)
    batch.batch["returns"] = torch.randn(n, 16, generator=g)
    batch.batch["values"] = torch.randn(n, 16, generator=g)
    batch.batch["old_log_probs"] = -torch.rand(n, 16, generator=g)
    batch.batch["sampler_log_probs"] = batch.batch["old_log_probs"] + 0.01 * torch.randn(n, 16, generator=g)
    whole = M.compute_data_metrics(batch, use_critic=True)
    parts = [M.compute_data_metrics(batch.select_idxs(ix), use_critic=True, include_detail=True) for ix in ([0, 1, 2], [3, 4])]
    red = M.reduce_data_metrics(parts)
    for k in ("critic/score/mean", "critic/advantages/mean", "critic/returns/max", "response_length/mean", "prompt_length/min",
              "critic/values/mean"):
        assert abs(whole[k] - red[k]) < 1e-5, k
    mm_whole = M.aggregate_trainer_sampler_metrics([M.compute_trainer_sampler_mismatch_metrics(batch)])
    mm_parts = M.aggregate_trainer_sampler_metrics([M.compute_trainer_sampler_mismatch_metrics(batch.select_idxs(ix))
                                                    for ix in ([0, 1], [2, 3, 4])])
    for k, v in mm_whole.items():
        assert abs(v - mm_parts[k]) < 1e-6, k
    assert mm_whole["batch/sampler_actor_probs_pearson_corr"] > 0.99
    t = M.compute_timing_metrics(batch, {"gen": 2.0, "forward_backward": 1.0})
    assert abs(t["timing_per_token_ms/gen"] - 2000 / float(batch.batch["response_mask"].sum())) < 1e-9
    assert M.has_repetition("ab" * 8000) and not M.has_repetition("short")
    assert M.reduce_metrics({"x/max": [1, 3], "y_min": [2, 1], "minimum": [1, 3]}) == {"x/max": 3.0, "y_min": 2.0 if False else 1.0, "minimum": 2.0}
