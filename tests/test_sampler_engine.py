"""Generation engine: sampler log-probs agree with the trainer's forward on the same tokens,
continuous batching with a tight page pool, pause/sleep semantics."""
import pytest
import torch

from axon_b200.models.config import tiny_gpu, tiny_qwen3
from axon_b200.models.dense import DenseModel, PackedBatch
from axon_b200.sampler.engine import GenerationEngine
from axon_b200.sampler.params import SamplingParams


def _make(cfg, device, dtype):
    m = DenseModel(cfg, device=device, dtype=dtype)
    m.params.init_random(std=0.08, seed=3)
    return m


def _trainer_logprobs(model, prompt, out_ids, temperature):
    seq = torch.tensor(prompt + out_ids)
    batch = PackedBatch.from_sequences([seq], model.device)
    lp, _ = model.forward(batch, temperature)
    return lp[len(prompt) - 1: len(prompt) - 1 + len(out_ids)].float().cpu()


def _agreement(cfg, device, dtype, tol):
    torch.manual_seed(0)
    model = _make(cfg, device, dtype)
    eng = GenerationEngine(model, num_pages=24, max_num_seqs=8)
    prompts = [torch.randint(2, cfg.vocab_size, (n,)).tolist() for n in (5, 130, 47, 260, 9)]
    sp = SamplingParams(temperature=0.8, max_tokens=40, ignore_eos=True)
    outs = eng.generate(prompts, sp)
    assert eng.cache.num_free() == 24
    worst = 0.0
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 40 and o.finish_reason == "length"
        ref = _trainer_logprobs(model, p, o.token_ids, 0.8)
        worst = max(worst, (torch.tensor(o.logprobs) - ref).abs().max().item())
    assert worst < tol, worst
    return eng, model


def test_sampler_trainer_agreement_cpu():
    _agreement(tiny_qwen3(), "cpu", torch.float32, 1e-4)


@pytest.mark.gpu
def test_sampler_trainer_agreement_gpu():
    eng, _ = _agreement(tiny_gpu(), "cuda", torch.bfloat16, 0.12)
    from axon_b200.ops import _common as C
    C.check_status()


def test_preemption_eos_and_pause_cpu():
    cfg = tiny_qwen3()
    model = _make(cfg, "cpu", torch.float32)
    eng = GenerationEngine(model, num_pages=5, max_num_seqs=4)   # tight pool forces queueing / preemption
    prompts = [torch.randint(2, cfg.vocab_size, (120,)).tolist() for _ in range(4)]
    sp = SamplingParams(temperature=0.0, max_tokens=20)
    outs = eng.generate(prompts, sp)
    assert all(o.finish_reason in ("length", "stop") for o in outs)
    assert eng.cache.num_free() == 5
    # greedy decoding is reproducible and independent of batching
    eng2 = GenerationEngine(model, num_pages=32, max_num_seqs=8)
    outs2 = eng2.generate(prompts, sp)
    assert [o.token_ids for o in outs] == [o.token_ids for o in outs2]
    # hold: nothing advances; reset: running sequences come back aborted
    for p in prompts[:2]:
        eng2.add_request(p, SamplingParams(temperature=1.0, max_tokens=50, ignore_eos=True))
    eng2.step()
    n_before = [len(s.out.token_ids) for s in eng2.running]
    eng2.pause("hold")
    eng2.step()
    assert [len(s.out.token_ids) for s in eng2.running] == n_before
    eng2.pause("reset")
    assert not eng2.running and sum(o.finish_reason == "abort" for o in eng2.finished.values()) == 2
    eng2.sleep()
    assert eng2.cache is None
    eng2.wake_up()
    eng2.resume()
    eng2.finished.clear()
    out = eng2.generate([prompts[0]], sp)[0]
    assert out.token_ids == outs[0].token_ids


def _shared_prompt_run(device, dtype, share, cascade=False):
    torch.manual_seed(0)
    cfg = tiny_qwen3() if device == "cpu" else tiny_gpu()
    model = _make(cfg, device, dtype)
    eng = GenerationEngine(model, num_pages=40, max_num_seqs=16)
    eng.share_prompts = share
    eng.cascade_attention, eng.cascade_min_batch = cascade, 1
    g = torch.Generator().manual_seed(5)
    base = [torch.randint(2, cfg.vocab_size, (n,), generator=g).tolist() for n in (256, 150, 7)]   # full pages only / partial tail / no full page
    prompts = [p for p in base for _ in range(4)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.9, max_tokens=24, ignore_eos=True))
    assert eng.cache.num_free() == 40 and all(r == 0 for r in eng.cache.ref)
    return eng, [(o.token_ids, o.logprobs) for o in outs]


def _check_shared(device, dtype, tol, exact=True):
    eng_a, a = _shared_prompt_run(device, dtype, True)
    eng_b, b = _shared_prompt_run(device, dtype, False)
    assert eng_a.stats.get("shared_prompt_seqs", 0) == 9 and eng_b.stats.get("shared_prompt_seqs", 0) == 0
    assert eng_a.stats["prefill_tokens"] == 256 + 150 + 7 and eng_b.stats["prefill_tokens"] == 4 * (256 + 150 + 7)
    same = 0
    for (ta, la), (tb, lb) in zip(a, b):
        if exact:
            assert ta == tb
            assert max(abs(x - y) for x, y in zip(la, lb)) < tol
        same += int(ta == tb)
    # bf16 on the GPU: a different prefill batch may pick a different GEMM split, so a sampled token can flip
    assert same >= (len(a) if exact else len(a) - 3), same
    # samples of one prompt differ from each other (independent random streams)
    assert len({tuple(t) for t, _ in a[:4]}) > 1


def test_samples_of_one_prompt_share_its_pages_cpu():
    _check_shared("cpu", torch.float32, 1e-5)


@pytest.mark.gpu
def test_samples_of_one_prompt_share_its_pages_gpu():
    _check_shared("cuda", torch.bfloat16, 1e-5, exact=False)


@pytest.mark.gpu
def test_shared_prefix_attention_in_the_decode_graph_gpu():
    """Decode graphs with the shared-prefix attention kernel give the same samples as the plain kernel."""
    _, a = _shared_prompt_run("cuda", torch.bfloat16, True, cascade=True)
    _, b = _shared_prompt_run("cuda", torch.bfloat16, True, cascade=False)
    same = sum(int(ta == tb) for (ta, _), (tb, _) in zip(a, b))
    assert same >= len(a) - 3, same
    first = max(abs(la[0] - lb[0]) for (_, la), (_, lb) in zip(a, b))
    assert first < 0.05, first


def _routing_capture_roundtrip(device, dtype, tol):
    """The sampler records every token's routed experts; a teacher-forced trainer forward that REPLAYS the record
    reproduces the sampler's log-probs, and (deterministic CPU arithmetic) recomputes the very same experts."""
    from axon_b200.models.config import get_config
    from axon_b200.models.moe import MoEModel
    cfg = get_config("tiny-moe" if device == "cpu" else "tiny-moe-gpu")
    torch.manual_seed(1)
    model = MoEModel(cfg, device=device, dtype=dtype)
    model.params.init_random(std=0.08, seed=4)
    eng = GenerationEngine(model, num_pages=32, max_num_seqs=8)
    eng.enable_routing_capture(True)
    p_shared = torch.randint(2, cfg.vocab_size, (140,)).tolist()
    prompts = [p_shared, p_shared, torch.randint(2, cfg.vocab_size, (9,)).tolist()]       # two samples share a prompt
    outs = eng.generate(prompts, SamplingParams(temperature=0.9, max_tokens=12, ignore_eos=True))
    L, k, E = cfg.num_hidden_layers, cfg.num_experts_per_tok, cfg.num_experts
    for p, o in zip(prompts, outs):
        rm = o.moe_routermap
        n = len(p) + len(o.token_ids)
        assert rm.shape == (n, L, k) and str(rm.dtype) == "int16"
        assert (rm[-1] == -1).all() and (rm[:-1] >= 0).all() and (rm[:-1] < E).all()
        seq = torch.tensor(p + o.token_ids)
        batch = PackedBatch.from_sequences([seq], model.device)
        batch.routermap = torch.from_numpy(rm.astype("int64")).to(model.device)          # -1 rows fall back to computed routing
        lp, _ = model.forward(batch, 0.9)
        ref = lp[len(p) - 1: len(p) - 1 + len(o.token_ids)].float().cpu()
        assert (torch.tensor(o.logprobs) - ref).abs().max().item() < tol
        if device == "cpu":
            model.capture_routing, model.last_routing = True, None
            plain = PackedBatch.from_sequences([seq], model.device)
            model.forward(plain, 0.9)
            again = torch.stack(model.last_routing, 1)[: n - 1].sort(-1).values
            model.last_routing = None
            assert torch.equal(again, torch.from_numpy(rm[: n - 1].astype("int64")).sort(-1).values)
    assert (outs[0].moe_routermap[: len(p_shared)] == outs[1].moe_routermap[: len(p_shared)]).all()
    eng.enable_routing_capture(False)
    assert eng.generate([prompts[2]], SamplingParams(max_tokens=3, ignore_eos=True))[0].moe_routermap is None


def test_routed_experts_capture_and_replay_cpu():
    _routing_capture_roundtrip("cpu", torch.float32, 1e-4)


@pytest.mark.gpu
def test_routed_experts_capture_and_replay_gpu():
    _routing_capture_roundtrip("cuda", torch.bfloat16, 0.15)
    from axon_b200.ops import _common as C
    C.check_status()


def _same_generation(want, got, tol, exact):
    for a, b in zip(want, got):
        if exact:
            assert a.token_ids == b.token_ids
            assert (torch.tensor(a.logprobs) - torch.tensor(b.logprobs)).abs().max().item() < tol
        else:           # bf16: another prefill shape may round a near-tie the other way; the first step must still agree
            assert abs(a.logprobs[0] - b.logprobs[0]) < tol
    assert sum(int(a.token_ids == b.token_ids) for a, b in zip(want, got)) >= (len(want) if exact else len(want) - 1)


def _prefix_and_chunk_run(device, dtype, tol, exact=True):
    """A second turn that extends an earlier request's text reuses its pages; a prompt longer than the token budget is
    prefilled in chunks. Both give the tokens and log-probs of the plain engine (greedy sampling)."""
    cfg = tiny_qwen3() if device == "cpu" else tiny_gpu()
    model = _make(cfg, device, dtype)
    g = torch.Generator().manual_seed(5)
    first = [torch.randint(2, cfg.vocab_size, (n,), generator=g).tolist() for n in (300, 140)]
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)

    cached = GenerationEngine(model, num_pages=40, max_num_seqs=8)
    cached.enable_prefix_caching = True
    turn1 = cached.generate(first, sp)
    second = [p + o.token_ids + torch.randint(2, cfg.vocab_size, (37,), generator=g).tolist() for p, o in zip(first, turn1)]
    plain = GenerationEngine(model, num_pages=40, max_num_seqs=8)
    _same_generation(plain.generate(first, sp), turn1, tol, exact)
    want = plain.generate(second, sp)
    held = 40 - cached.cache.num_free()
    assert held == (300 + 24 - 1) // 128 + (140 + 24 - 1) // 128            # full pages of the finished turns stay cached
    got = cached.generate(second, sp)
    assert cached.stats["prefix_cache_hit_tokens"] == 2 * 128 + 1 * 128
    _same_generation(want, got, tol, exact)
    # a weight update (sleep / wake-up, or an explicit reset) drops every cached page
    cached.reset_prefix_cache()
    assert cached.cache.num_free() == 40

    # eviction: a small pool keeps serving by dropping the least recently used cached pages
    small = GenerationEngine(model, num_pages=6, max_num_seqs=2)
    small.enable_prefix_caching = True
    for p in first + second:
        out = small.generate([p], sp)[0]
        assert len(out.token_ids) == 24
    small.reset_prefix_cache()
    assert small.cache.num_free() == 6

    chunked = GenerationEngine(model, num_pages=40, max_num_seqs=8, max_num_batched_tokens=128)
    got = chunked.generate(second, sp)
    assert chunked.stats["prefill_tokens"] == sum(len(p) for p in second)
    _same_generation(want, got, tol, exact)
    assert chunked.cache.num_free() == 40


def test_prefix_caching_and_chunked_prefill_cpu():
    _prefix_and_chunk_run("cpu", torch.float32, 1e-4)


@pytest.mark.gpu
def test_prefix_caching_and_chunked_prefill_gpu():
    _prefix_and_chunk_run("cuda", torch.bfloat16, 0.12, exact=False)
    from axon_b200.ops import _common as C
    C.check_status()


def _speculative_run(device, dtype, exact):
    """N-gram speculative decoding returns what plain decoding returns (greedy and sampled), accepts drafts on
    repetitive text and reports how many."""
    cfg = tiny_qwen3() if device == "cpu" else tiny_gpu()
    model = _make(cfg, device, dtype)
    g = torch.Generator().manual_seed(7)
    motif = torch.randint(2, cfg.vocab_size, (12,), generator=g).tolist()
    prompts = [motif * 6, torch.randint(2, cfg.vocab_size, (50,), generator=g).tolist(), (motif[:5] * 9)[:40]]
    for temp in (0.0, 0.7):
        sp = SamplingParams(temperature=temp, max_tokens=40, ignore_eos=True)
        plain = GenerationEngine(model, num_pages=24, max_num_seqs=8, seed=3)
        want = plain.generate(prompts, sp)
        spec = GenerationEngine(model, num_pages=24, max_num_seqs=8, seed=3)
        spec.speculative_ngram = 4
        got = spec.generate(prompts, sp)
        assert spec.cache.num_free() == 24
        assert spec.stats["spec_draft_tokens"] > 0 and spec.stats["spec_verify_steps"] > 0
        for a, b in zip(want, got):
            assert len(b.token_ids) == 40 and len(b.logprobs) == 40
            if exact:
                assert a.token_ids == b.token_ids, temp
                assert (torch.tensor(a.logprobs) - torch.tensor(b.logprobs)).abs().max().item() < 1e-4
        assert 0 <= spec.stats["spec_accepted_tokens"] <= spec.stats["spec_draft_tokens"]
        # every request reports its own rounds; together they are the engine's totals, and plain decoding reports none
        per = [o.spec_decode_metrics for o in got if o.spec_decode_metrics is not None]
        assert per and all(o.spec_decode_metrics is None for o in want)
        assert sum(m.num_draft_tokens for m in per) == spec.stats["spec_draft_tokens"]
        assert sum(m.num_accepted_tokens for m in per) == spec.stats["spec_accepted_tokens"]
        assert all(m.num_completions > 0 and 0.0 <= m.accept_rate <= 1.0 and m.accept_length >= 1.0 for m in per)
    return spec


def test_ngram_speculative_decoding_matches_plain_decoding_cpu():
    _speculative_run("cpu", torch.float32, True)


@pytest.mark.gpu
def test_ngram_speculative_decoding_gpu():
    _speculative_run("cuda", torch.bfloat16, False)
    from axon_b200.ops import _common as C
    C.check_status()
