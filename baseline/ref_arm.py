"""Reference arm of ``bench.py`` (``--impl reference``): the same RL step on the libraries the reference calls.

The reference's own entry point (``python -m axon.driver.train_agent_ppo``) cannot start in this image: it
imports ray, hydra, omegaconf and tensordict, none of which is installed or in the wheelhouse, and its sampler
needs a patched vLLM 0.19 build. What CAN run is every library call its colocated FSDP recipe for Qwen3-8B makes
(recipes/math/train_math_qwen_8b.sh, axon/driver/sync_ppo.py:285-454), so this arm is "library-equivalent":

    rollout      vLLM (the stock 0.22 of the image), one engine per GPU, sleep mode, in-process worker
                 (axon/sampler/vllm/server.py:379-625, engine.py:300-304)
    weight sync  FSDP state_dict -> full tensors -> ``model.load_weights`` inside the vLLM worker
                 (axon/sampler/mixins/sync_mixin.py:86-168, axon/sampler/vllm/engine.py:305-424)
    training     HF ``Qwen3ForCausalLM`` under torch FSDP2 (fp32 master parameters, bf16 compute, fp32
                 gradient reduction, per-layer wrapping, gradient checkpointing), flash-attn varlen through
                 packed ``position_ids``, torch AdamW, gradient clipping
                 (axon/trainer/fsdp_trainer.py:362-422,587-771, axon/utils/fsdp/utils.py:386-448)
    fused head   the reference's own Triton ``linear_cross_entropy`` (log-probs + entropy without [T, V]
                 logits), loaded UNMODIFIED by file path from ``baseline/_ref``
                 (axon/utils/kernel/linear_cross_entropy.py, kernels.py; called as in
                 axon/models/transformers/dense_common.py:147-225)

Stock reference code on this path: the two kernel files above and ``axon/utils/torch/device.py``. Everything
else in this file is harness: the step loop, GRPO advantages and the PPO-clip loss (a few lines of torch with
the reference's mini-batch-global token mean and its x world-size gradient compensation for FSDP2's mean
reduction, axon/trainer/fsdp_trainer.py:600-612), packing into 8k-token micro-batches and the timing.

Nothing here imports ``axon_b200`` or loads its native library. Workload, budget rule and output schema are
those of the repository's own arm.
"""
from __future__ import annotations

import importlib
import json
import os
import sys
import tempfile
import time
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")

MODEL_CONFIGS = {
    "qwen3-8b": {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 4096, "intermediate_size": 12288,
                 "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
                 "vocab_size": 151936, "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
                 "hidden_act": "silu", "tie_word_embeddings": False, "torch_dtype": "bfloat16", "attention_bias": False,
                 "attention_dropout": 0.0, "bos_token_id": 151643, "eos_token_id": 151645, "use_cache": True},
}


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}), flush=True)


def load_reference_fused_head():
    """The reference's Triton log-prob / entropy head, imported from the untouched install. The ``axon`` and
    ``axon.utils`` packages are entered as bare namespaces so that their ``__init__`` files (which pull in
    omegaconf and ray) do not run; the kernel modules themselves execute as shipped."""
    if not os.path.isdir(os.path.join(REF_ROOT, "axon", "utils", "kernel")):
        raise RuntimeError("baseline/_ref/axon is absent (install the reference with pip --target baseline/_ref)")
    for name, rel in (("axon", "axon"), ("axon.utils", "axon/utils")):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.__path__ = [os.path.join(REF_ROOT, rel)]
            sys.modules[name] = m
    mod = importlib.import_module("axon.utils.kernel.linear_cross_entropy")
    return mod.linear_cross_entropy, os.path.relpath(mod.__file__, HERE)


def pack_bins(lengths: list[int], max_tokens: int, k_min: int = 1) -> list[list[int]]:
    """Longest-first into the emptiest of k bins; k grows until every bin holds at most ``max_tokens`` (a
    single longer sequence gets a bin of its own)."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    k = max(k_min, -(-sum(lengths) // max_tokens), 1)
    while True:
        bins, load = [[] for _ in range(k)], [0] * k
        for i in order:
            j = min(range(k), key=load.__getitem__)
            bins[j].append(i)
            load[j] += lengths[i]
        if all(l <= max_tokens or len(b) == 1 for l, b in zip(load, bins)) or k >= len(lengths):
            return bins
        k += 1


def run_reference_arm(args, t_start: float, ClockSampler, plan_steps, synthetic_inputs, metric: str) -> None:
    try:
        _run(args, t_start, ClockSampler, plan_steps, synthetic_inputs, metric)
    except Exception as e:  # noqa: BLE001 - the arm must always leave one JSON line
        import traceback
        traceback.print_exc()
        _unavailable(f"library-equivalent arm failed: {type(e).__name__}: {e}")


def _run(args, t_start, ClockSampler, plan_steps, synthetic_inputs, metric) -> None:
    if args.model not in MODEL_CONFIGS:
        return _unavailable(f"no reference-side config for model '{args.model}'")
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
    os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")      # the worker lives in this process, as in the reference
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
    os.environ.setdefault("VLLM_LOGGING_STREAM", "ext://sys.stderr")       # stdout carries the result lines only
    for k, v in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0"), ("MASTER_ADDR", "127.0.0.1")):
        os.environ.setdefault(k, v)
    if "MASTER_PORT" not in os.environ:
        import socket
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            os.environ["MASTER_PORT"] = str(s.getsockname()[1])
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])

    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    linear_cross_entropy, kernel_file = load_reference_fused_head()

    mcfg = dict(MODEL_CONFIGS[args.model])
    if args.layers:
        mcfg["num_hidden_layers"] = args.layers
    cfg_dir = tempfile.mkdtemp(prefix="ref_arm_cfg_")
    with open(os.path.join(cfg_dir, "config.json"), "w") as f:
        json.dump(mcfg, f)

    # ---- sampler: one vLLM engine per rank (tensor parallel 1), built while the GPU is still empty
    from vllm import LLM, SamplingParams
    total = torch.cuda.mem_get_info(dev)[1]
    n_params = _param_count(mcfg)
    trainer_resident = n_params * 12 / world                       # fp32 master + two fp32 Adam moments, sharded
    util = min(0.80, max(0.30, (total - trainer_resident - 24e9) / total))
    max_len = args.prompt_len + args.max_response
    llm = LLM(model=cfg_dir, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", enable_sleep_mode=True,
              gpu_memory_utilization=util, max_model_len=max_len, seed=args.seed, enable_prefix_caching=True,
              enable_chunked_prefill=True, max_num_seqs=args.prompts_per_gpu * args.group,
              max_num_batched_tokens=max(32768, max_len), tensor_parallel_size=1,
              distributed_executor_backend="external_launcher", disable_log_stats=True)
    llm.sleep(level=1)
    torch.cuda.empty_cache()

    # ---- trainer: HF model under FSDP2
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
    from transformers import AutoConfig, AutoModelForCausalLM
    hf_cfg = AutoConfig.from_pretrained(cfg_dir)
    attn_impl = "flash_attention_2"
    try:
        import flash_attn  # noqa: F401
    except Exception:  # noqa: BLE001
        attn_impl = "sdpa"
    torch.manual_seed(args.seed)
    with torch.device(dev):
        model = AutoModelForCausalLM.from_config(hf_cfg, dtype=torch.float32, attn_implementation=attn_impl)
    model.gradient_checkpointing_enable(gradient_checkpointing_kwargs={"use_reentrant": False})
    model.config.use_cache = False
    model.train()

    def ppo_forward(self, input_ids, position_ids, temperature: float = 1.0):
        """Base model -> hidden states -> the reference's fused log-prob / entropy head (labels rolled by one)."""
        hidden = self.model(input_ids=input_ids, position_ids=position_ids, use_cache=False).last_hidden_state
        labels = torch.roll(input_ids, shifts=-1, dims=-1)
        return linear_cross_entropy(hidden, self.lm_head.weight, labels, float(temperature), "none")

    model.forward = types.MethodType(ppo_forward, model)
    mesh = init_device_mesh("cuda", (world,))
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32, cast_forward_inputs=True)
    fs = dict(mesh=mesh, mp_policy=mp, reshard_after_forward=False)
    for layer in model.model.layers:
        fully_shard(layer, **fs)
    fully_shard(model.model.embed_tokens, **fs)
    fully_shard(model, **fs)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-6, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)

    P, G = args.prompts_per_gpu, args.group
    rng = np.random.default_rng(args.seed + 1000 * rank)
    pinned = torch.empty(P, args.prompt_len, dtype=torch.int32, pin_memory=True)
    n_minis = max(1, (P * world) // 64)
    timing: dict[str, float] = {}

    def sync_weights_and_wake():
        """Hybrid-engine hand-over: wake the weights, stream every full tensor into the vLLM model, wake the KV pool."""
        torch.cuda.empty_cache()
        llm.wake_up(tags=["weights"])
        sd = model.state_dict()

        def full_tensors():
            for name, p in sd.items():
                yield name, (p.full_tensor() if hasattr(p, "full_tensor") else p)

        llm.collective_rpc(lambda worker: worker.model_runner.model.load_weights(full_tensors()) and None)
        del sd
        torch.cuda.empty_cache()
        llm.wake_up(tags=["kv_cache"])
        llm.reset_prefix_cache()

    def forward_logprobs(seqs, grad: bool, temperature=1.0):
        """seqs: list of int64 tensors (one packed micro-batch). Returns per-token log-probs / entropies of the packed row."""
        ids = torch.cat(seqs).to(dev, non_blocking=True)[None]
        pos = torch.cat([torch.arange(len(s)) for s in seqs]).to(dev, non_blocking=True)[None]
        with torch.set_grad_enabled(grad):
            lp, ent = model(input_ids=ids, position_ids=pos, temperature=temperature)
        return lp.reshape(-1), ent.reshape(-1)

    def one_step():
        t0 = time.perf_counter()
        prompts, caps, rewards = synthetic_inputs(rng, mcfg["vocab_size"], P, G, args.prompt_len, args.mean_response,
                                                  args.max_response)
        pinned.copy_(torch.from_numpy(prompts))
        prompts_dev = pinned.to(dev, non_blocking=True)                 # the step's inputs cross PCIe here
        prompt_lists = prompts_dev.cpu().tolist()
        # ---- rollout
        sync_weights_and_wake()
        torch.cuda.synchronize(dev)
        t1 = time.perf_counter()
        reqs = [{"prompt_token_ids": prompt_lists[i]} for i in range(P) for _ in range(G)]
        sps = [SamplingParams(temperature=1.0, max_tokens=int(caps[k]), ignore_eos=True, logprobs=0, detokenize=False)
               for k in range(P * G)]
        outs = llm.generate(reqs, sps, use_tqdm=False)
        torch.cuda.synchronize(dev)
        t2 = time.perf_counter()
        llm.sleep(level=1)
        torch.cuda.empty_cache()
        t3 = time.perf_counter()
        # ---- batch, advantages (group-normalised), old log-probs
        seqs, resp_start, samp_lp = [], [], []
        for k, o in enumerate(outs):
            c = o.outputs[0]
            toks = list(c.token_ids)
            seqs.append(torch.tensor(prompt_lists[k // G] + toks, dtype=torch.int64))
            resp_start.append(args.prompt_len)
            samp_lp.append(torch.tensor([next(iter(d.values())).logprob for d in c.logprobs], dtype=torch.float32)
                           if c.logprobs else torch.zeros(len(toks)))
        r = torch.from_numpy(rewards).view(P, G)
        adv = ((r - r.mean(1, keepdim=True)) / (r.std(1, keepdim=True) + 1e-6)).reshape(-1)
        lens = [len(s) for s in seqs]
        k_local = len(pack_bins(lens, args.micro_batch_tokens))
        kt = torch.tensor([k_local], device=dev)
        dist.all_reduce(kt, op=dist.ReduceOp.MAX)                        # FSDP collectives need equal micro-batch counts
        old_lp = [None] * len(seqs)
        for b in pack_bins(lens, args.micro_batch_tokens, int(kt)):
            if not b:
                b = [0]
            lp, _ = forward_logprobs([seqs[i] for i in b], grad=False)
            off = 0
            for i in b:
                old_lp[i] = lp[off:off + lens[i]].float()
                off += lens[i]
        gap_num = sum(float(((old_lp[i][resp_start[i] - 1:lens[i] - 1].exp().cpu() - samp_lp[i].exp()).abs()).sum()) for i in range(len(seqs)))
        torch.cuda.synchronize(dev)
        t4 = time.perf_counter()
        # ---- mini-batches: forward + backward over packed micro-batches, clip, AdamW
        per_mini = -(-len(seqs) // n_minis)
        loss_total, gnorm = 0.0, 0.0
        for m in range(n_minis):
            idx = list(range(m * per_mini, min(len(seqs), (m + 1) * per_mini)))
            ntok = torch.tensor([float(sum(lens[i] - resp_start[i] for i in idx))], device=dev)
            dist.all_reduce(ntok)                                        # mini-batch-global token count
            bins = pack_bins([lens[i] for i in idx], args.micro_batch_tokens)
            kt = torch.tensor([len(bins)], device=dev)
            dist.all_reduce(kt, op=dist.ReduceOp.MAX)
            bins = pack_bins([lens[i] for i in idx], args.micro_batch_tokens, int(kt))
            for b in bins:
                rows = [idx[j] for j in b] or [idx[0]]
                weight = 1.0 if b else 0.0
                lp, _ = forward_logprobs([seqs[i] for i in rows], grad=True)
                old = torch.cat([old_lp[i] for i in rows])
                mask = torch.cat([torch.cat([torch.zeros(resp_start[i] - 1), torch.ones(lens[i] - resp_start[i]), torch.zeros(1)])
                                  for i in rows]).to(dev)
                a = torch.cat([adv[i].expand(lens[i]) for i in rows]).to(dev)
                ratio = torch.exp(lp.float() - old)
                pg = torch.maximum(-a * ratio, -a * ratio.clamp(1 - 0.2, 1 + 0.2))
                loss = (pg * mask).sum() / ntok.clamp_min(1.0) * weight
                (loss * world).backward()                                # FSDP2 averages gradients over ranks
                loss_total += float(loss.detach())
            gnorm = float(torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0))
            opt.step()
            opt.zero_grad(set_to_none=True)
        torch.cuda.synchronize(dev)
        t5 = time.perf_counter()
        n_tok, n_resp = sum(lens), sum(lens[i] - resp_start[i] for i in range(len(seqs)))
        timing.update(setup_and_sync=t1 - t0, rollout=t2 - t1, sleep=t3 - t2, prepare_and_old_logprob=t4 - t3, train=t5 - t4,
                      total=t5 - t0)
        loss_host = torch.tensor([loss_total], device=dev).cpu()          # the step's result is read back to the host
        return {"tokens": n_tok, "response_tokens": n_resp, "loss": float(loss_host), "grad_norm": gnorm,
                "sampler_probs_diff_mean": gap_num / max(n_resp, 1)}

    def barrier():
        dist.barrier()
        torch.cuda.synchronize(dev)

    def agree(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    t_w = time.time()
    one_step()
    barrier()
    first = agree(time.time() - t_w)
    extra_warm, n_timed = plan_steps(first, agree(time.time() - t_start), args.max_seconds, args.steps, args.warmup)
    for _ in range(extra_warm):
        one_step()
    n_warm = 1 + extra_warm
    barrier()
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    ev0 = torch.cuda.Event(enable_timing=True)
    barrier()
    t_host0 = time.perf_counter()
    ev0.record()
    tokens = resp = 0
    phase: dict[str, float] = {}
    out = None
    for k in range(1, n_timed + 1):
        last = one_step()
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        ev.synchronize()
        host_ms = (time.perf_counter() - t_host0) * 1e3
        dev_ms = ev0.elapsed_time(ev)
        tokens += last["tokens"]
        resp += last["response_tokens"]
        for kk, v in timing.items():
            phase[kk] = phase.get(kk, 0.0) + v
        st = torch.tensor([dev_ms, host_ms, float(tokens), float(resp)], dtype=torch.float64, device=dev)
        mx, sm = st.clone(), st.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        if rank == 0:
            g_dev, g_host, g_tok, g_resp = float(mx[0]), float(mx[1]), float(sm[2]), float(sm[3])
            out = {
                "metric": metric, "value": g_tok / (g_dev / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": k,
                "warmup": n_warm, "steps_requested": args.steps, "warmup_requested": args.warmup,
                "max_seconds": args.max_seconds, "ms_per_step": g_dev / k, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic (uniform-random prompts, truncated-geometric lengths, random-init weights)",
                "impl": "reference", "reference_class": "library-equivalent", "same_config": not args.layers,
                "reference_stock_code": [kernel_file, "_ref/axon/utils/kernel/kernels.py", "_ref/axon/utils/torch/device.py"],
                "config": {"model": args.model + (f"[layers={args.layers}]" if args.layers else ""),
                           "global_batch": P * G * world, "prompts_per_gpu": P, "group": G,
                           "seq_len": args.prompt_len + args.max_response, "prompt_len": args.prompt_len,
                           "max_response": args.max_response, "mean_response": args.mean_response,
                           "micro_batch_tokens": args.micro_batch_tokens,
                           "parallelism": f"dp{world} fsdp2 (fp32 master, bf16 compute) + vllm tp1 per gpu, colocated, sleep level 1",
                           "attention": attn_impl, "old_log_probs": "recomputed", "optimizer_steps_per_rl_step": n_minis,
                           "vllm": {"version": _vllm_version(), "gpu_memory_utilization": round(util, 3), "prefix_caching": True},
                           "l2": "inputs larger than L2 (weights + KV cache streamed every step)",
                           "tokens_counted": "prompt + response tokens of every sampled sequence",
                           "response_tokens_per_s": g_resp / (g_dev / 1e3)},
                "clocks": clocks.read(),
                "e2e": {"value": g_tok / (g_host / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": pinned.numel() * 4,
                        "d2h_bytes_per_step": 4},
                "gpu_launches": None,
                "phase_seconds_per_step": {kk: v / k for kk, v in phase.items()},
                "last_step": {kk: last.get(kk) for kk in ("loss", "grad_norm", "sampler_probs_diff_mean")},
                "peak_mem_gib": torch.cuda.max_memory_allocated(dev) / 2 ** 30,
                "wall_s_since_start": time.time() - t_start,
            }
            print(json.dumps(out), flush=True)
    barrier()
    if rank == 0 and out is not None:
        out["clocks"] = clocks.stop()
        out["final"] = True
        print(json.dumps(out), flush=True)
    dist.destroy_process_group()


def _param_count(c: dict) -> int:
    H, L, V, F = c["hidden_size"], c["num_hidden_layers"], c["vocab_size"], c["intermediate_size"]
    q, kv = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    per_layer = H * (q + 2 * kv) + q * H + 3 * H * F + 2 * H + 2 * c["head_dim"]
    return L * per_layer + V * H * (1 if c.get("tie_word_embeddings") else 2) + H


def _vllm_version() -> str:
    try:
        import vllm
        return vllm.__version__
    except Exception:  # noqa: BLE001
        return "?"
