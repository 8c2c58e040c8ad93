"""Disaggregated topology of the headline benchmark: half of the GPUs train, half sample.

Launched by ``bench.py --topology disaggregated --gpus N`` under ``torch.distributed.run`` (N even): ranks
``[0, N/2)`` are trainers (data parallel, fused ZeRO-1 among themselves), ranks ``[N/2, N)`` are samplers (one
engine per GPU). The global workload is the colocated benchmark's (32 prompts x group 8 per GPU of the job),
so every sampler generates for two GPUs' worth of prompts and every trainer trains on two GPUs' worth.

One iteration is the reference's one-step-off pipeline
(recipes/frozenlake/train_frozenlake_qwen_30b_a3b_p2p_one_off_pipeline.sh, axon/driver/sync_ppo.py:149-179):

    samplers: generate batch k                 |  trainers: train on batch k-1
    ---------------------------------------------------------------------------- barrier
    batch k travels to the trainers (host objects over the world group)
    trainers -> samplers weight push: the RoutingTable plan, executed by the peer-store kernel through the
    production mixins (``TrainerP2PMixin.send_trainer_to_sampler_weights`` /
    ``SamplerP2PMixin.receive_trainer_to_sampler_weights``), timed on the device

The first iteration only generates (nothing to train on yet) and is part of the warm-up. Reported: tokens/s of
the whole job, and ``weight_sync``: seconds per push (max over ranks), bytes per sampler, GB/s per sending GPU
from the kernel's own events, and that rate as a fraction of the measured NVLink peer-copy rate (770 GB/s per
direction on this machine class).
"""
from __future__ import annotations

import json
import os
import threading
import time
from types import SimpleNamespace

import numpy as np

NVLINK_PEER_COPY_GBS = 770.0      # measured peer copy, one direction, per GPU


def run_disaggregated(args, t_start: float, ClockSampler, plan_steps, synthetic_inputs) -> None:
    import torch
    import torch.distributed as dist

    from ..models.config import get_config
    from ..models.dense import DenseModel
    from ..ops import _common as C
    from ..sampler.engine import GenerationEngine
    from ..sampler.kv_cache import PagedKVCache
    from ..sampler.mixins.p2p_mixin import SamplerP2PMixin
    from ..sampler.params import SamplingParams
    from ..trainer.mixins.p2p_mixin import TrainerP2PMixin
    from ..trainer.policy import OptimConfig
    from ..utils.p2p.routing_table import RoutingTable
    from .colocated import ColocatedRLRunner, RLStepConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2 or world % 2:
        if rank == 0:
            print(json.dumps({"impl": "ours", "topology": "disaggregated",
                              "unavailable": "needs an even number of GPUs >= 2 (launch with torch.distributed.run)"}), flush=True)
        return
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    n_train = world // 2
    n_samp = world - n_train
    is_trainer = rank < n_train
    trainer_pg = dist.new_group(list(range(n_train)))
    dist.new_group(list(range(n_train, world)))                   # sampler ranks (created on every rank, as new_group requires)

    cfg = get_config(args.model)
    if args.layers:
        cfg.num_hidden_layers = args.layers
    model = DenseModel(cfg, device=dev)
    model.params.init_random(0.02, seed=args.seed + (0 if is_trainer else 1))   # samplers start with OTHER weights: the first push must fix them
    P_job, G = args.prompts_per_gpu * world, args.group
    P_samp = P_job // n_samp                                      # prompts generated per sampler rank
    rl = RLStepConfig(n_samples=G, max_prompt_length=args.prompt_len, max_response_length=args.max_response,
                      temperature=1.0, loss="ppo", loss_args={"clip_ratio": 0.2}, advantage="grpo",
                      mini_batch_size=max(1, 64 // n_train), max_token_len_per_gpu=args.micro_batch_tokens,
                      max_num_seqs=min(256, P_samp * G), optim=OptimConfig(lr=1e-6, weight_decay=0.1, grad_clip=1.0))

    # ---- the two ends of the weight push, on the production mixins
    port = torch.tensor([0], dtype=torch.int64, device=dev)
    if rank == 0:
        import socket
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port[0] = s.getsockname()[1]
    dist.broadcast(port, 0)
    runner = engine = None
    if is_trainer:
        runner = ColocatedRLRunner(model, rl, trainer_pg, seed=args.seed)
        end = type("TrainerEnd", (TrainerP2PMixin,), {})()
        end.rank, end.world_size, end.device, end.model = rank, n_train, dev, model
        end.connect_trainer_to_sampler("127.0.0.1", int(port[0]), world, 0)
    else:
        srank = rank - n_train
        end = type("SamplerEnd", (SamplerP2PMixin,), {})()
        end.rank, end.world_size, end.device, end.model, end.tp = srank, n_samp, dev, model, 1
        end.server, end.scfg, end.engine = SimpleNamespace(_ctl_lock=threading.Lock()), {}, None
        end.connect_sampler_to_trainer("127.0.0.1", int(port[0]), world, n_train)
        need = PagedKVCache.bytes_per_page(cfg, 2)
        want = min(256, P_samp * G) * ((args.prompt_len + args.max_response) // 128 + 1)
        pages = int(min(want, torch.cuda.mem_get_info(dev)[0] * 0.85 // need))
        engine = GenerationEngine(model, num_pages=pages, max_num_seqs=min(256, P_samp * G), seed=args.seed + rank)   # decode graphs are captured up to 256 rows
        engine.set_max_model_len(args.prompt_len + args.max_response)
        end.engine = engine
    maps = [None] * world
    dist.all_gather_object(maps, end.get_parameter_mapping())
    table = RoutingTable(maps[:n_train], maps[n_train:])

    rng = np.random.default_rng(args.seed + 1000 * rank)
    pinned = torch.empty(P_samp, args.prompt_len, dtype=torch.int32, pin_memory=True)
    sync_log: list[dict] = []

    def push_weights(first: bool) -> None:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        ev0.record()
        t0 = time.perf_counter()
        if is_trainer:
            r = end.send_trainer_to_sampler_weights(routing_table=table if first else None)
        else:
            r = end.receive_trainer_to_sampler_weights(routing_table=table if first else None)
        ev1.record()
        ev1.synchronize()
        sync_log.append({"seconds": time.perf_counter() - t0, "device_ms": ev0.elapsed_time(ev1),
                         "kernel_ms": r.get("kernel_ms", 0.0), "bytes": r["bytes"], "transport": r["transport"]})

    def generate_batch():
        prompts, caps, rewards = synthetic_inputs(rng, cfg.vocab_size, P_samp, G, args.prompt_len, args.mean_response,
                                                  args.max_response)
        pinned.copy_(torch.from_numpy(prompts))
        prompts_h = pinned.to(dev, non_blocking=True).cpu().tolist()          # H2D of the step's inputs, then host token lists
        ps, sp = [], []
        for i in range(P_samp):
            for j in range(G):
                ps.append(prompts_h[i])
                sp.append(SamplingParams(temperature=1.0, max_tokens=int(caps[i * G + j]), ignore_eos=True))
        outs = engine.generate(ps, sp)
        torch.cuda.synchronize(dev)
        return {"prompts": prompts_h, "tokens": [o.token_ids for o in outs], "logprobs": [o.logprobs for o in outs],
                "rewards": rewards}

    def train_batch(batches: list[dict], step: int) -> dict:
        """Trainer rank r takes every n_train-th prompt group of the gathered batches."""
        from ..sampler.params import TokenOutput
        prompts, outs, rewards, groups = [], [], [], []
        gidx = 0
        for b in batches:
            for i, p in enumerate(b["prompts"]):
                if gidx % n_train == rank:
                    for j in range(G):
                        k = i * G + j
                        prompts.append(p)
                        outs.append(TokenOutput(token_ids=b["tokens"][k], logprobs=b["logprobs"][k], finish_reason="length"))
                        rewards.append(b["rewards"][k])
                        groups.append(f"{step}-{gidx}")
                gidx += 1
        runner._enter_training()
        return runner.train_on_samples(prompts, outs, np.array(rewards, dtype=np.float32), groups)

    def iteration(step: int, pending):
        """Generate batch ``step`` on the samplers while the trainers train on ``pending``; move the new batch over;
        push the weights. Returns (new pending batch list, training result or None)."""
        res = None
        t0 = time.perf_counter()
        mine = None
        if is_trainer:
            if pending is not None:
                res = train_batch(pending, step)
        else:
            mine = generate_batch()
        t1 = time.perf_counter()
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        new_pending = [g for g in gathered[n_train:]]
        t2 = time.perf_counter()
        push_weights(first=(step == 0))
        phase = {"work": t1 - t0, "batch_transfer": t2 - t1, "weight_sync": time.perf_counter() - t2}
        return new_pending, res, phase

    def agree_max(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    # ---- warm-up: iteration 0 fills the pipeline (no training yet), iteration 1 is the first full one
    pending, _, _ = iteration(0, None)
    t_w = time.time()
    pending, _, _ = iteration(1, pending)
    first = agree_max(time.time() - t_w)
    extra_warm, n_timed = plan_steps(first, agree_max(time.time() - t_start), args.max_seconds, args.steps, max(1, args.warmup - 1))
    step = 2
    for _ in range(extra_warm):
        pending, _, _ = iteration(step, pending)
        step += 1
    n_warm = 2 + extra_warm
    dist.barrier()
    torch.cuda.synchronize(dev)
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    launches0 = C.LAUNCH_COUNT
    sync_log.clear()
    ev0 = torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize(dev)
    t_host0 = time.perf_counter()
    ev0.record()
    tokens = resp = 0.0
    phases: dict[str, float] = {}
    out = None
    for k in range(1, n_timed + 1):
        pending, res, ph = iteration(step, pending)
        step += 1
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        ev.synchronize()
        dev_ms, host_ms = ev0.elapsed_time(ev), (time.perf_counter() - t_host0) * 1e3
        if res is not None:
            tokens += res["tokens"]
            resp += res["response_tokens"]
        for kk, v in ph.items():
            phases[kk] = phases.get(kk, 0.0) + v
        s_last = sync_log[-1]
        st = torch.tensor([dev_ms, host_ms, tokens, resp, s_last["seconds"], s_last["kernel_ms"],
                           float(torch.sum(model.params.flat, dtype=torch.float64))], dtype=torch.float64, device=dev)
        mx, mn, sm = st.clone(), st.clone(), st.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(mn, op=dist.ReduceOp.MIN)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        launches = torch.tensor([float(C.LAUNCH_COUNT - launches0)], dtype=torch.float64, device=dev)
        dist.all_reduce(launches)
        if rank == 0:
            g_dev, g_host, g_tok, g_resp = float(mx[0]), float(mx[1]), float(sm[2]), float(sm[3])
            sent = [s for s in sync_log if s["transport"] == "peer-store kernel"]
            per_trainer_bytes = float(np.mean([s["bytes"] for s in sync_log])) if sync_log else 0.0
            kernel_s = float(mx[5]) / 1e3
            gbs = per_trainer_bytes / kernel_s / 1e9 if kernel_s > 0 else None
            value = g_tok / (g_dev / 1e3)
            out = {
                "metric": "RL step tokens/sec (rollout+train+sync), Qwen3-8B GRPO", "value": value, "unit": "tokens/s",
                "n_gpus": world, "steps": k, "warmup": n_warm, "steps_requested": args.steps, "warmup_requested": args.warmup,
                "max_seconds": args.max_seconds, "ms_per_step": g_dev / k, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "impl": "ours", "topology": "disaggregated",
                "data": "synthetic (uniform-random prompts, truncated-geometric lengths, random-init weights)",
                "config": {"model": args.model + (f"[layers={args.layers}]" if args.layers else ""),
                           "global_batch": P_job * G, "trainer_gpus": n_train, "sampler_gpus": n_samp, "group": G,
                           "prompt_len": args.prompt_len, "max_response": args.max_response, "mean_response": args.mean_response,
                           "micro_batch_tokens": args.micro_batch_tokens,
                           "parallelism": f"{n_train} trainer GPUs (dp, fused zero1) + {n_samp} sampler GPUs (tp1), one-step-off pipeline",
                           "staleness_steps": 1, "response_tokens_per_s": g_resp / (g_dev / 1e3),
                           "l2": "inputs larger than L2 (weights + KV cache streamed every step)"},
                "weight_sync": {"seconds": float(mx[4]), "kernel_ms": float(mx[5]), "transport": sync_log[-1]["transport"],
                                "bytes_per_trainer_gpu": per_trainer_bytes, "gbs_per_sending_gpu": gbs,
                                "fraction_of_measured_peer_copy": (gbs / NVLINK_PEER_COPY_GBS) if gbs else None,
                                "peer_store_pushes": len(sent),
                                "params_checksum_equal_across_trainers_and_samplers": bool(mx[6] == mn[6])},
                "clocks": clocks.read(),
                "e2e": {"value": g_tok / (g_host / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": P_samp * args.prompt_len * 4 * n_samp,
                        "d2h_bytes_per_step": 32 * n_train},
                "gpu_launches": int(launches[0]),
                "phase_seconds_per_step": {kk: v / k for kk, v in phases.items()},
                "last_step": {kk: (res or {}).get(kk) for kk in ("loss", "grad_norm", "sampler_probs_diff_mean")},
                "wall_s_since_start": time.time() - t_start,
            }
            print(json.dumps(out), flush=True)
    dist.barrier()
    torch.cuda.synchronize(dev)
    C.check_status()
    if rank == 0 and out is not None:
        out["clocks"] = clocks.stop()
        out["final"] = True
        print(json.dumps(out), flush=True)
    dist.destroy_process_group()
