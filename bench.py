"""Headline benchmark: RL step tokens/s (rollout + train + weight hand-over), Qwen3-8B GRPO, colocated.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched by torch.distributed.run)
    python bench.py --impl reference ...                     (the unmodified reference arm)

Workload per GPU (weak scaling; the named config is 256 prompts x group 8 on 8 GPUs): 32 prompts of
1024 uniform-random tokens, 8 samples each, response lengths truncated-geometric (mean 1500, cap
4096), Bernoulli(0.3) rewards, GRPO advantages, PPO-clip loss, 8k-token packed micro-batches,
mini-batches of 64 prompts (global), bf16 compute with fp32 AdamW master weights. Synthetic data,
random-init weights of the Qwen3-8B architecture.

The timed region calls the public step API once per step; every step copies its prompts from pinned
host memory to the device and reads the step's loss back to the host. ``value`` is timed on the
device with CUDA events (max over ranks); ``e2e.value`` is timed on the host around the same calls.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

import numpy as np

BASELINE_TOKENS_PER_S = None  # the reference publishes no throughput number


def reference_arm(args) -> None:
    """The reference installs offline only without its dependencies; its entry points import ray,
    hydra, omegaconf and tensordict, none of which exist in this image or its wheelhouse."""
    here = os.path.dirname(os.path.abspath(__file__))
    ref = os.path.join(here, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref, "axon")):
        why = "baseline/_ref is absent (pip install --no-index of the reference was not run)"
    else:
        sys.path.insert(0, ref)
        try:
            import axon.driver.train_agent_ppo  # noqa: F401
        except Exception as e:  # noqa: BLE001
            why = f"reference import fails offline: {type(e).__name__}: {e}"
    if why is None:
        why = "reference needs a Ray cluster, a vLLM 0.19 fork and HF checkpoints that are not available offline"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc = gpu_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = sorted(sm)[len(sm) // 4:]
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (invalid as a result)")
    ap.add_argument("--prompts-per-gpu", type=int, default=32)
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--max-response", type=int, default=4096)
    ap.add_argument("--mean-response", type=float, default=1500.0)
    ap.add_argument("--micro-batch-tokens", type=int, default=8192)
    ap.add_argument("--seed", type=int, default=1234)
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from axon_b200.driver.colocated import ColocatedRLRunner, RLStepConfig
    from axon_b200.models.config import get_config
    from axon_b200.models.dense import DenseModel
    from axon_b200.ops import _common as C
    from axon_b200.trainer.policy import OptimConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    pg = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        pg = dist.group.WORLD

    cfg = get_config(args.model)
    if args.layers:
        cfg.num_hidden_layers = args.layers
    model = DenseModel(cfg, device=dev)
    model.params.init_random(0.02, seed=args.seed)          # same weights on every rank
    rl = RLStepConfig(n_samples=args.group, max_prompt_length=args.prompt_len, max_response_length=args.max_response,
                      temperature=1.0, loss="ppo", loss_args={"clip_ratio": 0.2}, advantage="grpo",
                      mini_batch_size=max(1, 64 // world), max_token_len_per_gpu=args.micro_batch_tokens,
                      max_num_seqs=args.prompts_per_gpu * args.group,
                      optim=OptimConfig(lr=1e-6, weight_decay=0.1, grad_clip=1.0))
    runner = ColocatedRLRunner(model, rl, pg, seed=args.seed)
    rng = np.random.default_rng(args.seed + 1000 * rank)
    P, G = args.prompts_per_gpu, args.group
    pinned = torch.empty(P, args.prompt_len, dtype=torch.int32, pin_memory=True)

    def make_inputs():
        pinned.copy_(torch.from_numpy(rng.integers(0, cfg.vocab_size, (P, args.prompt_len), dtype=np.int32)))
        p = 1.0 / args.mean_response
        caps = np.minimum(rng.geometric(p, P * G), args.max_response).astype(np.int64)
        rewards = rng.binomial(1, 0.3, P * G).astype(np.float32)
        return caps, rewards

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        caps, rewards = make_inputs()
        runner.step(pinned, response_caps=caps, rewards=rewards)
    barrier()
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    launches0 = C.LAUNCH_COUNT
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tokens = resp_tokens = 0
    h2d = d2h = 0
    phase = {}
    barrier()
    t_host0 = time.perf_counter()
    ev0.record()
    last = {}
    for _ in range(args.steps):
        caps, rewards = make_inputs()
        last = runner.step(pinned, response_caps=caps, rewards=rewards)   # H2D of prompts, D2H of metrics inside
        tokens += last["tokens"]
        resp_tokens += last["response_tokens"]
        h2d += pinned.numel() * 4
        d2h += 8 * 4
        for k, v in runner.timing.items():
            phase[k] = phase.get(k, 0.0) + v
    ev1.record()
    barrier()
    t_host = time.perf_counter() - t_host0
    clk = clocks.stop() if rank == 0 else None
    dev_ms = ev0.elapsed_time(ev1)
    C.check_status()
    stats = torch.tensor([dev_ms, t_host * 1e3, float(tokens), float(resp_tokens)], dtype=torch.float64, device=dev)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        dev_ms, host_ms = float(mx[0]), float(mx[1])
        tokens, resp_tokens = float(sm[2]), float(sm[3])
    else:
        host_ms = t_host * 1e3
    if rank == 0:
        value = tokens / (dev_ms / 1e3)
        e2e = tokens / (host_ms / 1e3)
        out = {
            "metric": "RL step tokens/sec (rollout+train+sync), Qwen3-8B GRPO", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
            "dtype": "bf16", "data": "synthetic (uniform-random prompts, truncated-geometric lengths, random-init weights)",
            "impl": "ours",
            "config": {"model": args.model + (f"[layers={args.layers}]" if args.layers else ""),
                       "global_batch": P * G * world, "prompts_per_gpu": P, "group": G, "seq_len": args.prompt_len + args.max_response,
                       "prompt_len": args.prompt_len, "max_response": args.max_response, "mean_response": args.mean_response,
                       "micro_batch_tokens": args.micro_batch_tokens, "parallelism": f"dp{world} zero1 colocated",
                       "old_log_probs": "recomputed", "optimizer_steps_per_rl_step": max(1, (P * world) // 64),
                       "l2": "inputs larger than L2 (16 GB weights + KV cache streamed every step)",
                       "tokens_counted": "prompt + response tokens of every sampled sequence",
                       "response_tokens_per_s": resp_tokens / (dev_ms / 1e3)},
            "clocks": clk,
            "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d // args.steps,
                    "d2h_bytes_per_step": d2h // args.steps},
            "gpu_launches": int(C.LAUNCH_COUNT - launches0),
            "phase_seconds_per_step": {k: v / args.steps for k, v in phase.items()},
            "last_step": {k: last.get(k) for k in ("loss", "grad_norm", "sampler_probs_diff_mean", "entropy")},
            "peak_mem_gib": torch.cuda.max_memory_allocated(dev) / 2 ** 30,
            "runner": {k: runner.phase_detail.get(k) for k in ("kv_pages", "kv_peak_pages", "offloaded", "recompute", "preempted")},
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
