"""Headline benchmark: RL step tokens/s (rollout + train + weight hand-over), Qwen3-8B GRPO.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torch.distributed.run)
    python bench.py --impl reference ...                       (library-equivalent arm, see baseline/ref_arm.py)
    python bench.py --topology disaggregated --gpus N ...      (N/2 trainer + N/2 sampler GPUs, weight sync timed)

Workload per GPU (weak scaling; the named config is 256 prompts x group 8 on 8 GPUs): 32 prompts of
1024 uniform-random tokens, 8 samples each, response lengths truncated-geometric (mean 1500, cap
4096), Bernoulli(0.3) rewards, GRPO advantages, PPO-clip loss, 8k-token packed micro-batches,
mini-batches of 64 prompts (global), bf16 compute with fp32 AdamW master weights. Synthetic data,
random-init weights of the Qwen3-8B architecture.

One RL step of this workload takes on the order of a minute per GPU, so the run obeys a wall-clock
budget (``--max-seconds``, counted from process start, model construction included): after the first
warm-up step the step time is known and the number of warm-up and timed steps is cut to what fits
(at least one of each); ``steps`` / ``warmup`` in the output are the counts actually run,
``steps_requested`` / ``warmup_requested`` the command line's. A complete cumulative JSON line is
printed and flushed after EVERY timed step, so the last line on stdout is always a valid result.

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
import tempfile
import time

T_PROCESS_START = time.time()

import numpy as np  # noqa: E402

BASELINE_TOKENS_PER_S = None  # the reference publishes no throughput number
METRIC = "RL step tokens/sec (rollout+train+sync), Qwen3-8B GRPO"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms into a file; ``read()`` summarises what
    has been written so far without stopping the sampler."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.path, self.fh = gpu_index, None, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="bench_clocks_", suffix=".csv")
            self.fh = os.fdopen(fd, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=self.fh,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def read(self) -> dict:
        if self.proc is None or self.path is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        try:
            with open(self.path) as f:
                out = f.read()
        except OSError:
            out = ""
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

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
                self.proc.wait()
        out = self.read()
        try:
            if self.fh is not None:
                self.fh.close()
            if self.path is not None:
                os.unlink(self.path)
        except OSError:
            pass
        self.proc = None
        return out


def plan_steps(first_step_s: float, elapsed_s: float, budget_s: float, steps: int, warmup: int) -> tuple[int, int]:
    """How many MORE warm-up steps and how many timed steps fit in the budget after one warm-up step
    took ``first_step_s``. Later steps are a little faster than the first (graphs captured, pools
    sized), so the first step's time is a safe estimate. Timed steps come first: extra warm-up steps
    are only run while at least min(steps, 3) timed steps still fit."""
    per = max(first_step_s, 1e-3) * 1.05
    fit = int(max(0.0, budget_s - elapsed_s) // per)
    fit = max(fit, 1)                                   # always one timed step
    want_timed = min(steps, 3)
    extra_warm = max(0, min(warmup - 1, fit - want_timed))
    timed = max(1, min(steps, fit - extra_warm))
    return extra_warm, timed


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--topology", default="colocated", choices=["colocated", "disaggregated"])
    ap.add_argument("--max-seconds", type=float, default=600.0,
                    help="wall-clock budget from process start; warm-up and timed step counts are cut to fit")
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (invalid as a result)")
    ap.add_argument("--prompts-per-gpu", type=int, default=32)
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--max-response", type=int, default=4096)
    ap.add_argument("--mean-response", type=float, default=1500.0)
    ap.add_argument("--micro-batch-tokens", type=int, default=8192)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--via-driver", action="store_true",
                    help="diagnostic: the same model through train_agent (driver, worker groups, Engine, programs) and through the "
                         "single-process runner on fixed-length responses; reports both rates")
    ap.add_argument("--fixed-response", type=int, default=512, help="--via-driver: response tokens per sample")
    ap.add_argument("--ab-nccl", action="store_true",
                    help="N > 1: after the timed steps run one extra step with the NCCL optimizer path and report its time")
    return ap.parse_args(argv)


def synthetic_inputs(rng, vocab: int, P: int, G: int, prompt_len: int, mean_response: float, max_response: int):
    """One step's synthetic workload: prompts [P, prompt_len] int32, per-sample length caps and rewards."""
    prompts = rng.integers(0, vocab, (P, prompt_len), dtype=np.int32)
    caps = np.minimum(rng.geometric(1.0 / mean_response, P * G), max_response).astype(np.int64)
    rewards = rng.binomial(1, 0.3, P * G).astype(np.float32)
    return prompts, caps, rewards


def main() -> None:
    args = parse_args()
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, here)
    if args.impl == "reference":
        from baseline.ref_arm import run_reference_arm
        run_reference_arm(args, T_PROCESS_START, ClockSampler, plan_steps, synthetic_inputs, METRIC)
        return
    if args.via_driver:
        from axon_b200.driver.via_driver_bench import run_via_driver
        run_via_driver(args, T_PROCESS_START, ClockSampler)
        return
    if args.topology == "disaggregated":
        from axon_b200.driver.disaggregated_bench import run_disaggregated
        run_disaggregated(args, T_PROCESS_START, ClockSampler, plan_steps, synthetic_inputs)
        return

    import torch
    import torch.distributed as dist
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
        prompts, caps, rewards = synthetic_inputs(rng, cfg.vocab_size, P, G, args.prompt_len, args.mean_response,
                                                  args.max_response)
        pinned.copy_(torch.from_numpy(prompts))
        return caps, rewards

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def agree(x: float, op) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=op)
        return float(t[0])

    # ---- warm-up: the first step tells how long a step is; the plan is the same on every rank
    t_w = time.time()
    caps, rewards = make_inputs()
    runner.step(pinned, response_caps=caps, rewards=rewards)
    barrier()
    first = agree(time.time() - t_w, dist.ReduceOp.MAX if world > 1 else None)
    elapsed = agree(time.time() - T_PROCESS_START, dist.ReduceOp.MAX if world > 1 else None)
    extra_warm, n_timed = plan_steps(first, elapsed, args.max_seconds, args.steps, args.warmup)
    for _ in range(extra_warm):
        caps, rewards = make_inputs()
        runner.step(pinned, response_caps=caps, rewards=rewards)
    n_warm = 1 + extra_warm
    barrier()

    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    launches0 = C.LAUNCH_COUNT
    ev0 = torch.cuda.Event(enable_timing=True)
    tokens = resp_tokens = 0
    h2d = d2h = 0
    phase: dict[str, float] = {}
    barrier()
    t_host0 = time.perf_counter()
    ev0.record()
    out = None
    for k in range(1, n_timed + 1):
        caps, rewards = make_inputs()
        last = runner.step(pinned, response_caps=caps, rewards=rewards)   # H2D of prompts, D2H of metrics inside
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        ev.synchronize()
        host_ms = (time.perf_counter() - t_host0) * 1e3
        dev_ms = ev0.elapsed_time(ev)
        tokens += last["tokens"]
        resp_tokens += last["response_tokens"]
        h2d += pinned.numel() * 4
        d2h += 8 * 4
        for kk, v in runner.timing.items():
            phase[kk] = phase.get(kk, 0.0) + v
        stats = torch.tensor([dev_ms, host_ms, float(tokens), float(resp_tokens), float(torch.sum(model.params.flat, dtype=torch.float64)) if world > 1 else 0.0],
                             dtype=torch.float64, device=dev)
        checks = {}
        if world > 1:
            mx = stats.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            mn = stats.clone(); dist.all_reduce(mn, op=dist.ReduceOp.MIN)
            sm = stats.clone(); dist.all_reduce(sm, op=dist.ReduceOp.SUM)
            g_dev, g_host = float(mx[0]), float(mx[1])
            g_tok, g_resp = float(sm[2]), float(sm[3])
            # every rank holds the same parameters after the fused reduce + AdamW + broadcast
            checks = {"params_checksum": float(mx[4]), "params_checksum_equal_across_ranks": bool(mx[4] == mn[4]),
                      "optimizer_path": "fused peer-memory zero1" if runner.policy.fused is not None else "nccl"}
        else:
            g_dev, g_host, g_tok, g_resp = dev_ms, host_ms, float(tokens), float(resp_tokens)
        if rank == 0:
            value = g_tok / (g_dev / 1e3)
            out = {
                "metric": METRIC, "value": value, "unit": "tokens/s",
                "n_gpus": world, "steps": k, "warmup": n_warm, "steps_requested": args.steps,
                "warmup_requested": args.warmup, "max_seconds": args.max_seconds, "ms_per_step": g_dev / k,
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
                           "tokens_counted": "prompt + response tokens of every sampled sequence (each prompt is prefilled once per group; training processes every token)",
                           "response_tokens_per_s": g_resp / (g_dev / 1e3),
                           "weight_sync": "zero-copy hand-over (sampler reads the trainer's buffer); seconds = 0 by construction, see --topology disaggregated"},
                "clocks": clocks.read(),
                "e2e": {"value": g_tok / (g_host / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d // k,
                        "d2h_bytes_per_step": d2h // k},
                "gpu_launches": int(C.LAUNCH_COUNT - launches0),
                "phase_seconds_per_step": {kk: v / k for kk, v in phase.items()},
                "last_step": {kk: last.get(kk) for kk in ("loss", "grad_norm", "sampler_probs_diff_mean", "entropy")},
                "peak_mem_gib": torch.cuda.max_memory_allocated(dev) / 2 ** 30,
                "runner": {kk: runner.phase_detail.get(kk) for kk in ("kv_pages", "kv_peak_pages", "offloaded", "recompute", "preempted", "decode_steps",
                                                                            "decode_host_prep_s")},
                "multi_gpu_checks": checks,
                "wall_s_since_start": time.time() - T_PROCESS_START,
            }
            print(json.dumps(out), flush=True)
    barrier()
    C.check_status()
    clk = clocks.stop() if rank == 0 else None
    if args.ab_nccl and world > 1 and runner.policy.fused is not None:
        # one extra step on the NCCL collectives (reduce-scatter + all-gather) for comparison
        fused, runner.policy.fused = runner.policy.fused, None
        caps, rewards = make_inputs()
        runner.step(pinned, response_caps=caps, rewards=rewards)
        runner.policy.fused = fused
        nccl_train = agree(runner.timing["train"], dist.ReduceOp.MAX)
        if rank == 0 and out is not None:
            out["multi_gpu_checks"]["train_seconds_nccl_optimizer_path"] = nccl_train
            out["multi_gpu_checks"]["train_seconds_fused_optimizer_path"] = out["phase_seconds_per_step"]["train"]
    if rank == 0 and out is not None:
        out["clocks"] = clk
        out["final"] = True
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
