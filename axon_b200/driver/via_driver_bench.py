"""``bench.py --via-driver``: what the full product path costs over the single-process runner.

The headline benchmark drives ``ColocatedRLRunner`` (one process: sampler engine, policy engine, zero-copy weight
hand-over). The path a user of the framework takes is longer: ``train_agent`` -> ``SyncPPO`` -> worker groups ->
``Engine`` (program pool, prefix tree, chat template, tokenizer) -> ``ReactProgram`` -> sampler server -> trainer
worker (reference: axon/driver/sync_ppo.py:149-179,285-454). This arm runs the SAME model on a workload both paths can
express - fixed-length responses, since the driver gives every request the same token cap - first through the
driver, then through the runner, and reports both rates and their ratio. It is a diagnostic, not the headline number:
the line carries ``"metric": "... via driver"`` and a ``via_driver`` block.
"""
from __future__ import annotations

import json
import os
import random
import tempfile
import time


def _dataset(path: str, rows: int, prompt_chars: int, seed: int) -> None:
    rng = random.Random(seed)
    words = ["alpha", "beta", "gamma", "delta", "river", "stone", "cloud", "ember", "north", "quiet", "seven", "amber"]
    with open(path, "w") as f:
        for i in range(rows):
            text = []
            n = 0
            while n < prompt_chars:
                w = rng.choice(words)
                text.append(w)
                n += len(w) + 1
            f.write(json.dumps({"question": " ".join(text)[:prompt_chars], "ground_truth": str(i), "data_source": "synthetic",
                                "reward_fn": "bernoulli"}) + "\n")


def _driver_arm(a: dict, out_path: str) -> None:
    """The driver half, in a process of its own (so that all of its device memory is gone before the runner half)."""
    import numpy as np
    import torch
    from ..ops import _common as C
    from ..utils.config import compose_config
    from .train_agent_ppo import train_agent
    P, G, R, warm, timed, tmp = a["P"], a["G"], a["R"], a["warm"], a["timed"], a["tmp"]
    data = os.path.join(tmp, "train.jsonl")
    _dataset(data, P * (warm + timed + 1), a["prompt_len"], a["seed"])
    os.environ["AXON_FILE_LOGGER_ROOT"] = tmp
    cfg = compose_config([
        f"train_files={data}", f"model_path={a['model']}", f"train_batch_size={P}", f"decoding.n={G}", f"mini_batch_size={P}",
        f"max_prompt_length={a['prompt_len'] + 128}", f"max_seq_length={a['prompt_len'] + 128 + R}", f"max_tokens_per_step={R}",
        f"output_dir={tmp}/out", "advantage=grpo", "validation.before_train=false", "drop_zero_advantage_samples=false",
        f"actor.max_token_len_per_gpu={a['micro_batch_tokens']}", "save_programs_flag=false", "logger=[file]", "num_gpus_per_node=1",
        f"total_training_steps={warm + timed}", "save_steps=-1", "resume_from_checkpoint=false", "+decoding.ignore_eos=true",
        f"sampler.max_num_seqs={P * G}"] + ([] if torch.cuda.is_available() else ["+force_cpu=true"]))
    launches0 = C.LAUNCH_COUNT
    t0 = time.perf_counter()
    drv = train_agent(cfg, backend="inline", keep_alive=True)
    drv.shutdown()
    wall = time.perf_counter() - t0
    logs = [json.loads(line) for line in open(os.path.join(tmp, "axon-agent_ppo.jsonl"))]
    steps = [r["data"] for r in logs][warm:]
    out = {"s_per_step": float(np.mean([s["timing_s/step"] for s in steps])),
           "tokens_per_step": float(np.mean([s["perf/throughput_tokens_per_s"] * s["timing_s/step"] for s in steps])),
           "phase": {k[len("timing_s/"):]: float(np.mean([s[k] for s in steps])) for k in steps[0] if k.startswith("timing_s/")},
           "prompt_tokens": float(np.mean([s.get("prompt_length/mean", a["prompt_len"]) for s in steps])),
           "launches": int(C.LAUNCH_COUNT - launches0), "wall_s": wall, "steps": len(steps)}
    with open(out_path, "w") as f:
        json.dump(out, f)


def run_via_driver(args, t_process_start: float, ClockSampler) -> None:
    import subprocess
    import sys
    import numpy as np
    import torch
    from ..driver.colocated import ColocatedRLRunner, RLStepConfig
    from ..models.config import get_config
    assert args.gpus == 1, "--via-driver compares the two single-GPU paths"
    P, G, R = args.prompts_per_gpu, args.group, int(args.fixed_response)
    warm, timed = max(1, min(args.warmup, 1)), max(1, min(args.steps, 2))
    tmp = tempfile.mkdtemp(prefix="axb_via_driver_")
    clocks = ClockSampler(0)
    clocks.start()
    arm = {"P": P, "G": G, "R": R, "warm": warm, "timed": timed, "tmp": tmp, "prompt_len": args.prompt_len, "seed": args.seed,
           "model": args.model, "micro_batch_tokens": args.micro_batch_tokens}
    out_path = os.path.join(tmp, "driver_arm.json")
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-c", "import json, sys; from axon_b200.driver.via_driver_bench import _driver_arm; "
                        "_driver_arm(json.loads(sys.argv[1]), sys.argv[2])", json.dumps(arm), out_path], cwd=root,
                       stdout=sys.stderr, stderr=sys.stderr)
    if r.returncode != 0 or not os.path.exists(out_path):
        raise RuntimeError(f"the driver arm failed with exit code {r.returncode}")
    d = json.load(open(out_path))
    d_step, d_tok, d_phase = d["s_per_step"], d["tokens_per_step"], d["phase"]
    driver_wall, driver_launches = d["wall_s"], d["launches"]
    prompt_tokens = int(d["prompt_tokens"])
    on_gpu = torch.cuda.is_available()

    # ---- the runner on the same shape of work: P prompts x G samples, every response exactly R tokens
    from ..models.dense import DenseModel
    mcfg = get_config(args.model)
    model = DenseModel(mcfg, device="cuda" if on_gpu else "cpu", dtype=torch.bfloat16 if on_gpu else torch.float32)
    model.params.init_random(std=0.02, seed=args.seed)
    from ..trainer.policy import OptimConfig
    rl = RLStepConfig(n_samples=G, max_prompt_length=args.prompt_len + 128, max_response_length=R, temperature=1.0, loss="ppo",
                      loss_args={"clip_ratio": 0.2}, advantage="grpo", mini_batch_size=P, max_token_len_per_gpu=args.micro_batch_tokens,
                      max_num_seqs=P * G, optim=OptimConfig(lr=1e-6, weight_decay=0.1, grad_clip=1.0))
    runner = ColocatedRLRunner(model, rl, None, seed=args.seed)
    rng = np.random.default_rng(args.seed)
    r_times, r_tokens = [], []
    for i in range(warm + timed):
        prompts = rng.integers(0, mcfg.vocab_size, (P, prompt_tokens), dtype=np.int32)
        caps = np.full(P * G, R, dtype=np.int64)
        rewards = rng.binomial(1, 0.3, P * G).astype(np.float32)
        if on_gpu:
            torch.cuda.synchronize()
        a = time.perf_counter()
        host = torch.from_numpy(prompts)
        out = runner.step(host.pin_memory() if on_gpu else host, response_caps=caps, rewards=rewards)
        if on_gpu:
            torch.cuda.synchronize()
        if i >= warm:
            r_times.append(time.perf_counter() - a)
            r_tokens.append(float(out["tokens"]))
    r_step, r_tok = float(np.mean(r_times)), float(np.mean(r_tokens))
    line = {"metric": "RL step tokens/sec via driver (diagnostic: full product path vs single-process runner)",
            "value": d_tok / d_step, "unit": "tokens/s", "n_gpus": 1, "steps": int(d["steps"]), "warmup": warm, "ms_per_step": d_step * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (word-salad prompts through the byte tokenizer and chat template, fixed-length responses, random-init weights)",
            "config": {"model": args.model, "prompts": P, "group": G, "prompt_tokens": prompt_tokens, "response_tokens": R,
                       "micro_batch_tokens": args.micro_batch_tokens, "parallelism": "1 GPU colocated"},
            "clocks": clocks.stop(), "gpu_launches": int(driver_launches),
            "via_driver": {"driver_tokens_per_s": d_tok / d_step, "driver_s_per_step": d_step, "driver_tokens_per_step": d_tok,
                           "driver_phase_seconds": d_phase, "driver_wall_s_with_init": driver_wall,
                           "runner_tokens_per_s": r_tok / r_step, "runner_s_per_step": r_step, "runner_tokens_per_step": r_tok,
                           "driver_over_runner_time": d_step / r_step if r_step else None},
            "wall_s_since_start": time.time() - t_process_start, "final": True}
    print(json.dumps(line), flush=True)
