"""Decode-step time of a tensor-parallel sampler group and latency of its activation sum.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 --master-port P \\
        -m axon_b200.sampler.tp_bench --model qwen3-8b --batch 256 --prompt 1000 --steps 64 --out FILE.json

Every rank builds its shard of the model (random weights), the group prefills ``batch`` prompts of ``prompt`` tokens
and decodes; timed are ``steps`` decode steps after the decode graph exists (synchronise on both sides, maximum over
ranks). The second part times the sum of a [batch, hidden] bf16 tensor over the group, once through the
peer-memory kernel and once through the process group's all-reduce (CUDA events, 200 calls each after 20 warm-up
calls, maximum over ranks). With W = 1 only the decode part runs (the single-GPU figure to compare with).
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--prompt", type=int, default=1000)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from ..models.config import get_config
    from ..models.moe import build_model_for
    from ..models.tp_infer import Shard, ShardedDenseModel, ShardedMoEModel
    from ..ops import _common as C
    from .engine import GenerationEngine
    from .params import SamplingParams
    cfg = get_config(a.model)
    group = dist.new_group(list(range(world)))
    shard = Shard.create(group, dev)
    if world > 1:
        model = (ShardedMoEModel if cfg.num_experts else ShardedDenseModel)(cfg, shard, device=dev, dtype=torch.bfloat16)
        model.params.init_random(seed=1)
        model.share_replicated_from_first_rank()
    else:
        model = build_model_for(cfg, dev, torch.bfloat16)
        model.params.init_random(seed=1)
    pages = a.batch * ((a.prompt + a.steps + 40 + 127) // 128 + 1)
    eng = GenerationEngine(model, num_pages=pages, max_num_seqs=a.batch, max_num_batched_tokens=32768, seed=3)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(2, cfg.vocab_size, (a.prompt,), generator=g).tolist() for _ in range(a.batch)]
    sp = SamplingParams(temperature=1.0, max_tokens=a.steps + 24, ignore_eos=True)
    for p in prompts:
        eng.add_request(p, sp)
    while eng.stats["decode_steps"] < 8:                 # prefill everything, then a few decode steps (graph capture)
        eng.step()
    torch.cuda.synchronize()
    dist.barrier(group=group)
    t0 = time.perf_counter()
    for _ in range(a.steps):
        eng.step()
    torch.cuda.synchronize()
    dt = torch.tensor([(time.perf_counter() - t0) / a.steps * 1e3], device=dev)
    dist.all_reduce(dt, op=dist.ReduceOp.MAX, group=group)
    res = {"model": a.model, "world": world, "batch": a.batch, "context": a.prompt + 8 + a.steps // 2, "decode_step_ms": round(float(dt.item()), 3),
           "running": len(eng.running), "graphs": len(eng._graphs), "reduce_calls": dict(shard.reduce.calls)}
    if world > 1:
        x = torch.randn(a.batch, cfg.hidden_size, device=dev).to(torch.bfloat16)

        def timed(fn):
            for _ in range(20):
                fn()
            torch.cuda.synchronize()
            dist.barrier(group=group)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(200):
                fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / 200 * 1e3], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            return round(float(t.item()), 2)
        shard.reduce.begin_step()
        res["sum_bytes"] = x.numel() * 2
        res["sum_peer_kernel_us"] = timed(lambda: shard.reduce(x.mul_(0.5)))          # the scaling keeps the values finite
        res["sum_process_group_us"] = timed(lambda: dist.all_reduce(x.mul_(0.5), group=group))
        res["scale_only_us"] = timed(lambda: x.mul_(0.5))
    C.check_status()
    if rank == 0:
        print(json.dumps(res))
        if a.out:
            with open(a.out, "w") as f:
                json.dump(res, f)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
