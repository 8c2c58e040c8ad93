"""Timed multi-GPU workloads of the fused compute + collective paths, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m axon_b200.utils.profiler.multi_rank_cases <case> [--iters K]

Cases: ``tp`` (all-gather -> GEMM and GEMM -> reduce-scatter at Qwen3-8B projection shapes against the same
products on whole operands), ``zero3`` (forward + backward of 4 Qwen3-8B layers with parameter shards gathered
inside the GEMMs against whole parameters), ``sync`` (the weight-sync plan kernel pushing a parameter-sized
buffer to the next rank). Every number is the median of CUDA-event timings, taken as the MAX over ranks; rank 0
prints one JSON line with the time, the roofline bound (the slower of FLOPs at the given GEMM rate and bytes at
the given link rate) and achieved / bound. Never run these under a profiler: the ranks wait on one another.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _timed(fn, iters: int, dev) -> float:
    ts = []
    for _ in range(iters + 2):
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    t = torch.tensor(sorted(ts[2:])[len(ts[2:]) // 2], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def case_tp(world, rank, dev, iters, peaks):
    from ...ops import gemm as G
    from ...parallel.tp import TPContext
    Tt, H, Nq = 8192, 4096, 6144
    tp = TPContext(dist.group.WORLD, dev, max_rows_per_rank=Tt // world, max_width=Nq)
    x_loc = torch.randn(Tt // world, H, device=dev).to(torch.bfloat16)
    x_all = torch.randn(Tt, H, device=dev).to(torch.bfloat16)
    w_col = (torch.randn(Nq // world, H, device=dev) * 0.02).to(torch.bfloat16)       # column-parallel shard
    a_all = torch.randn(Tt, H // world, device=dev).to(torch.bfloat16)
    w_row = (torch.randn(H, H // world, device=dev) * 0.02).to(torch.bfloat16)        # row-parallel shard
    out = {}
    out["ms_allgather_gemm_fused"] = _timed(lambda: tp.allgather_gemm(x_loc, w_col), iters, dev)
    out["ms_gemm_whole_rows"] = _timed(lambda: G.gemm_nt(x_all, w_col), iters, dev)
    out["ms_gemm_reduce_scatter_fused"] = _timed(lambda: tp.gemm_reduce_scatter(a_all, w_row), iters, dev)
    out["ms_gemm_partial_only"] = _timed(lambda: G.gemm_nt(a_all, w_row), iters, dev)
    ag_flops, ag_bytes = 2.0 * Tt * (Nq // world) * H, 2.0 * (world - 1) * (Tt // world) * H
    rs_flops, rs_bytes = 2.0 * Tt * H * (H // world), 2.0 * (world - 1) * (Tt // world) * H
    for key, fl, by in (("allgather_gemm", ag_flops, ag_bytes), ("gemm_reduce_scatter", rs_flops, rs_bytes)):
        bound = max(fl / (peaks["tflops"] * 1e12), by / (peaks["link_gbs"] * 1e9)) * 1e3
        out[f"bound_ms_{key}"] = bound
        out[f"roofline_fraction_{key}"] = bound / out[f"ms_{key}_fused"]
    return out


def case_zero3(world, rank, dev, iters, peaks):
    from ...models.config import qwen3_8b
    from ...models.dense import DenseModel, PackedBatch
    from ...models.zero3_dense import Zero3DenseModel
    from ...parallel.zero3 import ShardContext
    big = qwen3_8b()
    big.num_hidden_layers = 4
    ctx = ShardContext(dist.group.WORLD, dev)
    seqs = [torch.randint(0, big.vocab_size, (2048,)) for _ in range(4)]
    batch = PackedBatch.from_sequences(seqs, dev)
    glp = torch.ones(batch.input_ids.numel(), device=dev)
    out = {}
    for label, build in (("whole", lambda: DenseModel(big, device=dev)), ("sharded", lambda: Zero3DenseModel(big, ctx, device=dev))):
        mod = build()
        (mod.params.init_random if label == "whole" else mod.init_random)(std=0.02, seed=3)
        mod.recompute = "selective"
        mod.params.alloc_grads()

        def step(mod=mod):
            mod.forward(batch, 1.0, save_for_backward=True)
            mod.backward(glp, None)
        out[f"ms_fwd_bwd_{label}"] = _timed(step, iters, dev)
        del mod
        torch.cuda.empty_cache()
    return out


def case_sync(world, rank, dev, iters, peaks):
    import numpy as np

    from ...parallel.symm import SymmetricBuffer
    from ...utils.p2p.plan import copy_desc, execute_plan, plan_from_descs
    n = 1 << 30                                                      # 2 GiB of bf16 per rank
    dst = SymmetricBuffer(n, torch.bfloat16)
    src = torch.randn(n // 4, device=dev).to(torch.bfloat16).repeat(4)
    cols = 1 << 14
    plan = plan_from_descs([copy_desc(0, 0, n // cols, cols, cols, cols, (rank + 1) % world)])
    ms = _timed(lambda: execute_plan(plan, src, [None] * world, dst_ptrs=dst.ptrs), iters, dev)
    ok = bool(torch.equal(dst.tensor[: 1 << 20].cpu(), src[: 1 << 20].cpu())) if world == 1 else True
    gbs = 2.0 * n / (ms * 1e-3) / 1e9
    del np
    return {"ms_push_2gib": ms, "gbs_per_gpu": gbs, "fraction_of_link": gbs / peaks["link_gbs"], "checked": ok}


CASES = {"tp": case_tp, "zero3": case_zero3, "sync": case_sync}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--iters", type=int, default=7)
    ap.add_argument("--peak-tflops", type=float, default=float(os.environ.get("AXON_PEAK_TFLOPS", 1590.0)))
    ap.add_argument("--link-gbs", type=float, default=float(os.environ.get("AXON_LINK_GBS", 770.0)))
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from ...ops import _common as C
    res = CASES[args.case](world, rank, dev, args.iters, {"tflops": args.peak_tflops, "link_gbs": args.link_gbs})
    torch.cuda.synchronize()
    C.check_status()
    if rank == 0:
        print(json.dumps({"case": args.case, "world": world, **res}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
