"""Multi-GPU worker run under torch.distributed.run by tests/test_multi_gpu.py. Writes a JSON verdict."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(out_path: str) -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from axon_b200.ops import _common as C
    from axon_b200.parallel.symm import PeerBarrier, SymmetricBuffer
    from axon_b200.parallel.zero1 import FusedZero1
    res = {}

    # 1. device barrier + peer visibility
    buf = SymmetricBuffer(1024, torch.float32)
    buf.tensor.fill_(float(rank + 1))
    bar = PeerBarrier()
    bar()
    seen = [float(buf.peer_tensor(r)[0].item()) for r in range(world)]
    res["peer_values"] = seen
    bar()

    # 2. fused ZeRO-1 step vs NCCL reduce-scatter + torch AdamW + all-gather
    n = 128 * world * 2048
    torch.manual_seed(1234)
    init = torch.randn(n, device=dev) * 0.1
    torch.manual_seed(100 + rank)
    grad = torch.randn(n, device=dev)
    z = FusedZero1(n)
    z.grads.tensor.copy_(grad)
    z.params.tensor.copy_(init.to(torch.bfloat16))
    master = init[z.lo:z.lo + z.n].clone()
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    state = z.step(master, m, v, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1, max_norm=1.0)
    torch.cuda.synchronize()
    g_sum = grad.clone()
    dist.all_reduce(g_sum)
    norm = g_sum.norm()
    coef = min(1.0, 1.0 / (float(norm) + 1e-6))
    ref = torch.nn.Parameter(init.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref.grad = g_sum * coef
    opt.step()
    res["zero1_norm_err"] = abs(float(state[1]) - float(norm)) / float(norm)
    res["zero1_param_err"] = float((z.params.tensor.float() - ref.detach()).abs().max())
    res["zero1_master_err"] = float((master - ref.detach()[z.lo:z.lo + z.n]).abs().max())

    # 3. weight-sync plan: trainer ranks push re-sliced shards straight into the sampler ranks' buffers
    from axon_b200.models.config import ModelConfig
    from axon_b200.models.params import param_layout
    from axon_b200.utils.p2p.param_mapper import get_param_metadata, shard_rows
    from axon_b200.utils.p2p.plan import compile_plan, execute_plan
    from axon_b200.utils.p2p.routing_table import RoutingTable
    cfg = ModelConfig(vocab_size=1024, hidden_size=512, num_hidden_layers=2, num_attention_heads=8,
                      num_key_value_heads=4, head_dim=64, intermediate_size=1024)
    g = torch.Generator().manual_seed(7)
    full = {k: torch.randn(*s, generator=g).to(torch.bfloat16) for k, s in param_layout(cfg).items()}

    def side(tp, tpr):
        chunks, off, offs = [], 0, {}
        for name, t in full.items():
            t2 = t.reshape(t.shape[0], -1) if t.dim() > 1 else t.reshape(-1, 1)
            sh = torch.cat([t2[a:b, c:d].reshape(-1) for a, b, c, d in shard_rows(cfg, name, tp, tpr)])
            offs[name] = off
            pad = (-sh.numel()) % 128
            chunks += [sh, torch.zeros(pad, dtype=sh.dtype)]
            off += sh.numel() + pad
        return torch.cat(chunks), offs
    # trainer: every rank holds the full model (tp1, dp=world); sampler: tp=world over the same GPUs
    a_flat, a_offs = side(1, 0)
    s_flat, s_offs = side(world, rank)
    table = RoutingTable([get_param_metadata(cfg, r, 1, 0) for r in range(world)],
                         [get_param_metadata(cfg, r, world, r) for r in range(world)])
    all_s_offs = {r: side(world, r)[1] for r in range(world)}
    dst = SymmetricBuffer(max(side(world, r)[0].numel() for r in range(world)), torch.bfloat16)
    dst.tensor.zero_()
    bar()
    plan = compile_plan(table, rank, a_offs, all_s_offs)
    src = a_flat.to(dev)
    execute_plan(plan, src, [None] * world, dst_ptrs=dst.ptrs)
    torch.cuda.synchronize()
    bar()
    torch.cuda.synchronize()
    res["sync_exact"] = bool(torch.equal(dst.tensor[: s_flat.numel()].cpu(), s_flat))
    res["sync_bytes_sent"] = plan.total_bytes
    # bandwidth of the plan kernel on a large buffer (push to the next rank)
    big = 256 << 20
    sb = SymmetricBuffer(big // 2, torch.bfloat16)
    import numpy as np
    from axon_b200.utils.p2p.plan import DESC_DTYPE, SyncPlan
    d = np.zeros(1, dtype=DESC_DTYPE)
    d["rows"], d["cols"], d["src_stride"], d["dst_stride"], d["dst_rank"] = 1 << 14, big // 2 >> 14, big // 2 >> 14, big // 2 >> 14, (rank + 1) % world
    per = d["rows"].astype(np.int64) * (d["cols"].astype(np.int64) // 8)
    p2 = SyncPlan(d, np.zeros(1, np.int64), int(per.sum()), big)
    srcb = torch.randn(big // 2, device=dev).to(torch.bfloat16)
    for _ in range(3):
        execute_plan(p2, srcb, [None] * world, dst_ptrs=sb.ptrs)
    torch.cuda.synchronize()
    bar()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        execute_plan(p2, srcb, [None] * world, dst_ptrs=sb.ptrs)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / 5], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res["sync_push_gbs"] = big / (float(t) * 1e-3) / 1e9
    # 4. policy engine: optimizer step through the fused peer-memory path vs the NCCL path
    from axon_b200.models.config import get_config
    from axon_b200.models.dense import DenseModel
    from axon_b200.protocol import DataProto
    from axon_b200.trainer.policy import OptimConfig, PolicyEngine
    mcfg = get_config("tiny-gpu")
    engines = []
    for fused in (True, False):
        mdl = DenseModel(mcfg, device=dev, dtype=torch.bfloat16)
        mdl.params.init_random(seed=5)
        engines.append(PolicyEngine(mdl, OptimConfig(lr=1e-3, grad_clip=1.0), process_group=dist.group.WORLD,
                                    max_token_len_per_gpu=512, fused_zero1=fused))
    res["engine_fused_active"] = engines[0].fused is not None and engines[1].fused is None
    gen = torch.Generator().manual_seed(50 + rank)
    B, T = 4, 96
    ids = torch.randint(0, mcfg.vocab_size, (B, T), generator=gen)
    att = torch.ones(B, T, dtype=torch.long)
    att[0, 70:] = 0
    rmask = att.clone().float()
    rmask[:, :16] = 0
    for step in range(2):
        for e in engines:
            data = DataProto.from_dict({"input_ids": ids, "attention_mask": att, "response_mask": rmask,
                                        "advantages": torch.randn(B, T, generator=torch.Generator().manual_seed(step)) * rmask,
                                        "old_log_probs": torch.zeros(B, T)})
            data.batch["old_log_probs"] = e.forward(data, want_entropy=False).batch["log_probs"].cpu()
            data.meta_info["temperature"] = 1.0
            e.forward_backward(data, "ppo", {"clip_ratio": 0.2})
            out = e.optim_step()
            res.setdefault("engine_norms", []).append(out["grad_norm"])
    torch.cuda.synchronize()
    a, b = engines[0].model.params.flat.float(), engines[1].model.params.flat.float()
    res["engine_param_diff"] = float((a - b).abs().max())
    res["engine_param_moved"] = float((a - DenseModel(mcfg, device=dev).params.flat.float()).abs().max()) > 0
    chk = a.double().sum().reshape(1)
    allc = [torch.zeros_like(chk) for _ in range(world)]
    dist.all_gather(allc, chk)
    res["engine_replicas_equal"] = all(float(c) == float(allc[0]) for c in allc)
    bar()
    torch.cuda.synchronize()
    C.check_status()
    res["status_ok"] = True
    gathered = [None] * world
    dist.all_gather_object(gathered, res)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(gathered, f)
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
