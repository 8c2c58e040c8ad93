"""Tensor- plus expert-parallel sparse model (one group) against the unsharded model; W ranks (gloo / nccl)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(out_path: str, device_kind: str, how: str = "ep") -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if device_kind == "cuda":
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=dev)
        dtype, preset = torch.bfloat16, "tiny-moe-gpu"
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        dtype, preset = torch.float32, "tiny-moe"
    from axon_b200.models.config import get_config
    from axon_b200.models.dense import PackedBatch
    from axon_b200.models.moe import MoEModel
    from axon_b200.models.tp_dense import pad_packed_batch, slice_full_param
    from axon_b200.models.tp_moe import TPMoEModel
    from axon_b200.parallel.ep import EPContext
    from axon_b200.parallel.tp import TPContext
    cfg = get_config(preset)
    g = torch.Generator().manual_seed(0)
    seqs = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (150, 97, 260)]
    full = MoEModel(cfg, device=dev, dtype=dtype)
    full.params.init_random(std=0.05, seed=11)
    pb, T_real = pad_packed_batch(PackedBatch.from_sequences(seqs, dev), 128 * world)
    T = pb.input_ids.numel()
    glp = torch.randn(T, generator=g).to(dev) * (pb.labels >= 0).float()
    gent = (torch.randn(T, generator=g) * 0.1).to(dev)
    gent[T_real:] = 0
    full.params.alloc_grads()
    full.capture_routing, full.last_routing = True, None
    lp_f, ent_f = full.forward(pb, 1.0, save_for_backward=True)
    routing = torch.stack(full.last_routing, 1)
    full.capture_routing = False
    full.backward(glp, gent)
    tp = TPContext(dist.group.WORLD, dev, max_rows_per_rank=T // world, max_width=max(cfg.qkv_size, cfg.hidden_size))
    # "ep": whole experts per rank, tokens travel; "etp": a slice of every expert per rank, all ranks see all tokens
    ep = EPContext(dist.group.WORLD, dev, cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size, max_tokens=T // world,
                   top_k=cfg.num_experts_per_tok) if how == "ep" else None
    m = TPMoEModel(cfg, tp, ep, device=dev, dtype=dtype)
    m.load_full_state(full.params.views)
    m.params.alloc_grads()
    pb.routermap = routing                      # same expert choice as the reference run (bf16 near-ties aside)
    lp, ent = m.forward(pb, 1.0, save_for_backward=True)
    sl = m.local_slice(T)
    m.backward(glp[sl], gent[sl])
    m.sync_replicated_grads()
    if dev.type == "cuda":
        torch.cuda.synchronize()
        from axon_b200.ops import _common as C
        C.check_status()
    res = {"fused": tp.fused, "ep_fused": ep.fused if ep is not None else None, "lp_err": float((lp.float() - lp_f[sl].float()).abs().max()),
           "ent_err": float((ent.float() - ent_f[sl].float()).abs().max()), "grad_rel": {}}
    for name, gsh in m.params.grads.items():
        kw = dict(ep=world, ep_rank=rank) if how == "ep" else dict(etp=world, etp_rank=rank)
        ref = slice_full_param(cfg, name, full.params.grads[name], world, rank, False, **kw).float()
        res["grad_rel"][name] = float((gsh.float() - ref).norm() / (ref.norm() + 1e-12))
    ss = m.grad_sumsq().reshape(1).to(dev)
    dist.all_reduce(ss)
    res["norm_rel"] = abs(float(ss.sqrt()) - float(full.params.grad_flat.double().norm())) / float(full.params.grad_flat.double().norm())
    # without a record the model routes by itself and says what it chose
    m.capture_routing, m.last_routing = True, None
    pb.routermap = None
    m.forward(pb, 1.0)
    res["routing_equal"] = bool(torch.equal(torch.stack(m.last_routing, 1)[: max(0, min(T_real, sl.stop) - sl.start)].sort(-1).values,
                                            routing[sl][: max(0, min(T_real, sl.stop) - sl.start)].sort(-1).values))
    out = [None] * world
    dist.all_gather_object(out, res)
    if rank == 0:
        json.dump(out, open(out_path, "w"))
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2], sys.argv[3] if len(sys.argv) > 3 else "ep")
