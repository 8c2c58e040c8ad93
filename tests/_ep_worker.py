"""Expert-parallel MoE model against the unsharded model; W ranks (gloo on CPU, nccl on GPUs)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(out_path: str, device_kind: str) -> None:
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
    from axon_b200.parallel.ep import EPContext
    cfg = get_config(preset)
    g = torch.Generator().manual_seed(0)
    per_rank = [[torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in lens] for lens in ((90, 41), (33, 120, 17), (64,), (10, 75))]
    mine = per_rank[rank]
    full = MoEModel(cfg, device=dev, dtype=dtype)
    full.params.init_random(std=0.05, seed=21)
    # reference: the unsharded model on every rank's tokens (gradients add up over the ranks' batches)
    full.params.alloc_grads()
    full.params.zero_grads()
    ref_lp, routing = {}, {}
    for r in range(world):
        pb = PackedBatch.from_sequences(per_rank[r], dev)
        gg = torch.Generator().manual_seed(100 + r)
        T = pb.input_ids.numel()
        glp = torch.randn(T, generator=gg).to(dev) * (pb.labels >= 0).float()
        full.capture_routing, full.last_routing = True, None
        lp, ent = full.forward(pb, 1.0, save_for_backward=True)
        routing[r] = torch.stack(full.last_routing, 1)
        full.capture_routing = False
        full.backward(glp, None)
        ref_lp[r] = lp
    T_max = max(sum(s.numel() for s in seqs) for seqs in per_rank[:world])
    ep = EPContext(dist.group.WORLD, dev, cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size, max_tokens=T_max,
                   top_k=cfg.num_experts_per_tok)
    m = MoEModel(cfg, device=dev, dtype=dtype, ep=ep)
    m.load_full_state(full.params.views)
    m.params.alloc_grads()
    m.params.zero_grads()
    pb = PackedBatch.from_sequences(mine, dev)
    pb.routermap = routing[rank]                     # same expert choice as the reference run (bf16 ties aside)
    gg = torch.Generator().manual_seed(100 + rank)
    T = pb.input_ids.numel()
    glp = torch.randn(T, generator=gg).to(dev) * (pb.labels >= 0).float()
    # ranks have different token counts but must run the same number of collective phases: one batch each
    lp, ent = m.forward(pb, 1.0, save_for_backward=True)
    m.backward(glp, None)
    if dev.type == "cuda":
        torch.cuda.synchronize()
        from axon_b200.ops import _common as C
        C.check_status()
    # sum the partial gradients of the replicated parameters over the ranks
    res = {"fused": ep.fused, "lp_err": float((lp.float() - ref_lp[rank].float()).abs().max()), "grad_rel": {}}
    for name, gsh in m.params.grads.items():
        gsh = gsh.float().clone()
        ref = full.params.grads[name].float()
        if name.endswith("w13_weight") or name.endswith("w2_weight"):
            ref = ref[ep.local_experts()]
        else:
            dist.all_reduce(gsh)
        res["grad_rel"][name] = float((gsh - ref).norm() / (ref.norm() + 1e-12))
    out = [None] * world
    dist.all_gather_object(out, res)
    if rank == 0:
        json.dump(out, open(out_path, "w"))
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
