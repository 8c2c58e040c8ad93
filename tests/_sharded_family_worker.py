"""A family model with parameter shards against the unsharded model; W gloo ranks with different data each."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(out_path: str, presets: str) -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    from axon_b200.models.config import get_config
    from axon_b200.models.dense import PackedBatch
    from axon_b200.models.families import FamilyModel
    from axon_b200.models.sharded_family import ShardedFamilyModel, shard_key
    from axon_b200.parallel.zero3 import ShardContext
    res = {"rank": rank}
    for preset in presets.split(","):
        cfg = get_config(preset)
        full = FamilyModel(cfg, device="cpu", dtype=torch.float32)
        full.init_random(std=0.05, seed=11)
        g = torch.Generator().manual_seed(0)
        per_rank = [[torch.randint(2, cfg.vocab_size, (n,), generator=g) for n in lens] for lens in ((40, 21), (33, 17, 9), (25,), (10, 31))]
        # reference: the unsharded model on every rank's batch; gradients add up
        full.params.alloc_grads()
        ref_lp = {}
        for r in range(world):
            pb = PackedBatch.from_sequences(per_rank[r], "cpu")
            gg = torch.Generator().manual_seed(100 + r)
            glp = torch.randn(pb.input_ids.numel(), generator=gg) * (pb.labels >= 0).float()
            lp, ent = full.forward(pb, 1.0, save_for_backward=True)
            full.backward(glp, torch.full_like(glp, 0.01))
            ref_lp[r] = lp
        m = ShardedFamilyModel(cfg, ShardContext(dist.group.WORLD, "cpu"), device="cpu", dtype=torch.float32)
        m.load_full_state(full.params.views)
        pb = PackedBatch.from_sequences(per_rank[rank], "cpu")
        gg = torch.Generator().manual_seed(100 + rank)
        glp = torch.randn(pb.input_ids.numel(), generator=gg) * (pb.labels >= 0).float()
        lp, ent = m.forward(pb, 1.0, save_for_backward=True)
        m.backward(glp, torch.full_like(glp, 0.01))
        m.sync_replicated_grads()
        worst, worst_name = 0.0, ""
        for name, gsh in m.params.grads.items():
            if name in m.full_layout:
                ref = full.params.grads[name]
                err = float((gsh - ref).norm() / (ref.norm() + 1e-9))
                if err > worst:
                    worst, worst_name = err, name
        for l, table in m.layer_offsets.items():
            n = m.layer_len[l] // world
            piece = m.params.grads[shard_key(l)]
            for name, (o, k, shape) in table.items():
                a, b = max(o, rank * n), min(o + k, (rank + 1) * n)
                if b <= a:
                    continue
                ref = full.params.grads[name].reshape(-1)[a - o:b - o]
                err = float((piece[a - rank * n:b - rank * n] - ref).norm() / (ref.norm() + 1e-9))
                if err > worst:
                    worst, worst_name = err, name
        whole = {n: t.clone() for n, t in m.full_named_tensors()}
        res[preset] = {"lp_err": float((lp - ref_lp[rank]).abs().max()), "grad_rel": worst, "grad_name": worst_name,
                       "gathered_equal": all(torch.equal(whole[n].reshape(-1), full.params.views[n].reshape(-1)) for n in full.layout),
                       "piece_grad_norm": float(sum(m.params.grads[shard_key(l)].norm() for l in m.layer_offsets)),
                       "local_numel": int(m.params.numel), "full_numel": int(full.params.numel)}
    out = [None] * world
    dist.all_gather_object(out, res)
    if rank == 0:
        json.dump(out, open(out_path, "w"))
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
