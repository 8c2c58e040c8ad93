"""Parameter-sharded model against the unsharded model on W GPUs (nccl): every rank runs its own batch through
the fused weight-gather GEMMs; log-probs and the summed gradients must match one model that saw all batches."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(out_path: str) -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    from axon_b200.models.config import get_config
    from axon_b200.models.dense import DenseModel, PackedBatch
    from axon_b200.models.zero3_dense import Zero3DenseModel
    from axon_b200.ops import _common as C
    from axon_b200.parallel.zero3 import ShardContext, is_sharded
    cfg = get_config("tiny-gpu")
    res = {}
    full = DenseModel(cfg, device=dev)
    full.params.init_random(std=0.05, seed=11)
    full.recompute = "full"
    full.params.alloc_grads()
    ctx = ShardContext(dist.group.WORLD, dev)
    m = Zero3DenseModel(cfg, ctx, device=dev)
    m.init_random(std=0.05, seed=11)
    m.recompute = "full"
    m.params.alloc_grads()
    res["fused"] = ctx.fused
    lp_err = ent_err = 0.0
    for r in range(world):                       # the reference model sees every rank's batch
        gg = torch.Generator().manual_seed(5 + r)
        seqs = [torch.randint(0, cfg.vocab_size, (n,), generator=gg) for n in (150 + 7 * r, 97, 260 - 3 * r)]
        batch = PackedBatch.from_sequences(seqs, dev)
        T = batch.input_ids.numel()
        glp = torch.randn(T, generator=gg).to(dev) * (batch.labels >= 0).float()
        lp_f, ent_f = full.forward(batch, 1.0, save_for_backward=True)
        full.backward(glp, None)
        if r == rank:
            lp, ent = m.forward(batch, 1.0, save_for_backward=True)
            m.backward(glp, None)
            lp_err, ent_err = float((lp - lp_f).abs().max()), float((ent - ent_f).abs().max())
    m.sync_replicated_grads()
    num = den = 0.0
    for name, g in m.params.grads.items():
        ref = full.params.grads[name]
        if is_sharded(name):
            per = ref.shape[0] // world
            ref = ref[rank * per:(rank + 1) * per]
        num += float((g - ref).double().pow(2).sum())
        den += float(ref.double().pow(2).sum())
    res.update(lp_err=lp_err, ent_err=ent_err, grad_rel=(num / max(den, 1e-30)) ** 0.5)
    C.check_status()
    res["status_ok"] = True
    out = [None] * world
    dist.all_gather_object(out, res)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(out, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
