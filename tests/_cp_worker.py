"""Context-parallel model against the unsharded model on W GPUs (nccl): the K|V push over peer memory
against the all-gather path, then forward / backward of the whole model."""
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
    from axon_b200.models.cp import CPDenseModel, CPModelAdapter
    from axon_b200.models.dense import DenseModel, PackedBatch
    from axon_b200.ops import _common as C
    from axon_b200.parallel.cp import ContextParallel
    cfg = get_config("tiny-gpu")
    kw = 2 * cfg.kv_size
    res = {}
    fused = ContextParallel(dist.group.WORLD, dev, 1024, kw)
    plain = ContextParallel(dist.group.WORLD, dev, 1024, kw, fused=False)
    g = torch.Generator().manual_seed(100 + rank)
    exact = True
    for it in range(3):          # three rounds: both alternating buffers get reused
        x = torch.randn(384, cfg.qkv_size, generator=g).to(dev).to(torch.bfloat16)
        a, b = fused.gather_kv(x, cfg.q_size), plain.gather_kv(x, cfg.q_size)
        exact &= bool(torch.equal(a, b))
        d = torch.randn(world, 384, kw, generator=g).to(dev).to(torch.bfloat16).float()
        a2, b2 = fused.return_dkv(d), plain.return_dkv(d)
        exact &= bool(torch.allclose(a2, b2, rtol=1e-6, atol=1e-6))
    res["exchange_exact"] = exact
    res["fused"] = fused.fused
    gg = torch.Generator().manual_seed(0)
    seqs = [torch.randint(0, cfg.vocab_size, (n,), generator=gg) for n in (150, 97, 260)]
    batch = PackedBatch.from_sequences(seqs, dev)
    T = batch.input_ids.numel()
    full = DenseModel(cfg, device=dev)
    full.params.init_random(std=0.05, seed=11)
    full.recompute = "full"
    glp = (torch.randn(T, generator=gg).to(dev)) * (batch.labels >= 0).float()
    full.params.alloc_grads()
    lp_f, ent_f = full.forward(batch, 1.0, save_for_backward=True)
    full.backward(glp, None)
    inner = CPDenseModel(cfg, fused, device=dev)
    inner.params.flat.copy_(full.params.flat)
    inner.recompute = "full"
    m = CPModelAdapter(inner)
    m.params.alloc_grads()
    lp, ent = m.forward(batch, 1.0, save_for_backward=True)
    m.backward(glp, None)
    gsum = m.params.grad_flat.clone()
    dist.all_reduce(gsum)                       # partial over local tokens -> total
    res["lp_err"] = float((lp - lp_f).abs().max())
    res["ent_err"] = float((ent - ent_f).abs().max())
    ref = full.params.grad_flat
    res["grad_rel"] = float((gsum - ref).norm() / ref.norm().clamp_min(1e-12))
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
