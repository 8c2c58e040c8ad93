"""Tensor-parallel model against the unsharded model; run as W ranks (gloo on CPU, nccl on GPUs)."""
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
        dtype, preset = torch.bfloat16, "tiny-gpu"
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        dtype, preset = torch.float32, "tiny-qwen3"
    from axon_b200.models.config import get_config
    from axon_b200.models.dense import DenseModel, PackedBatch
    from axon_b200.models.tp_dense import TPDenseModel, pad_packed_batch
    from axon_b200.parallel.tp import TPContext
    cfg = get_config(preset)
    cfg.tie_word_embeddings = False
    g = torch.Generator().manual_seed(0)
    seqs = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (150, 97, 260)]
    full = DenseModel(cfg, device=dev, dtype=dtype)
    full.params.init_random(std=0.05, seed=11)
    pb, T_real = pad_packed_batch(PackedBatch.from_sequences(seqs, dev), 128 * world)
    T = pb.input_ids.numel()
    glp = torch.randn(T, generator=g).to(dev) * (pb.labels >= 0).float()
    gent = (torch.randn(T, generator=g) * 0.1).to(dev)
    gent[T_real:] = 0
    full.params.alloc_grads()
    lp_f, ent_f = full.forward(pb, 1.0, save_for_backward=True)
    full.backward(glp, gent)
    tp = TPContext(dist.group.WORLD, dev, max_rows_per_rank=T // world, max_width=max(cfg.qkv_size, 2 * cfg.intermediate_size, cfg.hidden_size))
    vp = len(sys.argv) > 3 and sys.argv[3] == "vp"
    m = TPDenseModel(cfg, tp, device=dev, dtype=dtype, vocab_parallel_head=vp)
    m.load_full_state(full.params.views)
    m.params.alloc_grads()
    lp, ent = m.forward(pb, 1.0, save_for_backward=True)
    sl = m.local_slice(T)
    m.backward(glp[sl], gent[sl])
    m.sync_replicated_grads()
    if dev.type == "cuda":
        torch.cuda.synchronize()
        from axon_b200.ops import _common as C
        C.check_status()
    from axon_b200.models.tp_dense import slice_full_param
    res = {"fused": tp.fused, "lp_err": float((lp.float() - lp_f[sl].float()).abs().max()),
           "ent_err": float((ent.float() - ent_f[sl].float()).abs().max()), "grad_rel": {}}
    for name, gsh in m.params.grads.items():
        ref = slice_full_param(cfg, name, full.params.grads[name], world, rank, m.shard_head).float()
        res["grad_rel"][name] = float((gsh.float() - ref).norm() / (ref.norm() + 1e-12))
    ss = m.grad_sumsq().reshape(1).to(dev)
    dist.all_reduce(ss)
    res["norm_rel"] = abs(float(ss.sqrt()) - float(full.params.grad_flat.double().norm())) / float(full.params.grad_flat.double().norm())
    out = [None] * world
    dist.all_gather_object(out, res)
    if rank == 0:
        json.dump(out, open(out_path, "w"))
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
