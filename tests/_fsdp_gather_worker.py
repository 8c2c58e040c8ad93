"""Weight-gather fused GEMM against all-gather + matmul; run as W ranks (gloo on CPU, nccl on GPUs)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(out_path: str, kind: str) -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if kind == "cuda":
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=dev)
        dtype = torch.bfloat16
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        dtype = torch.float32
    from axon_b200.parallel.fsdp_gather import ShardedLinear
    res = {"errs": []}
    for (T, F, K) in ((384, 1024, 512), (100, 2048, 1024), (2304, 4096, 2048)):
        g = torch.Generator().manual_seed(F + K)
        W = (torch.randn(F, K, generator=g) * 0.05)
        lin = ShardedLinear(W, F, K, dist.group.WORLD, dev, dtype=dtype)
        x = (torch.randn(T, K, generator=torch.Generator().manual_seed(rank * 7 + T))).to(dev).to(dtype)     # every rank its own tokens
        y = lin.forward(x)
        ref = x.float() @ W.to(dev).to(dtype).float().t()
        res["errs"].append(float((y.float() - ref).abs().max() / ref.abs().max()))
        res["fused"] = lin.fused
        # an "optimizer step" on the shard must be seen by the peers' next product
        lin.shard.mul_(2.0)
        lin.publish()
        y2 = lin.forward(x)
        res["errs"].append(float((y2.float() - 2 * ref).abs().max() / ref.abs().max()))
    if kind == "cuda":
        from axon_b200.ops import _common as C
        C.check_status()
    out = [None] * world
    dist.all_gather_object(out, res)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(out, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
