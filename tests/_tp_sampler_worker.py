"""A tensor-parallel sampler group against the unsharded model; run as W ranks (gloo on CPU, nccl on GPUs).

Stage "engine": every rank drives its engine with the same calls. Stage "server": only the group's first rank
receives requests and control calls that matter; the others follow its lockstep messages."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _trainer_logprobs(model, prompt, out, temperature):
    """The unsharded model's log-probs of the sampled tokens; a sparse model replays the experts the sampler recorded
    (a near-tie in the router may otherwise resolve differently in bf16)."""
    from axon_b200.models.dense import PackedBatch
    out_ids = out.token_ids
    batch = PackedBatch.from_sequences([torch.tensor(prompt + out_ids)], model.device)
    if out.moe_routermap is not None:
        batch.routermap = torch.from_numpy(out.moe_routermap.astype("int64")).to(model.device)
    lp, _ = model.forward(batch, temperature)
    return lp[len(prompt) - 1: len(prompt) - 1 + len(out_ids)].float().cpu()


def main(out_path: str, device_kind: str, how: str = "tp") -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if device_kind == "cuda":
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=dev)
        dtype, presets = torch.bfloat16, ("tiny-gpu", "tiny-moe-gpu")
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        dtype, presets = torch.float32, ("tiny-qwen3", "tiny-moe")
    from axon_b200.models.config import get_config
    from axon_b200.models.moe import build_model_for
    from axon_b200.models.tp_infer import Shard, ShardedDenseModel, ShardedMoEModel
    from axon_b200.sampler.engine import GenerationEngine
    from axon_b200.sampler.params import SamplingParams
    from axon_b200.sampler.server import Lockstep, SamplerServer
    group = dist.new_group(list(range(world)))
    ctl = dist.new_group(list(range(world)), backend="gloo")       # the servers' lockstep messages, nothing else
    side = dist.new_group(list(range(world)), backend="gloo")      # this script's own barriers and gathers
    shard = Shard.create(group, dev, reduce=how == "tp")       # "pp": the group is cut into pipeline stages instead
    res = {"rank": rank, "fused": shard.reduce.fused if how == "tp" else False}
    g = torch.Generator().manual_seed(5)
    for preset in presets:
        cfg = get_config(preset)
        full = build_model_for(cfg, dev, dtype)
        full.params.init_random(std=0.08, seed=3)
        if how == "tp":
            part = (ShardedMoEModel if cfg.num_experts else ShardedDenseModel)(cfg, shard, device=dev, dtype=dtype)
        else:
            from axon_b200.models.pp_infer import StagedDenseModel, StagedMoEModel
            part = (StagedMoEModel if cfg.num_experts else StagedDenseModel)(cfg, shard, device=dev, dtype=dtype)
        part.load_full_state(full.params.views)
        prompts = [torch.randint(2, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 130, 47, 260, 9, 33)]
        # ---------------- engines driven with the same calls on every rank
        sp = SamplingParams(temperature=0.8, max_tokens=24, ignore_eos=True)
        eng = GenerationEngine(part, num_pages=24, max_num_seqs=8, seed=7)
        if cfg.num_experts and how == "tp":
            eng.enable_routing_capture(True)
        outs = eng.generate(prompts, sp)
        worst = 0.0
        for p, o in zip(prompts, outs):
            ref = _trainer_logprobs(full, p, o, 0.8)
            worst = max(worst, (torch.tensor(o.logprobs) - ref).abs().max().item())
        toks = [o.token_ids for o in outs]
        everyone = [None] * world
        dist.all_gather_object(everyone, toks, group=side)
        key = preset
        res[key] = {"logprob_err": worst, "same_tokens_on_all_ranks": all(t == everyone[0] for t in everyone),
                    "graphs": len(getattr(eng, "_graphs", {}) or {}), "routed": outs[0].moe_routermap is not None}
        if device_kind == "cpu":                      # fp32: the sharded engine reproduces the unsharded one token by token
            ref_eng = GenerationEngine(full, num_pages=24, max_num_seqs=8, seed=7)
            res[key]["equals_unsharded"] = [o.token_ids for o in ref_eng.generate(prompts, sp)] == toks
        # ---------------- servers: requests and control on the first rank only
        eng2 = GenerationEngine(part, num_pages=24, max_num_seqs=8, seed=7)
        if cfg.num_experts and how == "tp":
            eng2.enable_routing_capture(True)
        srv = SamplerServer(eng2, name=f"s{rank}", lockstep=Lockstep(ctl)).start()
        greedy = SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True)
        if rank == 0:
            first = [f.result(timeout=300) for f in [srv.submit(p, greedy) for p in prompts]]
        dist.barrier(group=side)                      # control calls reach every rank only after the requests are done
        srv.sleep()
        srv.wake_up()
        other = build_model_for(cfg, dev, dtype)
        other.params.init_random(std=0.08, seed=19)
        n_up = srv.update_weights(list(other.params.views.items()))          # FULL tensors: every rank keeps its part
        srv.continue_generation()
        dist.barrier(group=side)                      # as the controller does: every rank has the new weights before requests resume
        if rank == 0:
            second = [f.result(timeout=300) for f in [srv.submit(p, greedy) for p in prompts[:3]]]
            long = srv.submit(prompts[1], SamplingParams(temperature=0.0, max_tokens=400, ignore_eos=True))
            import time
            time.sleep(0.3)
            srv.pause_generation("reset")
            aborted = long.result(timeout=300)
            srv.continue_generation()
            third = srv.submit(prompts[0], greedy).result(timeout=300)
            worst2 = 0.0
            for p, o in zip(prompts[:3], second):
                worst2 = max(worst2, (torch.tensor(o.logprobs) - _trainer_logprobs(other, p, o, 1.0)).abs().max().item())
            res[key].update(server_first_len=[len(o.token_ids) for o in first], updated=n_up, after_update_err=worst2,
                            aborted_reason=aborted.finish_reason, aborted_len=len(aborted.token_ids),
                            third_equals_second=third.token_ids == second[0].token_ids)
            # requests reach the server one by one, so batches differ from a one-shot run: compare against the trainer pass
            res[key]["server_first_err"] = max((torch.tensor(o.logprobs) - _trainer_logprobs(full, p, o, 1.0)).abs().max().item()
                                               for p, o in zip(prompts, first))
            srv.stop()
        else:
            srv._thread.join(timeout=600)             # ends with the leader's last message
            res[key]["follower_done"] = not srv._thread.is_alive()
            res[key]["follower_error"] = repr(srv.error) if srv.error else None
        dist.barrier(group=side)
    res["reduce_calls"] = dict(shard.reduce.calls) if how == "tp" else {}
    if device_kind == "cuda":
        from axon_b200.ops import _common as C
        torch.cuda.synchronize()
        res["status"] = int(C.status(dev).flatten()[0].item())
    allres = [None] * world
    dist.all_gather_object(allres, res, group=side)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(allres, f)
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2], sys.argv[3] if len(sys.argv) > 3 else "tp")
