"""RoutingTable + plan compiler: applying the plan equals 'gather the full tensors, slice for the sampler'."""
import itertools

import pytest
import torch

from axon_b200.models.config import ModelConfig
from axon_b200.models.params import param_layout
from axon_b200.utils.p2p.param_mapper import convert_hf_to_vllm_param_name, get_param_metadata, shard_rows
from axon_b200.utils.p2p.plan import compile_plan, execute_plan, fp8_block_quant_ref
from axon_b200.utils.p2p.routing_table import ParameterMetadata, RankMapping, RoutingTable


def cfg_dense():
    return ModelConfig(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=8,
                       num_key_value_heads=4, head_dim=32, intermediate_size=384, qk_norm=True)


def cfg_moe():
    return ModelConfig(model_type="qwen3_moe", vocab_size=256, hidden_size=128, num_hidden_layers=1, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=32, intermediate_size=256, num_experts=8, num_experts_per_tok=2,
                       moe_intermediate_size=128)


def full_tensors(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    return {n: torch.randn(*s, generator=g).to(torch.bfloat16) for n, s in param_layout(cfg).items()}


def local_shard(cfg, full, name, tp, tpr, ep, epr):
    """A rank's local storage of one parameter: its boxes concatenated."""
    t = full[name]
    t2 = t.reshape(t.shape[0], -1) if t.dim() > 1 else t.reshape(-1, 1)
    parts = [t2[r0:r1, c0:c1].reshape(-1) for r0, r1, c0, c1 in shard_rows(cfg, name, tp, tpr, ep, epr)]
    return torch.cat(parts)


def build_side(cfg, full, ranks):
    """ranks: list of (rank, tp, tp_rank, ep, ep_rank). Returns mappings, flat buffers, offsets."""
    maps, flats, offs = [], {}, {}
    for rank, tp, tpr, ep, epr in ranks:
        maps.append(get_param_metadata(cfg, rank, tp, tpr, ep, epr))
        chunks, off, o = [], 0, {}
        for name in param_layout(cfg):
            sh = local_shard(cfg, full, name, tp, tpr, ep, epr)
            o[name] = off
            chunks.append(sh)
            pad = (-sh.numel()) % 128
            if pad:
                chunks.append(torch.zeros(pad, dtype=sh.dtype))
            off += sh.numel() + pad
        flats[rank], offs[rank] = torch.cat(chunks), o
    return maps, flats, offs


@pytest.mark.parametrize("a_tp,a_dp,s_tp,s_dp", [(1, 1, 1, 1), (1, 2, 2, 1), (2, 1, 1, 2), (4, 1, 2, 2), (2, 2, 4, 1), (1, 4, 4, 2)])
def test_plan_equals_gather_then_slice_dense(a_tp, a_dp, s_tp, s_dp):
    cfg = cfg_dense()
    full = full_tensors(cfg)
    a_ranks = [(d * a_tp + t, a_tp, t, 1, 0) for d in range(a_dp) for t in range(a_tp)]
    s_ranks = [(d * s_tp + t, s_tp, t, 1, 0) for d in range(s_dp) for t in range(s_tp)]
    a_maps, a_flats, a_offs = build_side(cfg, full, a_ranks)
    s_maps, s_expected, s_offs = build_side(cfg, full, s_ranks)
    table = RoutingTable(a_maps, s_maps)
    dst = {r: torch.full_like(t, float("nan")) for r, t in s_expected.items()}
    dst_list = [dst[r] for r in sorted(dst)]
    sent = {}
    for rank, *_ in a_ranks:
        plan = compile_plan(table, rank, a_offs[rank], s_offs)
        execute_plan(plan, a_flats[rank], dst_list)
        sent[rank] = plan.total_bytes
    for r in dst:
        for name in param_layout(cfg):
            n = local_shard(cfg, full, name, *[x for x in s_ranks if x[0] == r][0][1:]).numel()
            o = s_offs[r][name]
            assert torch.equal(dst[r][o:o + n], s_expected[r][o:o + n]), (r, name)
    # the offline checker agrees: every sampler element written exactly once, nothing outside the shards
    from axon_b200.utils.p2p.verify_plan import verify_plans
    plans = {rank: compile_plan(table, rank, a_offs[rank], s_offs) for rank, *_ in a_ranks}
    spans = {r: [(s_offs[r][n], local_shard(cfg, full, n, *[x for x in s_ranks if x[0] == r][0][1:]).numel()) for n in param_layout(cfg)]
             for r in dst}
    rep = verify_plans(plans, spans)
    assert rep["ok"], rep
    if len(plans) > 1 or len(next(iter(plans.values())).descs) > 1:
        broken = dict(plans)
        first = next(iter(broken))
        import copy
        bad = copy.deepcopy(broken[first])
        bad.descs = bad.descs[:-1]                 # drop one slice: something must be reported missing
        broken[first] = bad
        assert not verify_plans(broken, spans)["ok"]
    # every destination byte is sent exactly once and the senders share the load
    total = sum(sum(local_shard(cfg, full, n, *x[1:]).numel() for n in param_layout(cfg)) for x in s_ranks) * 2
    assert sum(sent.values()) == total
    if a_dp > 1:
        assert max(sent.values()) <= 1.6 * (total / len(a_ranks)) + 4096
    stats = table.get_load_statistics()
    assert stats["total_bytes"] == total and "actor 0" in table.print_routing_table()


def test_expert_parallel_resharding():
    cfg = cfg_moe()
    full = full_tensors(cfg, 1)
    a_ranks = [(e, 1, 0, 4, e) for e in range(4)]           # trainer EP4
    s_ranks = [(e, 1, 0, 2, e) for e in range(2)]           # sampler EP2
    a_maps, a_flats, a_offs = build_side(cfg, full, a_ranks)
    s_maps, s_exp, s_offs = build_side(cfg, full, s_ranks)
    table = RoutingTable(a_maps, s_maps)
    dst = [torch.full_like(s_exp[r], float("nan")) for r in sorted(s_exp)]
    for rank, *_ in a_ranks:
        execute_plan(compile_plan(table, rank, a_offs[rank], s_offs), a_flats[rank], dst)
    for r in (0, 1):
        name = "model.layers.0.mlp.experts.w13_weight"
        n = local_shard(cfg, full, name, 1, 0, 2, r).numel()
        o = s_offs[r][name]
        assert torch.equal(dst[r][o:o + n], s_exp[r][o:o + n])
    # replicated tensors on an EP fleet: each sampler rank receives them from exactly one trainer rank
    per_dst = {s: sum(1 for (a, s2), items in table.routing_map.items() if s2 == s for it in items
                      if it["sampler"].param_name == "model.norm.weight") for s in (0, 1)}
    assert per_dst == {0: 1, 1: 1}


def test_fp8_block_quant_sync_matches_reference_math():
    cfg = cfg_dense()
    full = full_tensors(cfg, 2)
    a_maps, a_flats, a_offs = build_side(cfg, full, [(0, 1, 0, 1, 0)])
    s_maps, s_exp, s_offs = build_side(cfg, full, [(0, 1, 0, 1, 0)])
    table = RoutingTable(a_maps, s_maps)
    layout = param_layout(cfg)
    sc_offs, off = {}, 0
    for n, s in layout.items():
        if len(s) >= 2:
            sc_offs[n] = off
            off += ((s[0] + 127) // 128) * ((s[1] + 127) // 128)
    plan = compile_plan(table, 0, a_offs[0], s_offs, {0: sc_offs}, quant=True)
    dst = torch.zeros(s_exp[0].numel() * 2, dtype=torch.uint8)            # byte view: bf16 region doubles as fp8 bytes
    dst_bf16 = dst.view(torch.bfloat16)
    scales = torch.zeros(off)
    execute_plan(plan, a_flats[0], [dst_bf16], scale_flats=[scales])
    name = "model.layers.1.mlp.gate_up_proj.weight"
    R, Cc = layout[name]
    q_ref, s_ref = fp8_block_quant_ref(full[name])
    got_q = dst[s_offs[0][name]:s_offs[0][name] + R * Cc].view(R, Cc)
    assert torch.equal(got_q, q_ref.view(torch.uint8))
    assert torch.allclose(scales[sc_offs[name]:sc_offs[name] + s_ref.numel()].view_as(s_ref), s_ref)
    deq = q_ref.float().view(R // 128, 128, Cc // 128, 128) * s_ref[:, None, :, None]
    assert (deq.reshape(R, Cc) - full[name].float()).abs().max() < 0.2 * full[name].float().abs().max()
    # 1-D tensors still travel as bf16
    o = s_offs[0]["model.norm.weight"]
    assert torch.equal(dst_bf16[o:o + 256], full["model.norm.weight"])


def test_routing_errors_and_name_mapping():
    a = RankMapping(0, [ParameterMetadata("w", "w", (4, 4), (4, 4), torch.bfloat16, metadata={"boxes": [(0, 4, 0, 4)]})])
    s = RankMapping(0, [ParameterMetadata("v", "v", (4, 4), (4, 4), torch.bfloat16, metadata={"boxes": [(0, 4, 0, 4)]})])
    with pytest.raises(ValueError, match="Parameter name mismatch"):
        RoutingTable([a], [s])
    assert convert_hf_to_vllm_param_name("model.layers.3.self_attn.k_proj.weight") == ("model.layers.3.self_attn.qkv_proj.weight", "k")
    assert convert_hf_to_vllm_param_name("model.layers.0.mlp.up_proj.weight") == ("model.layers.0.mlp.gate_up_proj.weight", "up")
    assert convert_hf_to_vllm_param_name("model.layers.0.mlp.experts.7.down_proj.weight") == ("model.layers.0.mlp.experts.w2_weight", "w2:7")
    assert convert_hf_to_vllm_param_name("model.norm.weight") == ("model.norm.weight", None)


def test_tensor_parallel_trainer_with_whole_embedding_feeds_vocab_split_sampler():
    """A TP=2 trainer that keeps the embedding and the head whole (as the tensor-parallel model does)
    pushes to a TP=2 sampler that splits them over the vocabulary: built from the model's own layout."""
    from axon_b200.models.tp_dense import slice_full_param, tp_param_layout
    cfg = cfg_dense()
    full = full_tensors(cfg, 5)
    rep = [n for n in param_layout(cfg) if n.endswith("embed_tokens.weight") or n.endswith("lm_head.weight")]
    a_maps, a_flats, a_offs = [], {}, {}
    for r in range(2):
        a_maps.append(get_param_metadata(cfg, r, 2, r, replicated_names=rep))
        lay = tp_param_layout(cfg, 2, r, False)
        chunks, off, o = [], 0, {}
        for name in lay:
            sh = slice_full_param(cfg, name, full[name], 2, r).reshape(-1)
            assert tuple(slice_full_param(cfg, name, full[name], 2, r).shape) == tuple(lay[name])
            o[name], off = off, off + sh.numel()
            chunks.append(sh)
        a_flats[r], a_offs[r] = torch.cat(chunks), o
        for pm in a_maps[-1].params:
            assert tuple(pm.param_shape) == tuple(lay[pm.param_name]), pm.param_name
    s_maps, s_exp, s_offs = build_side(cfg, full, [(t, 2, t, 1, 0) for t in range(2)])
    table = RoutingTable(a_maps, s_maps)
    dst = [torch.full_like(s_exp[r], float("nan")) for r in sorted(s_exp)]
    for r in range(2):
        execute_plan(compile_plan(table, r, a_offs[r], s_offs), a_flats[r], dst)
    for r in range(2):
        for name in param_layout(cfg):
            n = local_shard(cfg, full, name, 2, r, 1, 0).numel()
            o = s_offs[r][name]
            assert torch.equal(dst[r][o:o + n], s_exp[r][o:o + n]), (r, name)
