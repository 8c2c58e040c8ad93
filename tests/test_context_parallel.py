"""Context parallelism: the zigzag index maps, block attention against whole-sequence attention (one
process plays every rank), and cp=2 trainers (x dp=1 and x dp=2, gloo on CPU) that match the
single-process trainer in log-probs, gradient norm and the parameters after a step."""
import numpy as np
import pytest
import torch

from test_megatron_trainer import _cfg, _run


def test_zigzag_maps_cover_every_token_once_and_balance_the_work():
    from axon_b200.parallel import cp as CP
    cu = torch.tensor([0, 37, 57, 108], dtype=torch.int32)
    for W in (1, 2, 4):
        new_cu, orig_pos, off = CP.pad_layout(cu, W, token_multiple=8)
        T_pad = int(new_cu[-1])
        assert T_pad % (8 * W) == 0 and orig_pos.numel() == 108
        assert all(int(x) % (2 * W) == 0 for x in (new_cu[1:] - new_cu[:-1]))
        idx = torch.cat([CP.local_index(new_cu, r, W) for r in range(W)])
        assert torch.equal(idx.sort().values, torch.arange(T_pad))
        # causal work (number of attended chunk pairs) is the same on every rank
        work = [sum(len(row) for row in CP._blocks(r, W)) for r in range(W)]
        assert len(set(work)) == 1, work


class _FakeGroup:
    """Plays rank ``me`` of ``W`` with the other ranks' tensors at hand (no processes)."""

    def __init__(self, me, W, kv_of_rank, sink):
        self.rank, self.world, self.kv_width = me, W, kv_of_rank[0].shape[1]
        self._kv, self._sink = kv_of_rank, sink

    def gather_kv(self, qkv, col0):
        return torch.stack(self._kv)

    def return_dkv(self, dkv_all):
        self._sink[self.rank] = dkv_all.float()
        return torch.zeros_like(dkv_all[0], dtype=torch.float32)


@pytest.mark.parametrize("W", [2, 4])
def test_block_attention_matches_whole_sequence_attention(W):
    from axon_b200.ops import attention as AT
    from axon_b200.parallel import cp as CP
    Hq, Hkv, D = 4, 2, 16
    g = torch.Generator().manual_seed(1)
    cu = torch.tensor([0, 40, 64, 136], dtype=torch.int32)      # every length a multiple of 2 W
    T, qs = int(cu[-1]), Hq * D
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, generator=g)
    do = torch.randn(T, qs, generator=g)
    o_ref, lse_ref = AT.attn_fwd(qkv, cu, Hq, Hkv, D)
    d_ref = AT.attn_bwd(do, qkv, o_ref, lse_ref, cu, Hq, Hkv, D)
    new_cu = cu.to(torch.int64)
    idx = [CP.local_index(new_cu, r, W) for r in range(W)]
    cu_half = (new_cu // (2 * W)).to(torch.int32)
    kv = [qkv[i][:, qs:].contiguous() for i in idx]
    sink, dq_kv_local = {}, {}
    for r in range(W):
        fake = _FakeGroup(r, W, kv, sink)
        o, lse = CP.attn_fwd(fake, qkv[idx[r]], cu_half, Hq, Hkv, D)
        torch.testing.assert_close(o, o_ref[idx[r]], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(lse, lse_ref[:, idx[r]], rtol=1e-4, atol=1e-5)
        dq_kv_local[r] = CP.attn_bwd(fake, do[idx[r]], qkv[idx[r]], o, lse, cu_half, Hq, Hkv, D)
    for r in range(W):
        torch.testing.assert_close(dq_kv_local[r][:, :qs], d_ref[idx[r]][:, :qs], rtol=1e-4, atol=1e-5)
        dkv = sum(sink[s][r] for s in range(W))
        torch.testing.assert_close(dkv, d_ref[idx[r]][:, qs:], rtol=1e-4, atol=1e-5)


def test_adapter_matches_dense_model_single_rank():
    """One rank still runs the two-chunk zigzag (second half attends the first unmasked)."""
    from axon_b200.models.config import get_config
    from axon_b200.models.cp import CPDenseModel, CPModelAdapter
    from axon_b200.models.dense import DenseModel, PackedBatch
    from axon_b200.parallel.cp import ContextParallel
    cfg = get_config("tiny-qwen3")
    g = torch.Generator().manual_seed(0)
    batch = PackedBatch.from_sequences([torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (37, 20, 51)], "cpu")
    full = DenseModel(cfg, device="cpu", dtype=torch.float32)
    full.params.init_random(std=0.05, seed=3)
    full.recompute = "full"
    glp = torch.randn(batch.input_ids.numel(), generator=g) * (batch.labels >= 0).float()
    full.params.alloc_grads()
    lp_f, ent_f = full.forward(batch, 1.0, save_for_backward=True)
    full.backward(glp, None)
    inner = CPDenseModel(cfg, ContextParallel(None, "cpu", 512, 2 * cfg.kv_size), device="cpu", dtype=torch.float32)
    inner.params.flat.copy_(full.params.flat)
    inner.recompute = "full"
    m = CPModelAdapter(inner)
    m.params.alloc_grads()
    lp, ent = m.forward(batch, 1.0, save_for_backward=True)
    m.backward(glp, None)
    torch.testing.assert_close(lp, lp_f, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(ent, ent_f, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(m.params.grad_flat, full.params.grad_flat, rtol=1e-3, atol=1e-5)


def _cp_cfg(cp):
    c = _cfg(1)
    c["megatron"]["context_parallel_size"] = cp
    return c


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world,cp", [(2, 2), (4, 2)])
def test_context_parallel_trainer_matches_single_process(world, cp):
    ref = _run("axon_b200.trainer.fsdp_trainer.TrainerWorker", _cfg(1), 1)
    got = _run("axon_b200.trainer.megatron_trainer.TrainerWorker", _cp_cfg(cp), world)
    torch.testing.assert_close(got[0], ref[0], rtol=1e-4, atol=1e-4)
    gn, gr = float(np.mean(got[2]["actor/grad_norm"])), float(np.mean(ref[2]["actor/grad_norm"]))
    assert abs(gn - gr) < 1e-3 * max(1.0, gr), (gn, gr)
    torch.testing.assert_close(got[3], ref[3], rtol=1e-3, atol=1e-3)
    assert (got[3] - got[0]).abs().max() > 1e-4


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_peer_push_and_model_on_two_gpus(tmp_path):
    import json, os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "cp.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29673", os.path.join(root, "tests", "_cp_worker.py"), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for x in json.loads(out.read_text()):
        assert x["fused"] and x["exchange_exact"] and x["status_ok"], x
        assert x["lp_err"] < 0.2 and x["ent_err"] < 0.15 and x["grad_rel"] < 0.08, x
