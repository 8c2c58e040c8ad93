"""Lightning indexer and sparse latent attention: the explicit forward / backward formulas against autograd
over a dense-masked implementation, and the native indexer kernel against the PyTorch one."""
import pytest
import torch

from axon_b200.ops import dsa


def _inputs(S=24, Skv=40, Hi=4, D=16, H=3, Dk=24, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(S, Hi, D, generator=g)
    k = torch.randn(Skv, D, generator=g)
    w = torch.randn(S, Hi, generator=g)
    ks = torch.randint(0, 6, (S,), generator=g)
    ke = (ks + torch.randint(1, Skv, (S,), generator=g)).clamp_max(Skv)
    qm = torch.randn(S, H, Dk, generator=g)
    kv = torch.randn(Skv, Dk, generator=g)
    return q, k, w, ks, ke, qm, kv


def test_indexer_logits_window_and_topk():
    q, k, w, ks, ke, _, _ = _inputs()
    lg = dsa.indexer_logits(q, k, w, ks, ke)
    dense = (torch.einsum("shd,jd->shj", q, k).relu() * w[..., None]).sum(1)
    for s in range(q.shape[0]):
        a, b = int(ks[s]), int(ke[s])
        torch.testing.assert_close(lg[s, a:b], dense[s, a:b], rtol=1e-5, atol=1e-5)
        assert torch.isinf(lg[s, :a]).all() and torch.isinf(lg[s, b:]).all()
    idx = dsa.indexer_topk(lg, 16)
    for s in range(q.shape[0]):
        n = min(16, int(ke[s] - ks[s]))
        sel = idx[s][idx[s] >= 0]
        assert sel.numel() == n and ((sel >= ks[s]) & (sel < ke[s])).all()
        assert lg[s, sel.long()].min() >= lg[s].topk(n).values.min() - 1e-6
    assert dsa.indexer_topk(lg, 64).shape == (q.shape[0], 64)


def test_indexer_backward_matches_autograd():
    q, k, w, ks, ke, _, _ = _inputs()
    idx = dsa.indexer_topk(dsa.indexer_logits(q, k, w, ks, ke), 8)
    g = torch.randn(idx.shape, generator=torch.Generator().manual_seed(1)) * (idx >= 0)
    qa, ka, wa = (t.clone().requires_grad_(True) for t in (q, k, w))
    dense = (torch.einsum("shd,jd->shj", qa, ka).relu() * wa[..., None]).sum(1)
    (dense.gather(1, idx.long().clamp_min(0)) * g).sum().backward()
    dq, dk, dw = dsa.indexer_bwd_ref(g, idx, q, k, w)
    torch.testing.assert_close(dq, qa.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dk, ka.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dw, wa.grad, rtol=1e-4, atol=1e-5)
    qb, kb, wb = (t.clone().requires_grad_(True) for t in (q, k, w))
    (dsa.indexer_logits_at(qb, kb, wb, idx) * g).sum().backward()
    torch.testing.assert_close(qb.grad, qa.grad, rtol=1e-4, atol=1e-5)


def test_sparse_mla_matches_dense_masked_attention():
    q, k, w, ks, ke, qm, kv = _inputs()
    S, Skv, d_v, scale = qm.shape[0], kv.shape[0], 16, 0.3
    idx = dsa.indexer_topk(dsa.indexer_logits(q, k, w, ks, ke), 8)
    idx[3] = -1                                                     # a query without keys
    mask = torch.zeros(S, Skv + 1, dtype=torch.bool)
    mask.scatter_(1, torch.where(idx >= 0, idx, torch.full_like(idx, Skv)).long(), True)
    mask = mask[:, :Skv]
    qa, kva = qm.clone().requires_grad_(True), kv.clone().requires_grad_(True)
    sc = (torch.einsum("shd,jd->shj", qa, kva) * scale).masked_fill(~mask[:, None, :], float("-inf"))
    p = torch.nan_to_num(sc.softmax(-1), nan=0.0)
    ref = torch.einsum("shj,jd->shd", p, kva[:, :d_v])
    do = torch.randn(ref.shape, generator=torch.Generator().manual_seed(2))
    (ref * do).sum().backward()
    out, lse = dsa.sparse_mla_fwd_ref(qm, kv, idx, scale, d_v)
    torch.testing.assert_close(out, ref.detach(), rtol=1e-4, atol=1e-5)
    assert torch.isinf(lse[3]).all() and float(out[3].abs().max()) == 0.0
    dq, dkv = dsa.sparse_mla_bwd_ref(do, qm, kv, out, lse, idx, scale, d_v)
    torch.testing.assert_close(dq, qa.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dkv, kva.grad, rtol=1e-4, atol=1e-5)
    qb, kvb = qm.clone().requires_grad_(True), kv.clone().requires_grad_(True)
    o2, _ = dsa.sparse_mla(qb, kvb, idx, scale, d_v)
    (o2 * do).sum().backward()
    torch.testing.assert_close(kvb.grad, kva.grad, rtol=1e-4, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("Hi,S,Skv", [(32, 200, 1000), (64, 96, 4096), (32, 1024, 2304)])
def test_native_indexer_matches_reference(Hi, S, Skv):
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(Hi + S)
    D = 128
    q = (torch.randn(S, Hi, D, generator=g) * 0.5).to(dev).to(torch.bfloat16)
    k = (torch.randn(Skv, D, generator=g) * 0.5).to(dev).to(torch.bfloat16)
    w = torch.randn(S, Hi, generator=g).to(dev)
    ks = torch.randint(0, 50, (S,), generator=g).to(dev)
    ke = (ks + torch.randint(1, Skv, (S,), generator=g).to(dev)).clamp_max(Skv)
    got = dsa.indexer_logits(q, k, w, ks, ke)
    ref = dsa.indexer_logits_ref(q, k, w, ks, ke)
    from axon_b200.ops import _common as C
    C.check_status()
    assert torch.equal(torch.isinf(got), torch.isinf(ref))
    fin = ~torch.isinf(ref)
    err = (got[fin] - ref[fin]).abs().max().item()
    assert err < 2e-2 * max(1.0, ref[fin].abs().max().item()), err
    again = dsa.indexer_logits(q, k, w, ks, ke)
    assert torch.equal(again, got)                      # reproducible, also with two warps per query


@pytest.mark.gpu
@pytest.mark.parametrize("Hi", [32, 64])
def test_native_indexer_backward_matches_reference(Hi):
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(Hi)
    S, Skv, D, topk = 150, 700, 128, 96
    q = (torch.randn(S, Hi, D, generator=g) * 0.5).to(dev).to(torch.bfloat16)
    k = (torch.randn(Skv, D, generator=g) * 0.5).to(dev).to(torch.bfloat16)
    w = torch.randn(S, Hi, generator=g).to(dev)
    ks = torch.zeros(S, dtype=torch.int64, device=dev)
    ke = torch.randint(40, Skv, (S,), generator=g).to(dev)
    idx = dsa.indexer_topk(dsa.indexer_logits(q, k, w, ks, ke), topk)
    assert (idx < 0).any() and (idx >= 0).any()
    gl = torch.randn(S, topk, generator=g).to(dev) * (idx >= 0)
    dq, dk, dw = dsa.indexer_bwd(gl, idx, q, k, w)
    rq, rk, rw = dsa.indexer_bwd_ref(gl, idx, q, k, w)
    from axon_b200.ops import _common as C
    C.check_status()
    for a, b in ((dq, rq), (dk, rk), (dw, rw)):
        assert (a - b).abs().max().item() < 1e-3 * max(1.0, b.abs().max().item())


def test_dense_masked_tensor_core_formulation_matches_gathering_one():
    """Runs the GEMM formulation through the CPU fall-backs of the GEMM ops (probabilities pass through bf16)."""
    q, k, w, ks, ke, qm, kv = _inputs(S=40, Skv=70, H=4, Dk=24)
    idx = dsa.indexer_topk(dsa.indexer_logits(q, k, w, ks, ke), 12)
    idx[5] = -1
    out_r, lse_r = dsa.sparse_mla_fwd_ref(qm, kv, idx, 0.3, 16)
    out, lse = dsa.sparse_mla_fwd_tc(qm, kv, idx, 0.3, 16)
    torch.testing.assert_close(lse, lse_r, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(out, out_r, rtol=2e-2, atol=2e-2)
    do = torch.randn(out.shape, generator=torch.Generator().manual_seed(4))
    dq_r, dkv_r = dsa.sparse_mla_bwd_ref(do, qm, kv, out_r, lse_r, idx, 0.3, 16)
    dq, dkv = dsa.sparse_mla_bwd_tc(do, qm, kv, out_r, lse_r, idx, 0.3, 16)
    assert (dq - dq_r).abs().max() < 3e-2 * max(1.0, float(dq_r.abs().max()))
    assert (dkv - dkv_r).abs().max() < 3e-2 * max(1.0, float(dkv_r.abs().max()))


@pytest.mark.gpu
def test_sparse_mla_on_gpu_matches_reference():
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(7)
    S, Skv, H, Dk, d_v, topk = 300, 1000, 16, 576, 512, 128
    q = (torch.randn(S, H, Dk, generator=g) * 0.3).to(dev).to(torch.bfloat16)
    kv = (torch.randn(Skv, Dk, generator=g) * 0.3).to(dev).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(Skv, generator=g)[:topk] for _ in range(S)]).int().to(dev)
    idx[:, -5:] = -1
    idx[7] = -1
    scale = Dk ** -0.5
    out, lse = dsa.sparse_mla_fwd(q, kv, idx, scale, d_v)
    out_r, lse_r = dsa.sparse_mla_fwd_ref(q, kv, idx, scale, d_v)
    from axon_b200.ops import _common as C
    C.check_status()
    torch.testing.assert_close(lse, lse_r, rtol=2e-3, atol=2e-3)
    assert (out.float() - out_r.float()).abs().max() < 2e-2
    do = (torch.randn(S, H, d_v, generator=g) * 0.3).to(dev).to(torch.bfloat16)
    dq, dkv = dsa.sparse_mla_bwd(do, q, kv, out, lse, idx, scale, d_v)
    dq_r, dkv_r = dsa.sparse_mla_bwd_ref(do, q, kv, out_r, lse_r, idx, scale, d_v)
    C.check_status()
    assert (dq.float() - dq_r.float()).abs().max() < 3e-2 * max(1.0, float(dq_r.float().abs().max()))
    assert (dkv - dkv_r).abs().max() < 3e-2 * max(1.0, float(dkv_r.abs().max()))


def test_dsa_layer_equals_causal_attention_when_topk_covers_the_sequence():
    g = torch.Generator().manual_seed(9)
    cu = torch.tensor([0, 11, 11, 30], dtype=torch.int32)          # an empty sequence in the middle
    T, H, Dk, d_v, Hi, Di = 30, 3, 24, 16, 4, 8
    q, kv = torch.randn(T, H, Dk, generator=g).requires_grad_(True), torch.randn(T, Dk, generator=g).requires_grad_(True)
    q_idx, k_idx, w_idx = torch.randn(T, Hi, Di, generator=g), torch.randn(T, Di, generator=g), torch.randn(T, Hi, generator=g)
    out, idx = dsa.dsa_attention(q, kv, q_idx, k_idx, w_idx, cu, topk=32, scale=0.25, d_v=d_v)
    ref = torch.zeros(T, H, d_v)
    for a, b in ((0, 11), (11, 30)):
        sc = torch.einsum("shd,jd->shj", q[a:b], kv[a:b]) * 0.25
        sc = sc.masked_fill(torch.ones(b - a, b - a, dtype=torch.bool).triu(1)[:, None, :], float("-inf"))
        ref[a:b] = torch.einsum("shj,jd->shd", sc.softmax(-1), kv[a:b, :d_v])
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)
    for t in range(T):                                             # selections stay inside the causal window
        sel = idx[t][idx[t] >= 0]
        lo = 0 if t < 11 else 11
        assert sel.numel() == t - lo + 1 and int(sel.min()) >= lo and int(sel.max()) <= t
    out.sum().backward()
    assert q.grad is not None and float(kv.grad.abs().sum()) > 0
    few, idx2 = dsa.dsa_attention(q.detach(), kv.detach(), q_idx, k_idx, w_idx, cu, topk=4, scale=0.25, d_v=d_v)
    assert idx2.shape == (T, 4) and not torch.allclose(few, ref)
