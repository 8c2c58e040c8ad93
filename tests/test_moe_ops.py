"""Mixture-of-experts ops: layout invariants and (on the GPU) native kernels against the references."""
import pytest
import torch

from axon_b200.ops import moe as M


def _setup(T=50, E=8, k=2, H=32, seed=0, device="cpu", dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    x = torch.randn(T, H, generator=g).to(dtype)
    return logits.to(device), x.to(device)


def test_route_and_replay_reference():
    logits, _ = _setup()
    ids, w = M.route(logits, 2)
    p = torch.softmax(logits, -1)
    tv, ti = torch.topk(p, 2, -1)
    assert torch.equal(ids.long(), ti) and torch.allclose(w, tv / tv.sum(-1, keepdim=True))
    _, w_raw = M.route(logits, 2, normalize=False)
    assert torch.allclose(w_raw, tv)
    replay = ti.clone().int()
    replay[3] = torch.tensor([5, -1])
    replay[7] = torch.tensor([-1, -1])
    ids2, w2 = M.route(logits, 2, replay=replay)
    assert ids2[3, 0] == 5 and ids2[3, 1] != 5 and torch.equal(ids2[7].long(), ti[7])
    assert torch.allclose(w2.sum(-1), torch.ones(50)) and torch.allclose(w2[3, 0] / w2[3, 1], p[3, 5] / p[3, ids2[3, 1].long()])
    wd = M.route_weights_from_probs(logits, ids)
    assert torch.allclose(wd, w)


def test_layout_gather_combine_roundtrip_and_grads():
    logits, x = _setup(T=70, E=8, k=3, H=16)
    ids, w = M.route(logits, 3)
    lay = M.align(ids, 8)
    off = lay.offsets.tolist()
    assert lay.max_rows % 128 == 0 and all(o % 128 == 0 for o in off) and off[-1] <= lay.max_rows
    assert lay.counts.sum() == 70 * 3 and (torch.bincount(ids.flatten().long(), minlength=8) == lay.counts).all()
    rows = lay.row_of.long()
    assert rows.unique().numel() == 210                                   # every assignment has its own row
    for e in range(8):
        mine = rows[ids.flatten() == e]
        assert ((mine >= off[e]) & (mine < off[e] + int(lay.counts[e]))).all()
        assert (mine[1:] > mine[:-1]).all()                               # token order inside an expert
        assert (lay.tile_expert[off[e] // 128:off[e + 1] // 128] == e).all()
    xs = M.gather(x, lay)
    assert torch.equal(xs[rows], x.repeat_interleave(3, 0)) and xs[lay.token_of < 0].abs().sum() == 0
    # identity experts: combine(gather(x)) = sum_j w_j x = x (normalised weights)
    assert torch.allclose(M.combine(xs, w, lay), x, atol=1e-5)
    assert torch.allclose(M.scatter_sum(xs, lay), 3 * x, atol=1e-5)
    # full MoE MLP against a dense per-token loop, forward and backward
    g = torch.Generator().manual_seed(1)
    w1 = (torch.randn(8, 256, 16, generator=g) * 0.2).requires_grad_(True)
    w2 = (torch.randn(8, 16, 128, generator=g) * 0.2).requires_grad_(True)
    xr = x.clone().requires_grad_(True)
    out_ref = torch.zeros(70, 16)
    for t in range(70):
        for j in range(3):
            e = int(ids[t, j])
            gu = w1[e] @ xr[t]
            a = torch.nn.functional.silu(gu[:128]) * gu[128:]
            out_ref[t] = out_ref[t] + w[t, j] * (w2[e] @ a)
    dout = torch.randn(70, 16, generator=g)
    out_ref.backward(dout)
    from axon_b200.ops.activation import swiglu_bwd, swiglu_fwd
    gu = M.grouped_fwd(xs, w1.detach(), lay)
    a = swiglu_fwd(gu)
    ys = M.grouped_fwd(a, w2.detach(), lay)
    out = M.combine(ys, w, lay)
    assert torch.allclose(out, out_ref.detach(), atol=1e-4)
    dys, dwt = M.combine_bwd(dout, ys, w, lay)
    dw2 = M.grouped_wgrad(dys, a, torch.zeros(8, 16, 128), lay)
    da = M.grouped_dgrad(dys, w2.detach(), lay)
    dgu = swiglu_bwd(da, gu)
    dw1 = M.grouped_wgrad(dgu, xs, torch.zeros(8, 256, 16), lay)
    dx = M.scatter_sum(M.grouped_dgrad(dgu, w1.detach(), lay), lay)
    assert torch.allclose(dw2, w2.grad, atol=1e-4) and torch.allclose(dw1, w1.grad, atol=1e-4)
    assert torch.allclose(dx, xr.grad, atol=1e-4)
    assert dwt.shape == (70, 3) and torch.allclose(dwt[5, 1], (dout[5] * ys[rows[16]]).sum(), atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("T,E,k", [(300, 128, 8), (64, 16, 2), (1, 128, 8), (1000, 64, 6)])
def test_native_routing_and_layout_match_reference(T, E, k):
    logits, _ = _setup(T=T, E=E, k=k, device="cuda")
    ids, w = M.route(logits, k)
    ids_r, w_r = M.route_ref(logits.cpu(), k)
    assert torch.equal(ids.cpu(), ids_r)
    torch.testing.assert_close(w.cpu(), w_r, rtol=1e-5, atol=1e-6)
    replay = ids_r.clone()
    replay[::3, 0] = -1
    replay[1::5] = torch.roll(replay[1::5], 1, -1)
    ids2, w2 = M.route(logits, k, replay=replay.cuda())
    ids2_r, w2_r = M.route_ref(logits.cpu(), k, replay=replay)
    assert torch.equal(ids2.cpu(), ids2_r)
    torch.testing.assert_close(w2.cpu(), w2_r, rtol=1e-5, atol=1e-6)
    lay, lay_r = M.align(ids, E), M.align(ids_r, E)
    for f in ("counts", "offsets", "row_of", "token_of", "tile_expert"):
        assert torch.equal(getattr(lay, f).cpu(), getattr(lay_r, f)), f


@pytest.mark.gpu
@pytest.mark.parametrize("T,E,k,H,F", [(300, 16, 4, 256, 128), (2000, 128, 8, 512, 256), (40, 8, 2, 128, 128)])
def test_native_moe_mlp_matches_reference(T, E, k, H, F):
    from axon_b200.ops import _common as C
    from axon_b200.ops.activation import swiglu_bwd, swiglu_fwd
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(T, E, generator=g)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(E, 2 * F, H, generator=g) * 0.1).to(torch.bfloat16)
    w2 = (torch.randn(E, H, F, generator=g) * 0.1).to(torch.bfloat16)
    dout = torch.randn(T, H, generator=g).to(torch.bfloat16)

    def run(dev):
        lg, xx, a1, a2, do = (t.to(dev) for t in (logits, x, w1, w2, dout))
        ids, w = M.route(lg, k)
        lay = M.align(ids, E)
        xs = M.gather(xx, lay)
        gu = M.grouped_fwd(xs, a1, lay)
        a = swiglu_fwd(gu)
        ys = M.grouped_fwd(a, a2, lay)
        out = M.combine(ys, w, lay)
        dys, dwt = M.combine_bwd(do, ys, w, lay)
        dw2 = M.grouped_wgrad(dys, a, torch.zeros(E, H, F, device=dev), lay)
        da = M.grouped_dgrad(dys, a2, lay)
        dgu = swiglu_bwd(da, gu)
        dw1 = M.grouped_wgrad(dgu, xs, torch.zeros(E, 2 * F, H, device=dev), lay)
        dx = M.scatter_sum(M.grouped_dgrad(dgu, a1, lay), lay)
        return [t.float().cpu() for t in (out, dwt, dw1, dw2, dx)]
    got, ref = run("cuda"), run("cpu")
    C.check_status()
    for name, a, b in zip(("out", "dw_router", "dw1", "dw2", "dx"), got, ref):
        scale = b.abs().max().clamp_min(1e-3)
        assert (a - b).abs().max() / scale < 3e-2, (name, float((a - b).abs().max()), float(scale))
