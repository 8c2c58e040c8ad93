"""Native sm_100a kernels vs the PyTorch fp32 reference path (same op called on CPU tensors)."""
import math

import pytest
import torch

from axon_b200.ops import _common as C
from axon_b200.ops import activation as A
from axon_b200.ops import attention as AT
from axon_b200.ops import norm as N
from axon_b200.ops import optim as O
from axon_b200.ops import rope as R

pytestmark = pytest.mark.gpu


def bf(*shape, scale=1.0):
    return (torch.randn(*shape) * scale).to(torch.bfloat16)


def close(a, b, atol, rtol=2e-2):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g} (tol {atol}); mean err {err.mean().item():.4g}"


@pytest.mark.parametrize("T,H", [(7, 256), (300, 4096), (64, 688 + 8), (33, 5120)])
def test_rmsnorm_fwd_bwd(T, H):
    torch.manual_seed(0)
    x, d, w, dy, dres = bf(T, H), bf(T, H), bf(H) * 0.1 + 1, bf(T, H), bf(T, H)
    y_r, rstd_r, xs_r = N.rmsnorm_fwd(x, w, 1e-6, delta=d)
    y, rstd, xs = N.rmsnorm_fwd(x.cuda(), w.cuda(), 1e-6, delta=d.cuda())
    close(y, y_r, 2e-2)
    close(xs, xs_r, 1e-2)
    close(rstd, rstd_r, 1e-3)
    y2, rstd2, _ = N.rmsnorm_fwd(x.cuda(), w.cuda(), 1e-6)
    close(y2, N.rmsnorm_fwd(x, w, 1e-6)[0], 2e-2)
    dw_r = torch.zeros(H)
    dx_r = N.rmsnorm_bwd(dy, xs_r, w, rstd_r, dw_r, dres=dres)
    dw = torch.zeros(H, device="cuda")
    dx = N.rmsnorm_bwd(dy.cuda(), xs.cuda(), w.cuda(), rstd, dw, dres=dres.cuda())
    close(dx, dx_r, 3e-2)
    close(dw, dw_r, 5e-2 * math.sqrt(T))
    C.check_status()


@pytest.mark.parametrize("T,Hq,Hkv,D,norm", [(50, 8, 2, 128, True), (129, 32, 8, 128, True), (40, 4, 4, 128, False),
                                           (31, 4, 2, 64, True)])
def test_qknorm_rope(T, Hq, Hkv, D, norm):
    torch.manual_seed(1)
    HT = Hq + 2 * Hkv
    qkv, dout = bf(T, HT * D), bf(T, HT * D)
    qw = (bf(D) * 0.1 + 1) if norm else None
    kw = (bf(D) * 0.1 + 1) if norm else None
    pos = torch.randint(0, 5000, (T,), dtype=torch.int32)
    cos, sin = R.rope_tables(8192, D, 1e6, "cpu")
    out_r = R.qknorm_rope_fwd(qkv, pos, cos, sin, Hq, Hkv, D, qw, kw)
    cg, sg = R.rope_tables(8192, D, 1e6, torch.device("cuda", 0))
    cu = lambda t: None if t is None else t.cuda()
    out = R.qknorm_rope_fwd(qkv.cuda(), pos.cuda(), cg, sg, Hq, Hkv, D, cu(qw), cu(kw))
    close(out, out_r, 3e-2)
    dqw_r, dkw_r = torch.zeros(D), torch.zeros(D)
    d_r = R.qknorm_rope_bwd(dout, qkv, pos, cos, sin, Hq, Hkv, D, qw, kw, dqw_r, dkw_r)
    dqw, dkw = torch.zeros(D, device="cuda"), torch.zeros(D, device="cuda")
    d = R.qknorm_rope_bwd(dout.cuda(), qkv.cuda(), pos.cuda(), cg, sg, Hq, Hkv, D, cu(qw), cu(kw), dqw, dkw)
    close(d, d_r, 4e-2)
    if norm:
        close(dqw, dqw_r, 5e-2 * math.sqrt(T * Hq))
        close(dkw, dkw_r, 5e-2 * math.sqrt(T * Hkv))
    C.check_status()


def test_swiglu_embedding_add():
    torch.manual_seed(2)
    T, F, V, H = 77, 1376, 1000, 256
    gu, da = bf(T, 2 * F), bf(T, F)
    close(A.swiglu_fwd(gu.cuda()), A.swiglu_fwd(gu), 2e-2)
    close(A.swiglu_bwd(da.cuda(), gu.cuda()), A.swiglu_bwd(da, gu), 3e-2)
    table, ids = bf(V, H), torch.randint(0, V, (T,), dtype=torch.int32)
    close(A.embedding_fwd(ids.cuda(), table.cuda()), A.embedding_fwd(ids, table), 0)
    dy = bf(T, H)
    dt = A.embedding_bwd(ids.cuda(), dy.cuda(), torch.zeros(V, H, device="cuda"))
    close(dt, A.embedding_bwd(ids, dy, torch.zeros(V, H)), 1e-3)
    a, b = bf(T, H), bf(T, H)
    close(A.add(a.cuda(), b.cuda()), A.add(a, b), 1e-2)


@pytest.mark.parametrize("lens,Hq,Hkv", [([128], 4, 4), ([256, 128], 4, 2), ([100, 300, 57, 513], 8, 2), ([1000], 32, 8)])
def test_attention_fwd_bwd(lens, Hq, Hkv):
    torch.manual_seed(3)
    D = 128
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    qkv = bf(T, (Hq + 2 * Hkv) * D, scale=0.7)
    do = bf(T, Hq * D)
    o_r, lse_r = AT.attn_fwd(qkv, cu, Hq, Hkv, D)
    o, lse = AT.attn_fwd(qkv.cuda(), cu.cuda(), Hq, Hkv, D)
    C.check_status()
    close(o, o_r, 2e-2)
    close(lse, lse_r, 2e-2)
    d_r = AT.attn_bwd(do, qkv, o_r, lse_r, cu, Hq, Hkv, D)
    d = AT.attn_bwd(do.cuda(), qkv.cuda(), o, lse, cu.cuda(), Hq, Hkv, D)
    C.check_status()
    close(d, d_r, 6e-2, rtol=5e-2)
    # run-twice determinism
    d2 = AT.attn_bwd(do.cuda(), qkv.cuda(), o, lse, cu.cuda(), Hq, Hkv, D)
    assert torch.equal(d, d2)


def test_adamw_and_clip():
    torch.manual_seed(4)
    n = 100_003
    master = torch.randn(n)
    grad = torch.randn(n) * 3
    m, v = torch.zeros(n), torch.zeros(n)
    mg, vg, pg = m.cuda(), v.cuda(), master.cuda()
    param = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    state_r, state = torch.zeros(4), torch.zeros(4, device="cuda")
    for g_dtype in (torch.float32, torch.bfloat16):
        g = grad.to(g_dtype)
        O.sumsq(g, state_r)
        O.sumsq(g.cuda(), state)
        close(state[:1], state_r[:1], 1e-2 * n, rtol=1e-4)
        O.clip_coef(state_r, 1.0)
        O.clip_coef(state, 1.0)
        close(state, state_r, 1e-3, rtol=1e-3)
        for step in (1, 2):
            O.adamw_step(master, None, g, m, v, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, state_r)
            O.adamw_step(pg, param, g.cuda(), mg, vg, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, state)
        close(pg, master, 1e-4, rtol=1e-4)
        close(param, master, 1e-2)
    # non-finite gradient -> step skipped
    bad = grad.clone()
    bad[5] = float("inf")
    O.sumsq(bad.cuda(), state)
    O.clip_coef(state, 1.0)
    before = pg.clone()
    O.adamw_step(pg, param, bad.cuda(), mg, vg, 1e-2, 0.9, 0.95, 1e-8, 0.1, 3, state)
    assert torch.equal(before, pg) and float(state[3]) == 1.0


@pytest.mark.parametrize("T,H,V,temp", [(100, 256, 1000, 1.0), (300, 512, 4096 + 24, 0.7), (513, 1024, 20000, 1.3)])
def test_lmhead_logprob_entropy(T, H, V, temp):
    from axon_b200.ops import lm_head as L
    torch.manual_seed(5)
    hidden, w = bf(T, H), bf(V, H, scale=0.05)
    labels = torch.randint(0, V, (T,), dtype=torch.int32)
    labels[3] = -100
    lp_r, ent_r, lse_r = L.lmhead_fwd(hidden, w, labels, temp)
    lp, ent, lse = L.lmhead_fwd(hidden.cuda(), w.cuda(), labels.cuda(), temp)
    C.check_status()
    close(lp, lp_r, 2e-2)
    close(ent, ent_r, 2e-2)
    close(lse, lse_r, 2e-2)
    g_lp, g_ent = torch.randn(T), torch.randn(T) * 0.1
    dw_r = torch.zeros(V, H)
    dh_r = L.lmhead_bwd(hidden, w, labels, lse_r, ent_r, g_lp, g_ent, temp, dweight=dw_r)
    dw = torch.zeros(V, H, device="cuda")
    dh = L.lmhead_bwd(hidden.cuda(), w.cuda(), labels.cuda(), lse, ent, g_lp.cuda(), g_ent.cuda(), temp, dweight=dw)
    C.check_status()
    close(dh, dh_r, 2e-2 * max(1.0, float(dh_r.abs().max())), rtol=5e-2)
    close(dw, dw_r, 2e-2 * max(1.0, float(dw_r.abs().max())), rtol=5e-2)


def test_lmhead_autograd_matches_torch():
    from axon_b200.ops import lm_head as L
    torch.manual_seed(6)
    T, H, V = 64, 256, 777 + 7
    hidden = bf(T, H).cuda().requires_grad_(True)
    w = bf(V, H, scale=0.05).cuda().requires_grad_(True)
    labels = torch.randint(0, V, (T,), dtype=torch.int32, device="cuda")
    lp, ent = L.linear_logprob_entropy(hidden, w, labels, 1.0)
    (lp.sum() * 0.5 - 0.01 * ent.sum()).backward()
    h2 = hidden.detach().float().requires_grad_(True)
    w2 = w.detach().float().requires_grad_(True)
    z = h2 @ w2.t()
    lsm = torch.log_softmax(z, -1)
    lp2 = lsm.gather(1, labels.long()[:, None])[:, 0]
    ent2 = -(lsm.exp() * lsm).sum(-1)
    (lp2.sum() * 0.5 - 0.01 * ent2.sum()).backward()
    close(lp, lp2, 2e-2)
    close(ent, ent2, 2e-2)
    close(hidden.grad, h2.grad, 2e-2, rtol=5e-2)
    close(w.grad, w2.grad, 3e-2, rtol=5e-2)


@pytest.mark.parametrize("lens,Hq,Hkv", [([5, 130, 257], 8, 2), ([1000, 40], 32, 8), ([3000], 8, 8)])
def test_paged_decode_and_kv_write(lens, Hq, Hkv):
    from axon_b200.ops import paged as P
    torch.manual_seed(7)
    D, B = 128, len(lens)
    max_pages = max((n + 127) // 128 for n in lens) + 1
    num_pages = sum((n + 127) // 128 for n in lens) + 3
    perm = torch.randperm(num_pages)
    bt = torch.full((B, max_pages), -1, dtype=torch.int32)
    nxt = 0
    for b, n in enumerate(lens):
        for i in range((n + 127) // 128):
            bt[b, i] = perm[nxt]
            nxt += 1
    HT = Hq + 2 * Hkv
    T = sum(lens)
    qkv = bf(T, HT * D, scale=0.7)
    tok_seq = torch.cat([torch.full((n,), b, dtype=torch.int32) for b, n in enumerate(lens)])
    tok_pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens])
    kc, vc = torch.zeros(num_pages, Hkv, 128, D, dtype=torch.bfloat16), torch.zeros(num_pages, Hkv, 128, D, dtype=torch.bfloat16)
    P.kv_write(qkv, kc, vc, tok_seq, tok_pos, bt, Hq, Hkv, D)
    kg, vg = torch.zeros_like(kc).cuda(), torch.zeros_like(vc).cuda()
    P.kv_write(qkv.cuda(), kg, vg, tok_seq.cuda(), tok_pos.cuda(), bt.cuda(), Hq, Hkv, D)
    assert torch.equal(kg.cpu(), kc) and torch.equal(vg.cpu(), vc)
    last = torch.tensor(lens).cumsum(0) - 1
    qlast = qkv[last]
    sl = torch.tensor(lens, dtype=torch.int32)
    o_r = P.paged_decode(qlast, kc, vc, bt, sl, Hq, Hkv, D)
    o = P.paged_decode(qlast.cuda(), kg, vg, bt.cuda(), sl.cuda(), Hq, Hkv, D)
    C.check_status()
    close(o, o_r, 2e-2)


def test_sampling_distribution_and_logprobs():
    from axon_b200.ops import paged as P
    torch.manual_seed(8)
    B, V = 6, 5000
    logits = (torch.randn(B, V) * 3).cuda()
    temp = torch.tensor([1.0, 0.7, 0.0, 1.0, 1.3, 1.0]).cuda()
    top_k = torch.tensor([0, 50, 0, 0, 20, 5], dtype=torch.int32).cuda()
    top_p = torch.tensor([1.0, 1.0, 1.0, 0.8, 0.9, 1.0]).cuda()
    ref_lp = P._ref_process(logits.cpu(), temp.cpu(), top_k.cpu(), top_p.cpu())
    counts = torch.zeros(B, V)
    n_draws = 300
    for it in range(n_draws):
        ctr = torch.full((B,), it, dtype=torch.int32, device="cuda")
        toks, lps = P.sample(logits, temp, top_k, top_p, seed=123, counters=ctr)
        toks, lps = toks.cpu().long(), lps.cpu()
        want = ref_lp.gather(1, toks[:, None])[:, 0]
        assert torch.isfinite(want).all(), "sampled a token outside the kept set"
        assert (lps - want).abs().max() < 2e-3, (lps, want)
        counts[torch.arange(B), toks] += 1
    assert counts[2].argmax() == logits[2].argmax().cpu() and counts[2].max() == n_draws
    assert (counts[5] > 0).sum() <= 5 and (counts[4] > 0).sum() <= 20
    # empirical frequency of the most likely token tracks its probability
    for b in (0, 3):
        top = ref_lp[b].argmax()
        pr = ref_lp[b, top].exp().item()
        assert abs(counts[b, top].item() / n_draws - pr) < 4 * (pr * (1 - pr) / n_draws) ** 0.5 + 0.02


@pytest.fixture
def persistent_decode():
    """Run the paged decode wrappers on the persistent kernels for the duration of a test."""
    from axon_b200.ops import paged as P
    old, P.DECODE_IMPL = P.DECODE_IMPL, "persistent"
    yield
    P.DECODE_IMPL = old


@pytest.mark.gpu
@pytest.mark.parametrize("lens,Hq,Hkv", [([1, 127, 128, 129, 700, 3000], 8, 2), ([5] * 40 + [2000] * 3 + [130] * 200, 32, 8),
                                          ([4096, 17], 4, 4)])
def test_persistent_paged_decode_matches_reference(persistent_decode, lens, Hq, Hkv):
    """One CTA per SM pulling (sequence, head, split) units from a counter: same numbers as the fp32 reference and as the
    one-CTA-per-unit kernel, on batches whose sequences differ in length by three orders of magnitude; twice in a row
    (the work counter is reset by every launch)."""
    from axon_b200.ops import paged as P
    torch.manual_seed(13)
    D, B = 128, len(lens)
    max_pages = max((n + 127) // 128 for n in lens) + 1
    num_pages = sum((n + 127) // 128 for n in lens) + 3
    perm = torch.randperm(num_pages)
    bt = torch.full((B, max_pages), -1, dtype=torch.int32)
    nxt = 0
    for b, n in enumerate(lens):
        for i in range((n + 127) // 128):
            bt[b, i] = perm[nxt]
            nxt += 1
    kc, vc = bf(num_pages, Hkv, 128, D, scale=0.7), bf(num_pages, Hkv, 128, D, scale=0.7)
    q = bf(B, (Hq + 2 * Hkv) * D, scale=0.7)
    sl = torch.tensor(lens, dtype=torch.int32)
    P.DECODE_IMPL = "classic"
    ref = P.paged_decode(q, kc, vc, bt, sl, Hq, Hkv, D)
    classic = P.paged_decode(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), sl.cuda(), Hq, Hkv, D)
    P.DECODE_IMPL = "persistent"
    for _ in range(2):
        got = P.paged_decode(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), sl.cuda(), Hq, Hkv, D)
        C.check_status()
        close(got, ref, 2e-2)
        close(got, classic, 2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (8, 1), (4, 4)])
def test_persistent_shared_prefix_decode(persistent_decode, Hq, Hkv):
    test_paged_decode_shared_prefix_matches_plain_decode(Hq, Hkv)


@pytest.mark.gpu
def test_sampling_full_vocabulary_logprob_mode():
    """With top-p / top-k active, ``logprobs_mode="full"`` returns the temperature-scaled log-softmax over the
    whole vocabulary for the token drawn from the truncated set."""
    from axon_b200.ops import paged as P
    torch.manual_seed(9)
    B, V = 4, 3000
    logits = (torch.randn(B, V) * 2).cuda()
    temp = torch.tensor([1.0, 0.8, 1.2, 1.0]).cuda()
    top_k = torch.tensor([0, 40, 0, 10], dtype=torch.int32).cuda()
    top_p = torch.tensor([0.5, 1.0, 0.7, 0.9]).cuda()
    kept = P._ref_process(logits.cpu(), temp.cpu(), top_k.cpu(), top_p.cpu())
    full = torch.log_softmax(logits.cpu().float() / temp.cpu()[:, None], -1)
    for it in range(20):
        ctr = torch.full((B,), it, dtype=torch.int32, device="cuda")
        toks, lps = P.sample(logits, temp, top_k, top_p, seed=5, counters=ctr, logprobs_mode="full")
        toks2, lps2 = P.sample(logits, temp, top_k, top_p, seed=5, counters=ctr)
        assert torch.equal(toks, toks2)                          # the draw does not depend on the reporting mode
        t = toks.cpu().long()
        assert torch.isfinite(kept.gather(1, t[:, None])).all()
        assert (lps.cpu() - full.gather(1, t[:, None])[:, 0]).abs().max() < 2e-3
        assert (lps2.cpu() - kept.gather(1, t[:, None])[:, 0]).abs().max() < 2e-3
        assert (lps <= lps2 + 1e-5).all()                        # truncation can only raise the reported probability


@pytest.mark.gpu
@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (8, 1), (4, 4)])
def test_paged_decode_shared_prefix_matches_plain_decode(Hq, Hkv):
    """Decode attention over a batch with shared prompt pages (one prefix item per group + a suffix item per
    sequence + merge) against the fp32 reference and the plain kernel; padded rows give zeros."""
    from axon_b200.ops import paged as P
    torch.manual_seed(11)
    D = 128
    rep = Hq // Hkv
    gmax = 32 // rep
    # (members, shared pages, private lengths)
    groups = [(min(8, gmax), 3, [5, 130, 128, 1, 300, 77, 256, 129]), (1, 0, [200]), (min(3, gmax), 1, [1, 64, 129]), (1, 0, [128])]
    rows, items = [], []
    page = 0
    for members, shared, priv in groups:
        shared_pages = list(range(page, page + shared)); page += shared
        first = len(rows)
        for m in range(members):
            n_priv = (priv[m] + 127) // 128
            rows.append((shared_pages + list(range(page, page + n_priv)), shared * 128 + priv[m], shared))
            page += n_priv
        if members >= 2:
            items.append((first, members, shared))
    B, Bpad = len(rows), len(rows) + 3                 # three padded rows, as in a graph bucket
    num_pages = page + 2
    max_pages = max(len(r[0]) for r in rows) + 1
    bt = torch.full((Bpad, max_pages), -1, dtype=torch.int32)
    sl = torch.zeros(Bpad, dtype=torch.int32)
    for b, (pg, n, _) in enumerate(rows):
        bt[b, :len(pg)] = torch.tensor(pg, dtype=torch.int32)
        sl[b] = n
    kc, vc = bf(num_pages, Hkv, 128, D, scale=0.7), bf(num_pages, Hkv, 128, D, scale=0.7)
    q = bf(Bpad, (Hq + 2 * Hkv) * D, scale=0.7)
    ng = max(1, Bpad // 2)
    z = lambda n: torch.zeros(n, dtype=torch.int32)     # noqa: E731
    sh = dict(seq_first=torch.arange(Bpad, dtype=torch.int32), seq_one=torch.ones(Bpad, dtype=torch.int32), seq_page0=z(Bpad),
              seq_keys=sl.clone(), grp_first=z(ng), grp_size=z(ng), grp_zero=z(ng), grp_keys=z(ng))
    for n, (a, m, s) in enumerate(items):
        sh["grp_first"][n], sh["grp_size"][n], sh["grp_keys"][n] = a, m, s * 128
        sh["seq_page0"][a:a + m] = s
        sh["seq_keys"][a:a + m] -= s * 128
    ref = P.paged_decode(q, kc, vc, bt, sl, Hq, Hkv, D)
    qg, kg, vg = q.cuda(), kc.cuda(), vc.cuda()
    plain = P.paged_decode(qg, kg, vg, bt.cuda(), sl.cuda(), Hq, Hkv, D)
    shg = {k: v.cuda() for k, v in sh.items()}
    shg["max_shared_pages"] = 4
    got = P.paged_decode_shared(qg, kg, vg, bt.cuda(), sl.cuda(), shg, Hq, Hkv, D)
    C.check_status()
    close(got[:B], ref[:B], 2e-2)
    close(got[:B], plain[:B], 2e-2)
    assert float(got[B:].abs().max()) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("D,Hq,Hkv", [(128, 8, 2), (128, 4, 4)])
def test_qknorm_rope_with_fused_kv_cache_write(D, Hq, Hkv):
    """One launch = QK-norm + RoPE and the K / V rows in their cache pages: against the two separate ops."""
    from axon_b200.ops import paged as P
    from axon_b200.ops import rope as R
    torch.manual_seed(5)
    T, page, max_pages, num_pages = 37, 128, 4, 16
    qkv = bf(T, (Hq + 2 * Hkv) * D).cuda()
    pos = torch.randperm(max_pages * page)[:T].to(torch.int32).cuda()      # distinct slots: no two tokens race for one
    tok_seq = torch.randint(0, 3, (T,), dtype=torch.int32).cuda()
    bt = torch.randperm(num_pages)[: 3 * max_pages].view(3, max_pages).to(torch.int32).cuda()
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.arange(max_pages * page).float()[:, None] * inv[None, :]
    cos_t, sin_t = ang.cos().cuda(), ang.sin().cuda()
    qw, kw = (bf(D) * 0.1 + 1).cuda(), (bf(D) * 0.1 + 1).cuda()
    k1, v1 = torch.zeros(num_pages, Hkv, page, D, dtype=torch.bfloat16, device="cuda"), torch.zeros(num_pages, Hkv, page, D, dtype=torch.bfloat16, device="cuda")
    k2, v2 = torch.zeros_like(k1), torch.zeros_like(v1)
    ref = R.qknorm_rope_fwd(qkv, pos, cos_t, sin_t, Hq, Hkv, D, qw, kw)
    P.kv_write(ref, k1, v1, tok_seq, pos, bt, Hq, Hkv, D)
    got = R.qknorm_rope_fwd(qkv, pos, cos_t, sin_t, Hq, Hkv, D, qw, kw, kv_cache=(k2, v2, tok_seq, bt))
    assert torch.equal(got, ref) and torch.equal(k1, k2) and torch.equal(v1, v2)
    assert float(k2.abs().sum()) > 0
