"""Canary bands around every buffer the op wrappers allocate: each output (and scratch) tensor is carved out of a
larger allocation whose leading and trailing 4 KiB are filled with a pattern; after the kernels have run on ragged
shapes the bands must be untouched. Catches stores past the edge of a tile that happen to land in memory the
allocator owns (which a plain numerics check never sees)."""
import contextlib

import pytest
import torch

pytestmark = pytest.mark.gpu

BAND = 4096          # bytes on each side
PATTERN = 0xA5


class Canaries:
    def __init__(self):
        self.records = []
        self._empty, self._empty_like = torch.empty, torch.empty_like

    def _alloc(self, shape, dtype, device):
        n = 1
        for s in shape:
            n *= int(s)
        item = torch.empty(0, dtype=dtype).element_size()
        payload = (n * item + 255) // 256 * 256
        raw = self._empty(BAND + payload + BAND, dtype=torch.uint8, device=device)
        raw.fill_(PATTERN)
        self.records.append((raw, payload))
        return raw[BAND:BAND + n * item].view(dtype).view(*shape) if n else self._empty(*shape, dtype=dtype, device=device)

    def empty(self, *size, dtype=None, device=None, **kw):
        dev = torch.device(device) if device is not None else torch.device("cpu")
        if dev.type != "cuda" or kw.get("pin_memory"):
            return self._empty(*size, dtype=dtype, device=device, **kw)
        shape = size[0] if len(size) == 1 and isinstance(size[0], (tuple, list, torch.Size)) else size
        return self._alloc(tuple(shape), dtype or torch.get_default_dtype(), dev)

    def empty_like(self, t, dtype=None, device=None, **kw):
        dev = torch.device(device) if device is not None else t.device
        if dev.type != "cuda":
            return self._empty_like(t, dtype=dtype, device=device, **kw)
        return self._alloc(tuple(t.shape), dtype or t.dtype, dev)

    def check(self):
        torch.cuda.synchronize()
        assert self.records, "no allocation went through the canary allocator"
        for raw, payload in self.records:
            head, tail = raw[:BAND], raw[BAND + payload:]
            assert bool((head == PATTERN).all()) and bool((tail == PATTERN).all()), \
                f"a kernel wrote outside a {payload}-byte buffer"


@contextlib.contextmanager
def canaries():
    c = Canaries()
    torch.empty, torch.empty_like = c.empty, c.empty_like
    try:
        yield c
    finally:
        torch.empty, torch.empty_like = c._empty, c._empty_like
    c.check()


def _bf(*shape, scale=0.5):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("M,N,K", [(136, 136, 8), (304, 200, 136), (72, 24, 72), (1000, 520, 264)])
def test_gemm_edges_stay_inside_their_outputs(M, N, K):
    from axon_b200.ops import _common as C
    from axon_b200.ops import gemm as G
    a, b, bt = _bf(M, K), _bf(N, K), _bf(K, N)
    with canaries():
        y1 = G.gemm_nt(a, b)
        y2 = G.gemm_nn(a, bt, out_dtype=torch.float32)
        y3 = G.gemm_tn(a.t().contiguous(), bt)
    C.check_status()
    ref = a.float() @ b.float().t()
    assert (y1.float() - ref).abs().max() < 0.05 * K ** 0.5 + 0.05
    assert (y3.float() - y2).abs().max() < 0.05 * K ** 0.5 + 0.05


def test_elementwise_and_norm_kernels_stay_inside_their_outputs():
    from axon_b200.ops import _common as C
    from axon_b200.ops import activation as A
    from axon_b200.ops import norm as N
    T, H, F = 77, 1032, 520
    x, d, w = _bf(T, H), _bf(T, H), _bf(H)
    gu, da = _bf(T, 2 * F), _bf(T, F)
    ids = torch.randint(0, 300, (T,), dtype=torch.int32, device="cuda")
    table = _bf(300, H)
    dw = torch.zeros(H, device="cuda")
    with canaries():
        y, rstd, xs = N.rmsnorm_fwd(x, w, 1e-6, delta=d)
        N.rmsnorm_bwd(y, xs, w, rstd, dw, dres=d)
        a = A.swiglu_fwd(gu)
        A.swiglu_bwd(da, gu)
        e = A.embedding_fwd(ids, table)
    C.check_status()
    assert torch.equal(e, table[ids.long()]) and torch.isfinite(a.float()).all()


def test_attention_with_ragged_sequences_stays_inside_its_outputs():
    from axon_b200.ops import _common as C
    from axon_b200.ops import attention as AT
    Hq, Hkv, D = 4, 2, 128
    lens = [1, 130, 77, 256, 3]
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    qkv = _bf(T, (Hq + 2 * Hkv) * D)
    with canaries():
        o, lse = AT.attn_fwd(qkv, cu, Hq, Hkv, D)
        do = torch.randn_like(o)
        dqkv = AT.attn_bwd(do, qkv, o, lse, cu, Hq, Hkv, D)
    C.check_status()
    assert torch.isfinite(o.float()).all() and torch.isfinite(dqkv.float()).all()


def test_fused_head_and_sampler_stay_inside_their_outputs():
    from axon_b200.ops import _common as C
    from axon_b200.ops import lm_head as LM
    from axon_b200.ops import paged as P
    T, H, V = 200, 256, 5003 // 8 * 8 + 8
    h, w = _bf(T, H), _bf(V, H, scale=0.1)
    labels = torch.randint(0, V, (T,), dtype=torch.int32, device="cuda")
    logits = torch.randn(9, 4999, device="cuda")
    with canaries():
        lp, ent, lse = LM.lmhead_fwd(h, w, labels, 1.0)
        toks, lps = P.sample(logits, torch.ones(9, device="cuda"), None, None, seed=1,
                             counters=torch.zeros(9, dtype=torch.int32, device="cuda"))
    C.check_status()
    ref = torch.log_softmax(h.float() @ w.float().t(), -1).gather(1, labels.long()[:, None])[:, 0]
    assert (lp.float() - ref).abs().max() < 0.1 and int(toks.max()) < 4999
