"""tcgen05 GEMM parity against an fp32 PyTorch reference, incl. ragged edges and all majors."""
import pytest
import torch

from axon_b200.ops import gemm as G
from axon_b200.ops import _common as C

SHAPES = [(128, 256, 64), (256, 512, 256), (304, 200, 136), (1024, 4096, 4096), (72, 24, 72),
          (4096, 1024, 512), (136, 136, 8), (200, 264, 16), (128, 128, 24), (392, 136, 40)]


def _rand(*shape):
    return (torch.randn(*shape, device="cuda") * 0.5).to(torch.bfloat16)


def _check(out, ref, K):
    """bf16 outputs: half an ulp of the result's magnitude (inputs ~N(0, 0.25), so |ref| ~ 0.25 sqrt(K)) plus slack.
    fp32 outputs carry only the accumulation-order error of exact bf16 products: 1e-3 of the result's scale."""
    scale = 0.25 * (K ** 0.5)
    err = (out.float() - ref).abs().max().item()
    if out.dtype == torch.float32:
        tol = 1e-3 * max(scale, ref.abs().max().item()) + 1e-5
    else:
        tol = 2e-2 * scale + 1e-2
    assert err < tol, f"max err {err} tol {tol} dtype {out.dtype}"


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_nt(M, N, K):
    M = M + 3 if M in (304, 72) else M  # K-major operands allow any row count
    a, b = _rand(M, K), _rand(N, K)
    ref = a.float() @ b.float().t()
    _check(G.gemm_nt(a, b), ref, K)
    _check(G.gemm_nt(a, b, out_dtype=torch.float32), ref, K)
    for bn in (64, 128, 256):
        _check(G.gemm_nt(a, b, bn_hint=bn), ref, K)
    C.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_nn_tn(M, N, K):
    a, b = _rand(M, K), _rand(K, N)
    ref = a.float() @ b.float()
    _check(G.gemm_nn(a, b), ref, K)
    at = a.t().contiguous()
    _check(G.gemm_tn(at, b, out_dtype=torch.float32), ref, K)
    C.check_status()


@pytest.mark.gpu
def test_gemm_accumulate_and_alpha():
    M, N, K = 256, 384, 192
    a, b = _rand(M, K), _rand(N, K)
    base = torch.randn(M, N, device="cuda")
    out = base.clone()
    G.gemm_nt(a, b, out=out, accumulate=True, alpha=0.5)
    _check(out, base + 0.5 * (a.float() @ b.float().t()), K)
    C.check_status()


@pytest.mark.gpu
def test_gemm_deterministic():
    a, b = _rand(512, 1024), _rand(768, 1024)
    assert torch.equal(G.gemm_nt(a, b), G.gemm_nt(a, b))


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(1, 512, 256), (17, 1024, 4096), (64, 6144, 4096), (100, 4096, 12288),
                                   (256, 24576 // 4, 4096), (200, 8192 + 40, 1024)])
def test_gemm_small_m_swap_ab(M, N, K):
    a, b = _rand(M, K), _rand(N, K)
    ref = a.float() @ b.float().t()
    _check(G.gemm_nt(a, b), ref, K)
    _check(G.gemm_nt(a, b, out_dtype=torch.float32), ref, K)
    _check(G.gemm_nt(a, b), ref, K)      # (bit-reproducibility is a property of the ordered split-K variants, tested below)
    C.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(1, 512, 256), (5, 1024, 512), (17, 1024, 4096), (64, 6144, 4096), (65, 4096, 4096),
                                   (128, 4096, 12288), (129, 6144, 4096), (256, 6144, 4096), (256, 4096, 12288),
                                   (200, 2048 + 40, 1024), (256, 1000, 576)])
def test_gemm_decode_cluster_matches_reference_and_split_kernel(M, N, K):
    """Cluster split-K kernel (partials reduced through distributed shared memory): against fp32
    PyTorch, against the global-workspace split-K kernel, run-to-run bit identical, and the batch
    rows do not depend on the batch size (row i of a 1-row and an M-row product agree)."""
    lib = C.lib()
    a, b = _rand(M, K), _rand(N, K)
    ref = a.float() @ b.float().t()
    cs = lib.axb_gemm_decode_cluster_size(M, N, K)
    assert 0 <= cs <= 8
    G.USE_CLUSTER_DECODE, G.USE_STREAM_DECODE = True, False
    try:
        out = G.gemm_nt(a, b)
        out32 = G.gemm_nt(a, b, out_dtype=torch.float32)
        again = G.gemm_nt(a, b)
        _check(out, ref, K)
        _check(out32, ref, K)
        assert torch.equal(out, again)
        G.USE_CLUSTER_DECODE = False
        old32 = G.gemm_nt(a, b, out_dtype=torch.float32)
    finally:
        G.USE_CLUSTER_DECODE, G.USE_STREAM_DECODE = True, True
    torch.testing.assert_close(out32, old32, rtol=1e-4, atol=1e-3 * (K ** 0.5) / 16)
    C.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(1, 512, 256), (5, 1024, 512), (17, 1024, 4096), (48, 6144, 4096), (64, 4096, 4096),
                                   (100, 4096, 12288), (129, 6144, 4096), (160, 24576, 4096), (256, 6144, 4096),
                                   (200, 2048 + 40, 1024), (256, 1000, 576), (33, 151936, 1024)])
def test_gemm_stream_matches_reference(M, N, K):
    """Weight-streaming decode kernel: against fp32 PyTorch for bf16 and fp32 outputs, bit-identical
    from run to run (the split-K sum order is fixed although the reducing CTA is not), under several
    forced plans (no split, many splits, one 256-wide token tile), and its arrival counters are back at
    zero after every launch."""
    a, b = _rand(M, K), _rand(N, K)
    ref = a.float() @ b.float().t()
    assert G.USE_STREAM_DECODE
    try:
        for knobs in (dict(), dict(force_splits=1), dict(force_splits=2), dict(force_splits=3), dict(force_splits=7, max_bn=256),
                      dict(max_bn=64, ring_kb_one=60, ring_kb_two=40, x_depth=2), dict(two_per_sm_tiles=1, force_splits=2, pdl=0),
                      dict(accumulate=0), dict(accumulate=0, force_splits=5, max_bn=256)):
            G.stream_tune(**G.STREAM_DEFAULTS)
            G.stream_tune(**knobs)
            out = G.gemm_nt(a, b)
            out32 = G.gemm_nt(a, b, out_dtype=torch.float32)
            _check(out, ref, K)
            _check(out32, ref, K)
            again = G.gemm_nt(a, b)
            if knobs.get("accumulate", 1) == 0 or knobs.get("force_splits", 0) in (1, 2):
                assert torch.equal(out, again), knobs            # fixed summation order
            else:
                _check(again, ref, K)
            for cnt in G._STREAM_COUNTERS.values():
                assert int(cnt.abs().sum()) == 0
            for acc in G._STREAM_ACC.values():
                assert float(acc.abs().max()) == 0.0             # accumulation tiles are left zeroed
    finally:
        G.stream_tune(**G.STREAM_DEFAULTS)
    C.check_status()


@pytest.mark.gpu
def test_gemm_decode_cluster_selection():
    lib = C.lib()
    assert lib.axb_gemm_decode_cluster_size(256, 6144, 4096) in (2, 3)   # 48 tiles: 3 only if 48 clusters of 3 fit at once
    assert lib.axb_gemm_decode_cluster_size(256, 4096, 4096) in (3, 4)   # 32 tiles x 4
    assert lib.axb_gemm_decode_cluster_size(256, 24576, 4096) == 0       # enough tiles without splitting
    assert lib.axb_gemm_decode_cluster_size(8, 512, 256) in (0, 1, 2, 4)  # 4 K blocks: at most 1 split of >= 4
