"""tcgen05 GEMM parity against an fp32 PyTorch reference, incl. ragged edges and all majors."""
import pytest
import torch

from axon_b200.ops import gemm as G
from axon_b200.ops import _common as C

SHAPES = [(128, 256, 64), (256, 512, 256), (304, 200, 136), (1024, 4096, 4096), (72, 24, 72),
          (4096, 1024, 512), (136, 136, 8)]


def _rand(*shape):
    return (torch.randn(*shape, device="cuda") * 0.5).to(torch.bfloat16)


def _check(out, ref, K):
    tol = 2e-2 * (K ** 0.5) * 0.25 + 1e-2
    err = (out.float() - ref).abs().max().item()
    assert err < tol, f"max err {err} tol {tol}"


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
    assert torch.equal(G.gemm_nt(a, b), G.gemm_nt(a, b))
    C.check_status()
