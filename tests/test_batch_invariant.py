import pytest
import torch

from axon_b200.ops import batch_invariant as BI
from axon_b200.ops import gemm as G


def test_mode_switch_and_cpu_fallbacks():
    assert not BI.is_batch_invariant_mode_enabled()
    with BI.batch_invariant_mode():
        assert BI.is_batch_invariant_mode_enabled() and G.FIXED_CONFIG
        with BI.batch_invariant_mode(False):
            assert not G.FIXED_CONFIG
        assert G.FIXED_CONFIG
    assert not G.FIXED_CONFIG
    x = torch.randn(5, 33)
    torch.testing.assert_close(BI.log_softmax(x), torch.log_softmax(x, -1))
    torch.testing.assert_close(BI.mean_dim(x), x.mean(-1))


@pytest.mark.gpu
def test_rows_do_not_depend_on_batch_size():
    torch.manual_seed(0)
    w = (torch.randn(2048, 1024, device="cuda") * 0.05).to(torch.bfloat16)
    x = (torch.randn(300, 1024, device="cuda")).to(torch.bfloat16)
    with BI.batch_invariant_mode():
        full = G.gemm_nt(x, w, out_dtype=torch.float32)
        for n in (1, 7, 64, 129, 256):
            part = G.gemm_nt(x[:n].contiguous(), w, out_dtype=torch.float32)
            assert torch.equal(part, full[:n]), n
        ls_full = BI.log_softmax(full)
        assert torch.equal(BI.log_softmax(full[:3].contiguous()), ls_full[:3])
        assert torch.equal(BI.mean_dim(full[:5].contiguous()), BI.mean_dim(full)[:5])
    torch.testing.assert_close(ls_full, torch.log_softmax(full, -1), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(BI.mean_dim(x), x.float().mean(-1), rtol=1e-5, atol=1e-6)
    ref = x.float() @ w.float().t()
    assert (full - ref).abs().max() < 0.05
