"""RMSNorm backward through the entry point that brings its own workspace.

The symbol is called through ctypes exactly as a C host would call it; results are compared with the
regular entry point (caller-owned workspace) and with a plain fp32 PyTorch reference, on two calls in
a row. The file sorts last so that it also runs after every other GPU test has used the device.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from axon_b200 import _native
    lib = _native.lib()
    lib.axb_rmsnorm_bwd_static_error.restype = ctypes.c_char_p
    return lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else None)


def _inputs(T, H, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    dy = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    dres = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    return x, dy, dres, w, rstd


def _reference(x, dy, dres, w, rstd):
    xh = x.float() * rstd[:, None]
    gg = dy.float() * w.float()
    dx = rstd[:, None] * (gg - xh * (gg * xh).mean(-1, keepdim=True)) + dres.float()
    return dx, (dy.float() * xh).sum(0)


def _call_static(lib, x, dy, dres, w, rstd, dw, accumulate):
    """The raw call, bracketed by a check that it took no device memory: neither through PyTorch's allocator
    (``memory_allocated`` / ``memory_reserved``) nor behind its back (free bytes reported by the driver)."""
    T, H = x.shape
    dx = torch.empty_like(x)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    before = (torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
    rc = lib.axb_rmsnorm_bwd_static(_p(dy), _p(x), _p(w), _p(rstd), _p(dres), _p(dx), _p(dw), int(accumulate),
                                    ctypes.c_longlong(T), int(H), stream)
    torch.cuda.synchronize()
    after = (torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
    assert after[1:] == before[1:], (before, after)
    assert after[0] >= before[0], (before, after)          # other processes may free memory meanwhile, this call takes none
    return rc, dx


@pytest.mark.parametrize("T,H", [(1000, 4096), (77, 1024), (3000, 2048)])
def test_static_workspace_matches_regular_entry_point(T, H):
    from axon_b200.ops import norm
    lib = _lib()
    torch.cuda.set_device(0)
    assert lib.axb_rmsnorm_bwd_static_setup() == 0, lib.axb_rmsnorm_bwd_static_error()
    for call in range(2):                                   # two calls in a row reuse the workspace
        x, dy, dres, w, rstd = _inputs(T, H, seed=call)
        dw_ref = torch.zeros(H, device="cuda")
        dx_ref = norm.rmsnorm_bwd(dy, x, w, rstd, dw_ref, dres=dres, accumulate_dw=False)
        dw = torch.full((H,), 7.0, device="cuda")           # overwritten, not accumulated
        rc, dx = _call_static(lib, x, dy, dres, w, rstd, dw, accumulate=False)
        assert rc == 0, lib.axb_rmsnorm_bwd_static_error()
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref)
        torch.testing.assert_close(dw, dw_ref, rtol=1e-5, atol=1e-4)
        dx32, dw32 = _reference(x, dy, dres, w, rstd)
        torch.testing.assert_close(dx.float(), dx32, rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(dw, dw32, rtol=2e-3, atol=2e-2)
        rc, _ = _call_static(lib, x, dy, dres, w, rstd, dw, accumulate=True)   # accumulate on top
        assert rc == 0
        torch.cuda.synchronize()
        torch.testing.assert_close(dw, 2 * dw_ref, rtol=1e-5, atol=2e-4)


def test_static_workspace_refuses_oversize_and_bad_shapes():
    lib = _lib()
    T, H = 4096, 8192                                       # 592 partial rows x 8192 floats > the workspace
    x, dy, dres, w, rstd = _inputs(8, H, seed=3)
    dw = torch.zeros(H, device="cuda")
    dx = torch.empty(8, H, device="cuda", dtype=torch.bfloat16)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # refused on the host before any launch, so the (short) buffers are never touched
    rc = lib.axb_rmsnorm_bwd_static(_p(dy), _p(x), _p(w), _p(rstd), _p(dres), _p(dx), _p(dw), 0,
                                    ctypes.c_longlong(T), int(H), stream)
    assert rc == -5
    assert b"workspace" in lib.axb_rmsnorm_bwd_static_error()
    rc = lib.axb_rmsnorm_bwd_static(_p(dy), _p(x), _p(w), _p(rstd), _p(dres), _p(dx), _p(dw), 0,
                                    ctypes.c_longlong(8), 8190, stream)
    assert rc == -1
    rc, _ = _call_static(lib, x, dy, dres, w, rstd, dw, accumulate=False)      # 8 rows x 8192 fits
    assert rc == 0
    torch.cuda.synchronize()
    assert lib.axb_rmsnorm_bwd_static_error() == b""
