"""Gated delta rule: CPU recurrence against a closed form on a tiny case, the CUDA kernel against the recurrence
(incl. state carry-over across two calls), gradients through the autograd wrapper."""
import pytest
import torch

from axon_b200.ops.gdn import gated_delta_rule, gated_delta_rule_ref


def _inputs(T=37, H=3, dk=64, dv=48, seed=0, dev="cpu", dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(T, H, dk, generator=g), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(T, H, dk, generator=g), dim=-1)
    v = torch.randn(T, H, dv, generator=g)
    gl = -torch.nn.functional.softplus(torch.randn(T, H, generator=g))
    beta = torch.sigmoid(torch.randn(T, H, generator=g))
    return [t.to(dev).to(dtype if t.dim() == 3 else torch.float32) for t in (q, k, v, gl, beta)]


def test_recurrence_reduces_to_decayed_linear_attention_when_beta_keys_orthogonal():
    # one head, orthonormal keys, beta = 1: S^T k_t = 0 for unseen keys, so o_t = scale * sum_s decay(s..t) (q_t.k_s) v_s
    T, dk, dv = 8, 64, 5
    k = torch.eye(dk)[:T].unsqueeze(1)
    q = torch.randn(T, 1, dk)
    v = torch.randn(T, 1, dv)
    gl = -torch.rand(T, 1)
    beta = torch.ones(T, 1)
    cu = torch.tensor([0, T])
    o, _ = gated_delta_rule_ref(q, k, v, gl, beta, cu, scale=1.0)
    cum = gl[:, 0].cumsum(0)
    want = torch.stack([sum(torch.exp(cum[t] - cum[s]) * (q[t, 0] @ k[s, 0]) * v[s, 0] for s in range(t + 1)) for t in range(T)])
    torch.testing.assert_close(o[:, 0], want, rtol=1e-5, atol=1e-5)


def test_state_carry_over_equals_one_pass_cpu():
    q, k, v, gl, beta = _inputs()
    cu = torch.tensor([0, 37])
    o_full, s_full = gated_delta_rule(q, k, v, gl, beta, cu)
    o1, s1 = gated_delta_rule(q[:20], k[:20], v[:20], gl[:20], beta[:20], torch.tensor([0, 20]))
    o2, s2 = gated_delta_rule(q[20:], k[20:], v[20:], gl[20:], beta[20:], torch.tensor([0, 17]), initial_state=s1)
    torch.testing.assert_close(torch.cat([o1, o2]), o_full, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(s2, s_full, rtol=1e-5, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("dk,dv", [(64, 48), (128, 128), (256, 64)])
def test_kernel_matches_recurrence_gpu(dk, dv):
    q, k, v, gl, beta = _inputs(T=150, H=4, dk=dk, dv=dv, dev="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0, 60, 61, 150], dtype=torch.int32, device="cuda")
    o, st = gated_delta_rule(q, k, v, gl, beta, cu)
    o_r, st_r = gated_delta_rule_ref(q, k, v, gl, beta, cu)
    torch.testing.assert_close(o.float(), o_r, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(st, st_r, rtol=2e-2, atol=2e-2)
    # carry-over through the kernel
    o1, s1 = gated_delta_rule(q[:60], k[:60], v[:60], gl[:60], beta[:60], cu[:2])
    torch.testing.assert_close(o1.float(), o_r[:60], rtol=3e-2, atol=3e-2)
    # gradients through the wrapper
    qq = q.clone().requires_grad_(True)
    vv = v.clone().requires_grad_(True)
    og, _ = gated_delta_rule(qq, k, vv, gl, beta, cu)
    og.float().square().sum().backward()
    assert qq.grad is not None and vv.grad is not None and float(vv.grad.abs().sum()) > 0


@pytest.mark.gpu
@pytest.mark.parametrize("dk,dv,with_state", [(64, 48, False), (128, 128, True), (256, 64, True)])
def test_backward_kernel_matches_autograd_of_the_recurrence_gpu(dk, dv, with_state):
    """Reverse-sweep kernel (chunk replay, per-slice partials) against autograd through the fp32 PyTorch recurrence on
    the same bf16 inputs: all five input gradients, and the gradient of an initial state, over ragged sequences that
    span several chunks, with a gradient flowing into the final state as well."""
    from axon_b200.ops import _common as C
    from axon_b200.ops import gdn as G
    q, k, v, gl, beta = _inputs(T=150, H=4, dk=dk, dv=dv, dev="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0, 70, 71, 150], dtype=torch.int32, device="cuda")
    gen = torch.Generator().manual_seed(3)
    do = (torch.randn(150, 4, dv, generator=gen) * 0.5).cuda().to(torch.bfloat16)
    dst = (torch.randn(3, 4, dk, dv, generator=gen) * 0.1).cuda()
    init = (torch.randn(3, 4, dk, dv, generator=gen) * 0.2).cuda() if with_state else None

    def grads(native):
        G.NATIVE_BACKWARD = native
        leaves = [t.detach().clone().requires_grad_(True) for t in (q, k, v, gl, beta)]
        s0 = init.detach().clone().requires_grad_(True) if init is not None else None
        o, st = gated_delta_rule(*leaves, cu, initial_state=s0)
        ((o.float() * do.float()).sum() + (st * dst).sum()).backward()
        return [t.grad.float() for t in leaves] + ([s0.grad.float()] if s0 is not None else [])
    try:
        got, want = grads(True), grads(False)
    finally:
        G.NATIVE_BACKWARD = True
    C.check_status()
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dbeta", "dstate"), got, want):
        tol = 3e-2 * max(1.0, float(b.abs().max()))
        assert float((a - b).abs().max()) < tol, (name, float((a - b).abs().max()), tol)


@pytest.mark.gpu
def test_family_delta_rule_runs_on_the_kernels_gpu():
    """The linear-attention layers of the Qwen3-Next / Qwen3.5 families call the CUDA kernels for bf16 CUDA tensors:
    outputs, final state and input gradients agree with the fp32 PyTorch recurrence of the same function."""
    from axon_b200.models.families import gated_delta_rule as family_rule
    q, k, v, gl, beta = _inputs(T=90, H=2, dk=128, dv=64, seed=4)
    st0 = torch.randn(2, 128, 64) * 0.1

    def run(dev, dtype):
        leaves = [t.detach().clone().to(dev).to(dtype if t.dim() == 3 else torch.float32).requires_grad_(True) for t in (q, k, v, gl, beta)]
        o, st = family_rule(*leaves, state=st0.to(dev))
        (o.float().square().sum() + st.sum()).backward()
        return o.float().cpu(), st.float().cpu(), [t.grad.float().cpu() for t in leaves]
    o_ref, st_ref, g_ref = run("cpu", torch.float32)
    o, st, g = run("cuda", torch.bfloat16)
    torch.testing.assert_close(o, o_ref, rtol=4e-2, atol=4e-2)
    torch.testing.assert_close(st, st_ref, rtol=3e-2, atol=3e-2)
    for a, b in zip(g, g_ref):
        assert float((a - b).abs().max()) < 5e-2 * max(1.0, float(b.abs().max()))
