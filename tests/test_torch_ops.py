"""Logits-path helpers, the chunked PyTorch vocabulary head (with soft-capping) and the
vocabulary-parallel log-prob / entropy exchange."""
import torch
import torch.nn.functional as F

from axon_b200.parallel import vocab_parallel as VP
from axon_b200.utils.torch import ops as O
from axon_b200.utils.torch.fused_linear import FusedLinearForPPO


def test_logits_helpers():
    torch.manual_seed(0)
    logits, labels = torch.randn(6, 50), torch.randint(0, 50, (6,))
    ref = F.log_softmax(logits, -1).gather(-1, labels[:, None]).squeeze(-1)
    torch.testing.assert_close(O.logprobs_from_logits(logits, labels), ref)
    torch.testing.assert_close(O.logprobs_from_logits_v2(logits, labels), ref)
    ent = -(F.softmax(logits, -1) * F.log_softmax(logits, -1)).sum(-1)
    torch.testing.assert_close(O.entropy_from_logits(logits), ent)
    torch.testing.assert_close(O.entropy_from_logits_with_chunking(logits, 4), ent)
    v, m = torch.tensor([[1.0, 2.0, float("nan")]]), torch.tensor([[1.0, 1.0, 0.0]])
    assert abs(O.masked_mean(v, m).item() - 1.5) < 1e-6
    assert O.get_response_mask(torch.tensor([[5, 2, 7, 2]]), eos_token=2).tolist() == [[1, 1, 0, 0]]
    am = torch.tensor([[1, 1, 0], [1, 1, 1]])
    idx, cu, mx = O.get_unpad_data(am)
    assert idx.tolist() == [0, 1, 3, 4, 5] and cu.tolist() == [0, 2, 5] and mx == 3
    assert O.pad_from_left([[1], [2, 3]], 0) == [[0, 1], [2, 3]]
    w = O.masked_whiten(torch.randn(4, 8), torch.ones(4, 8))
    assert abs(w.mean().item()) < 1e-5 and abs(w.var().item() - 1) < 1e-3


def test_chunked_head_matches_autograd_with_softcap():
    torch.manual_seed(1)
    T, H, V = 37, 16, 64
    h = torch.randn(T, H, requires_grad=True)
    w = torch.randn(V, H, requires_grad=True)
    labels = torch.randint(0, V, (T,))
    for cap in (None, 5.0):
        lp, ent = FusedLinearForPPO(chunk_size=8, softcap=cap)(h, w, labels, temperature=0.7)
        logits = h @ w.t()
        if cap:
            logits = torch.tanh(logits / cap) * cap
        z = logits / 0.7
        lp_ref = F.log_softmax(z, -1).gather(-1, labels[:, None]).squeeze(-1)
        ent_ref = -(F.softmax(z, -1) * F.log_softmax(z, -1)).sum(-1)
        torch.testing.assert_close(lp, lp_ref, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(ent, ent_ref, rtol=1e-5, atol=1e-5)
        gl, ge = torch.randn(T), torch.randn(T)
        g1 = torch.autograd.grad((lp * gl).sum() + (ent * ge).sum(), (h, w))
        g2 = torch.autograd.grad((lp_ref * gl).sum() + (ent_ref * ge).sum(), (h, w))
        for a, b in zip(g1, g2):
            torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-4)


def test_vocab_parallel_stats_merge_equals_full_softmax():
    """Emulates 4 vocabulary shards in one process: merging their per-token stats reproduces the
    full-vocabulary log-prob / entropy and the gradients of each shard's logits."""
    torch.manual_seed(2)
    T, V, W = 9, 64, 4
    logits = torch.randn(T, V) * 3
    labels = torch.randint(0, V, (T,))
    shards = [logits[:, r * 16:(r + 1) * 16].clone().requires_grad_(True) for r in range(W)]
    stats = torch.stack([VP.local_softmax_stats(s, labels, r * 16)[0] for r, s in enumerate(shards)])
    lse, mean_x, lab = VP.merge_softmax_stats(stats)
    full = logits.clone().requires_grad_(True)
    lp_ref = F.log_softmax(full, -1).gather(-1, labels[:, None]).squeeze(-1)
    ent_ref = -(F.softmax(full, -1) * F.log_softmax(full, -1)).sum(-1)
    torch.testing.assert_close(lab - lse, lp_ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(lse - mean_x, ent_ref, rtol=1e-5, atol=1e-5)
    # single-rank group: the autograd function alone must match autograd of the dense formula
    lp, ent = VP.vocab_parallel_log_probs_and_entropy(full, labels, 0, None)
    gl, ge = torch.randn(T), torch.randn(T)
    g = torch.autograd.grad((lp * gl).sum() + (ent * ge).sum(), full)[0]
    full2 = logits.clone().requires_grad_(True)
    lp2 = F.log_softmax(full2, -1).gather(-1, labels[:, None]).squeeze(-1)
    ent2 = -(F.softmax(full2, -1) * F.log_softmax(full2, -1)).sum(-1)
    g2 = torch.autograd.grad((lp2 * gl).sum() + (ent2 * ge).sum(), full2)[0]
    torch.testing.assert_close(g, g2, rtol=1e-4, atol=1e-5)
    lp3, ent3 = VP.softcap_linear_cross_entropy(torch.randn(T, 8), torch.randn(V, 8), labels, 0, temperature=0.9, softcap=4.0, chunk_size=4)
    assert lp3.shape == (T,) and (ent3 > 0).all()
