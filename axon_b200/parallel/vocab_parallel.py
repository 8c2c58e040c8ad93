"""Log-prob and entropy over a vocabulary that is sharded across a tensor-parallel group.

Each rank holds logits (or computes them from its slice of the output head) for a contiguous
vocabulary range. Per token the ranks exchange four numbers — running max, sum of exponentials,
sum of p*x, and the label's logit (owned by exactly one rank) — which is all log-softmax and
entropy need; no rank ever sees another rank's logits (reference: the three all-reduces of
axon/utils/megatron/tensor_parallel.py:109-139, axon/utils/kernel/kernels.py:644-676 and the
soft-capped variant axon/models/mcore/forward/softcap_cross_entropy.py:44-160).

Here the exchange is ONE all-gather of a ``[T, 4]`` fp32 block followed by a fixed-order merge, so the
result is bit-identical on every rank and independent of reduction order. The autograd functions
give exact gradients with respect to the local logits.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _gather_stats(stats: torch.Tensor, group) -> torch.Tensor:
    """[T, 4] -> [W, T, 4] (rank order)."""
    w = dist.get_world_size(group) if group is not None and dist.is_initialized() else 1
    if w == 1:
        return stats.unsqueeze(0)
    out = torch.empty(w, *stats.shape, dtype=stats.dtype, device=stats.device)
    dist.all_gather_into_tensor(out.view(-1, stats.shape[-1]), stats.contiguous(), group=group)
    return out


def merge_softmax_stats(all_stats: torch.Tensor):
    """Combine per-shard (max, sumexp, sum e*x, label logit) in rank order -> (lse, E[x], label logit)."""
    m = all_stats[..., 0].max(dim=0).values
    scale = torch.exp(all_stats[..., 0] - m)
    sumexp = (all_stats[..., 1] * scale).sum(0)
    sum_ex = (all_stats[..., 2] * scale).sum(0)
    label = all_stats[..., 3].sum(0)
    return m + torch.log(sumexp), sum_ex / sumexp, label


def local_softmax_stats(logits: torch.Tensor, labels: torch.Tensor, vocab_start: int):
    """Per-token stats of this rank's vocabulary slice ``[vocab_start, vocab_start + V_local)``."""
    x = logits.float()
    m = x.max(-1).values
    e = torch.exp(x - m.unsqueeze(-1))
    local = labels - vocab_start
    mine = (local >= 0) & (local < x.shape[-1])
    lab = torch.where(mine, x.gather(-1, local.clamp(0, x.shape[-1] - 1).unsqueeze(-1)).squeeze(-1), torch.zeros_like(m))
    return torch.stack([m, e.sum(-1), (e * x).sum(-1), lab], dim=-1), mine, local


class _VocabParallelLogProbEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, vocab_start, group):
        stats, mine, local = local_softmax_stats(logits, labels, vocab_start)
        lse, mean_x, label = merge_softmax_stats(_gather_stats(stats, group))
        ctx.save_for_backward(logits, lse, mean_x, mine, local)
        return label - lse, lse - mean_x

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        logits, lse, mean_x, mine, local = ctx.saved_tensors
        x = logits.float()
        p = torch.exp(x - lse.unsqueeze(-1))
        grad = torch.zeros_like(x)
        if g_lp is not None:
            g = g_lp.float().unsqueeze(-1)
            grad -= g * p
            onehot_rows = torch.nonzero(mine).flatten()
            grad[onehot_rows, local[onehot_rows]] += g_lp.float()[onehot_rows]
        if g_ent is not None:
            grad -= g_ent.float().unsqueeze(-1) * p * (x - mean_x.unsqueeze(-1))
        return grad.to(logits.dtype), None, None, None


def vocab_parallel_log_probs_and_entropy(vocab_parallel_logits, labels, vocab_start: int, group=None):
    shape = labels.shape
    lp, ent = _VocabParallelLogProbEntropy.apply(vocab_parallel_logits.reshape(-1, vocab_parallel_logits.shape[-1]),
                                                 labels.reshape(-1), vocab_start, group)
    return lp.view(shape), ent.view(shape)


def vocab_parallel_entropy(vocab_parallel_logits, vocab_start: int = 0, group=None):
    labels = torch.zeros(vocab_parallel_logits.shape[:-1], dtype=torch.long, device=vocab_parallel_logits.device)
    return vocab_parallel_log_probs_and_entropy(vocab_parallel_logits, labels, vocab_start, group)[1]


def vocab_parallel_log_probs_from_logits(logits, labels, vocab_start: int = 0, group=None):
    return vocab_parallel_log_probs_and_entropy(logits, labels, vocab_start, group)[0]


def softcap_linear_cross_entropy(hidden, weight_shard, labels, vocab_start: int, temperature: float = 1.0,
                                 softcap: float | None = None, group=None, chunk_size: int = 1024):
    """Vocab-parallel log-prob / entropy from hidden states with tanh soft-capped logits, chunked over
    tokens. Differentiable through ``hidden`` and ``weight_shard`` (autograd of the chunk graph)."""
    lps, ents = [], []
    h2 = hidden.reshape(-1, hidden.shape[-1])
    lab = labels.reshape(-1)
    for s in range(0, h2.shape[0], chunk_size):
        logits = (h2[s:s + chunk_size] @ weight_shard.t()).float()
        if softcap:
            logits = torch.tanh(logits / softcap) * softcap
        lp, ent = vocab_parallel_log_probs_and_entropy(logits / temperature, lab[s:s + chunk_size], vocab_start, group)
        lps.append(lp)
        ents.append(ent)
    return torch.cat(lps).view(labels.shape), torch.cat(ents).view(labels.shape)
