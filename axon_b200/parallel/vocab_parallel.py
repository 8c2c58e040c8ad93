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


# ---------------------------------------------------------------------------------------------------
# Fused head over a sharded vocabulary (hidden states row-sharded, head weight row-sharded)
# ---------------------------------------------------------------------------------------------------
class VocabParallelHead:
    """log-prob / entropy of the local tokens when the output head is split over the tensor-parallel
    group by vocabulary rows and the final hidden states are split by token rows.

    CUDA: one tcgen05 GEMM per rank reads every rank's hidden shard in place (all-gather fused),
    keeps per-token soft-max statistics in its epilogue, and a merge kernel sends four floats per token
    to the rank that owns the token (peer stores); after a device barrier the owner finishes
    log-prob / entropy. No logits, no gathered hidden states, no NCCL collective in the data path.
    Backward recomputes logits tiles into ``dlogits`` for the local vocabulary shard, gets
    d hidden by GEMM -> reduce-scatter and the weight gradient from the explicitly gathered hidden rows.
    CPU / gloo: the same mathematics with all-gathers and the autograd function above.
    """

    def __init__(self, tp, vocab_size: int):
        self.tp = tp
        assert vocab_size % tp.world == 0, "vocabulary must split evenly over the tensor-parallel group"
        self.vl = vocab_size // tp.world
        self.v0 = tp.rank * self.vl
        self._stats = self._hbuf = None

    def _local_labels(self, labels: torch.Tensor) -> torch.Tensor:
        loc = labels.to(torch.int64) - self.v0
        mine = (loc >= 0) & (loc < self.vl) & (labels >= 0)
        other = torch.where(labels >= 0, torch.full_like(loc, -2), torch.full_like(loc, -1))
        return torch.where(mine, loc, other).to(torch.int32)

    def forward(self, h_local: torch.Tensor, w_shard: torch.Tensor, labels_full: torch.Tensor, temperature: float = 1.0):
        """h_local [T/W, H]; w_shard [V/W, H]; labels_full int [T] (global ids, <0 ignored).
        Returns (logprob, entropy) of the local rows and a context for ``backward``."""
        tp = self.tp
        rows = h_local.shape[0]
        T = rows * tp.world
        sl = slice(tp.rank * rows, (tp.rank + 1) * rows)
        lab_loc = self._local_labels(labels_full)
        if not tp.fused:
            h_full = tp.all_gather_rows(h_local)
            logits = (h_full.float() @ w_shard.float().t()) / temperature
            stats, _, _ = local_softmax_stats(logits, labels_full.to(torch.long).clamp_min(0), self.v0)
            stats[:, 3] = torch.where(lab_loc >= 0, stats[:, 3], torch.zeros_like(stats[:, 3]))
            lse, mean_x, lab = merge_softmax_stats(_gather_stats(stats, tp.group))
            lp = torch.where(labels_full >= 0, lab - lse, torch.zeros_like(lse))
            ctx = dict(h_local=h_local, w=w_shard, lab_loc=lab_loc, lse=lse, ent=lse - mean_x, temperature=temperature, sl=sl)
            return lp[sl].contiguous(), (lse - mean_x)[sl].contiguous(), ctx
        import ctypes

        from ..ops import _common as C
        from .symm import SymmetricBuffer
        H = h_local.shape[1]
        if self._hbuf is None or self._hbuf.numel < rows * H:
            self._hbuf = SymmetricBuffer(rows * H, torch.bfloat16, tp.group, tp.device)
            self._stats = SymmetricBuffer(tp.world * rows * 4, torch.float32, tp.group, tp.device)
        self._hbuf.tensor[: rows * H].view(rows, H).copy_(h_local)
        tp._align_streams()
        tp.barrier()
        lib = C.lib()
        scratch = C.workspace(tp.device, lib.axb_lmhead_scratch_bytes(ctypes.c_longlong(T), self.vl), "lmhead")
        # Every vocabulary tile of the stats GEMM streams all hidden rows, and peer memory is not cached on the
        # reading side: handing the kernel the peers' buffers would move the remote rows over NVLink once per tile
        # (hundreds of times for a 76 k-column shard). The peers' rows are therefore copied once into local memory
        # and the kernel's per-rank pointers point into that copy.
        h_all = torch.empty(tp.world, rows, H, dtype=torch.bfloat16, device=tp.device)
        for r in range(tp.world):
            h_all[r].copy_(h_local if r == tp.rank else self._hbuf.peer_tensor(r, rows * H).view(rows, H))
        h_ptrs = (ctypes.c_ulonglong * tp.world)(*[h_all[r].data_ptr() for r in range(tp.world)])
        rc = lib.axb_lmhead_vp_stats(h_ptrs, tp.world, tp.rank, C.ptr(w_shard), C.ptr(lab_loc), rows, self.vl, H,
                                     ctypes.c_longlong(H), ctypes.c_longlong(w_shard.stride(0)), ctypes.c_float(temperature),
                                     C.ptr(scratch), self._stats.ptr_array(), C.ptr(C.status(tp.device)), C.stream())
        C.launched(rc, "lmhead_vp_stats", 2)
        tp._align_streams()
        tp.barrier()
        lp = torch.empty(rows, dtype=torch.float32, device=tp.device)
        ent, lse = torch.empty_like(lp), torch.empty_like(lp)
        lab_rows = labels_full[sl].to(torch.int32).contiguous()
        rc = lib.axb_lmhead_vp_finish(C.ptr(self._stats.tensor), C.ptr(lab_rows), C.ptr(lp), C.ptr(ent), C.ptr(lse), tp.world, rows,
                                      C.stream())
        C.launched(rc, "lmhead_vp_finish")
        ctx = dict(h_local=h_local, w=w_shard, lab_loc=lab_loc, lse_local=lse, ent_local=ent, temperature=temperature, sl=sl)
        return lp, ent, ctx

    def backward(self, ctx: dict, g_lp_local, g_ent_local, dweight: torch.Tensor | None = None) -> torch.Tensor:
        """Returns d hidden of the local rows; accumulates this rank's head-weight gradient into ``dweight``."""
        tp = self.tp
        h_local, w, lab_loc, temp = ctx["h_local"], ctx["w"], ctx["lab_loc"], ctx["temperature"]
        rows = h_local.shape[0]
        z = lambda t: t.float().contiguous() if t is not None else torch.zeros(rows, dtype=torch.float32, device=h_local.device)  # noqa: E731
        g_lp_full = tp.all_gather_rows(z(g_lp_local))
        g_ent_full = tp.all_gather_rows(z(g_ent_local))
        h_full = tp.all_gather_rows(h_local)
        if not tp.fused:
            lse, ent = ctx["lse"], ctx["ent"]
            zlog = (h_full.float() @ w.float().t()) / temp
            p = torch.exp(zlog - lse[:, None])
            glp = torch.where((lab_loc >= 0) | (lab_loc == -2), g_lp_full, torch.zeros_like(g_lp_full))
            d = -glp[:, None] * p - g_ent_full[:, None] * p * (zlog - lse[:, None] + ent[:, None])
            own = torch.nonzero(lab_loc >= 0).flatten()
            d[own, lab_loc[own].long()] += glp[own]
            d = (d / temp).to(h_local.dtype)
            if dweight is not None:
                dweight.add_((d.float().t() @ h_full.float()).to(dweight.dtype))
            return tp.reduce_scatter_rows((d.float() @ w.float()).to(h_local.dtype))
        import ctypes

        from ..ops import _common as C
        from ..ops import gemm as G
        lse_full = tp.all_gather_rows(ctx["lse_local"])
        ent_full = tp.all_gather_rows(ctx["ent_local"])
        T, H = h_full.shape
        dl = torch.empty(T, self.vl, dtype=torch.bfloat16, device=tp.device)
        rc = C.lib().axb_lmhead_dlogits(C.ptr(h_full), C.ptr(w), C.ptr(lab_loc), C.ptr(lse_full), C.ptr(ent_full), C.ptr(g_lp_full),
                                        C.ptr(g_ent_full), C.ptr(dl), ctypes.c_longlong(self.vl), T, self.vl, H, ctypes.c_longlong(H),
                                        ctypes.c_longlong(w.stride(0)), ctypes.c_float(temp), C.ptr(C.status(tp.device)), C.stream())
        C.launched(rc, "lmhead_dlogits")
        if dweight is not None:
            G.gemm_tn(dl, h_full, out=dweight, accumulate=True)
        return tp.gemm_reduce_scatter(dl, w, w_is_kn=True)
