"""Sequence-length balancing: partition sequences into k groups of similar cost, and split a batch
into micro-batches under a hard token cap.

Same cost model and entry points as the reference (axon/utils/seqlen_balancing.py:31-467):
``workload(s) = 24576 s + s^2`` (dense 7B-class block), Karmarkar-Karp largest-differencing with an
optional equal-size constraint, a greedy LPT alternative, ``rearrange_micro_batches`` (retries with
more splits until every micro-batch fits; optional MAX-sync of the count over a DP group),
``prepare_dynamic_batch`` / ``restore_dynamic_batch``.
"""
from __future__ import annotations

import heapq

import numpy as np
import torch


def calculate_workload(seqlen_list):
    s = torch.as_tensor(seqlen_list) if not isinstance(seqlen_list, (torch.Tensor, np.ndarray)) else seqlen_list
    return 24576 * s + s ** 2


def ceildiv(a, b):
    return -(a // -b)


def roundup_divisible(a, b):
    return ((a + b - 1) // b) * b


def karmarkar_karp(seqlen_list, k_partitions: int, equal_size: bool):
    """Largest differencing method for k-way partitioning. Returns k lists of indices."""
    n = len(seqlen_list)
    # A state is a tuple of k bins sorted by descending sum; heap keyed by (max - min) spread.
    def make_state(bins):
        bins = sorted(bins, key=lambda b: (-b[0], -len(b[1])))
        return (-(bins[0][0] - bins[-1][0]), next(counter), bins)

    counter = iter(range(1 << 62))
    heap = []
    order = sorted(range(n), key=lambda i: (seqlen_list[i], i))
    if equal_size:
        assert n % k_partitions == 0, f"{n} items cannot be split into {k_partitions} equal partitions"
        for s in range(0, n, k_partitions):
            grp = order[s:s + k_partitions]
            heapq.heappush(heap, make_state([(int(seqlen_list[i]), [i]) for i in grp]))
    else:
        for i in order:
            bins = [(int(seqlen_list[i]), [i])] + [(0, []) for _ in range(k_partitions - 1)]
            heapq.heappush(heap, make_state(bins))
    while len(heap) > 1:
        _, _, a = heapq.heappop(heap)
        _, _, b = heapq.heappop(heap)
        # pair the largest bin of one state with the smallest of the other
        merged = [(a[i][0] + b[k_partitions - 1 - i][0], a[i][1] + b[k_partitions - 1 - i][1])
                  for i in range(k_partitions)]
        heapq.heappush(heap, make_state(merged))
    bins = heap[0][2] if heap else [(0, []) for _ in range(k_partitions)]
    parts = [sorted(b[1]) for b in bins]
    if equal_size:
        assert all(len(p) == n // k_partitions for p in parts)
    return parts


def greedy_partition(seqlen_list, k_partitions: int, equal_size: bool):
    """Longest-processing-time greedy: assign each item (longest first) to the lightest bin."""
    bias = (max(seqlen_list) * len(seqlen_list) + 1) if equal_size and len(seqlen_list) else 0
    sums = [0] * k_partitions
    parts = [[] for _ in range(k_partitions)]
    for i in sorted(range(len(seqlen_list)), key=lambda i: -seqlen_list[i]):
        j = min(range(k_partitions), key=lambda b: sums[b])
        parts[j].append(i)
        sums[j] += seqlen_list[i] + bias
    if equal_size:
        assert all(len(p) == len(seqlen_list) // k_partitions for p in parts)
    return [sorted(p) for p in parts]


def get_seqlen_balanced_partitions(seqlen_list, k_partitions: int, equal_size: bool):
    """k index lists covering 0..n-1 exactly once with balanced sums, sorted by first index."""
    assert len(seqlen_list) >= k_partitions, f"{len(seqlen_list)} items < {k_partitions} partitions"
    parts = karmarkar_karp(list(map(int, seqlen_list)), k_partitions, equal_size)
    seen = sorted(i for p in parts for i in p)
    assert seen == list(range(len(seqlen_list))) and all(parts), "partitioning lost or duplicated an item"
    return sorted(parts, key=lambda p: p[0])


def log_seqlen_unbalance(seqlen_list, partitions, prefix):
    k = len(partitions)
    per = len(seqlen_list) // k
    naive = [sum(seqlen_list[i * per:(i + 1) * per]) for i in range(k)]
    bal = [sum(seqlen_list[i] for i in p) for p in partitions]
    return {f"{prefix}/min": min(naive), f"{prefix}/max": max(naive), f"{prefix}/minmax_diff": max(naive) - min(naive),
            f"{prefix}/balanced_min": min(bal), f"{prefix}/balanced_max": max(bal),
            f"{prefix}/mean": sum(naive) / k}


def _select_rows(batch, idx):
    t = torch.as_tensor(idx, dtype=torch.long)
    return batch[t]


def rearrange_micro_batches(batch, max_token_len, dp_group=None, num_batches_divided_by=None,
                            same_micro_num_in_dp=True, min_num_micro_batch=None, use_dynamic_bsz_balance=True,
                            strict_equal=False):
    """Split ``batch`` (needs ``attention_mask`` [B,S]) into micro-batches whose total real tokens never
    exceed ``max_token_len``. Returns (micro_batches, index_lists). With ``dp_group`` the count is raised to
    the group's maximum (ONE collective per call, so ranks cannot fall out of step); ``strict_equal``
    additionally refuses a rank that has fewer rows than that count (groups whose ranks exchange
    activations inside the model need exactly equal counts)."""
    lens = batch["attention_mask"].sum(1).to(torch.long).cpu()
    B = lens.numel()
    assert int(lens.max()) <= max_token_len, f"a sequence of {int(lens.max())} tokens exceeds the cap {max_token_len}"
    total = int(lens.sum())
    cost = calculate_workload(lens).tolist() if use_dynamic_bsz_balance else lens.tolist()

    def split(n):
        parts = get_seqlen_balanced_partitions(cost, n, equal_size=False)
        return parts, max(int(lens[torch.tensor(p)].sum()) for p in parts)

    n = max(1, min(B, ceildiv(total, max_token_len)))
    if min_num_micro_batch is not None:
        n = min(B, max(n, min_num_micro_batch))
    if num_batches_divided_by is not None:
        n = min(B, roundup_divisible(n, num_batches_divided_by))
    parts, worst = split(n)
    while worst > max_token_len and n < B:
        n += 1
        parts, worst = split(n)
    if dp_group is not None and same_micro_num_in_dp and torch.distributed.is_initialized():
        t = torch.tensor([n], device="cuda" if torch.distributed.get_backend(dp_group) == "nccl" else "cpu")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=dp_group)
        n_all = int(t.item())
        if num_batches_divided_by is not None:
            n_all = roundup_divisible(n_all, num_batches_divided_by)
        if strict_equal:
            assert B >= n_all, (f"this rank holds {B} rows but its group runs {n_all} micro-batches; give every rank at least "
                                f"as many rows as micro-batches (raise the token cap or the batch size)")
        if min(n_all, B) != n:
            n = min(n_all, B)
            parts, worst = split(n)
    if use_dynamic_bsz_balance:   # heavier micro-batches first
        parts.sort(key=lambda p: -sum(int(lens[i]) ** 2 for i in p))
    return [_select_rows(batch, p) for p in parts], parts


def get_reverse_idx(idx_map):
    rev = [0] * len(idx_map)
    for i, j in enumerate(idx_map):
        rev[j] = i
    return rev


def prepare_dynamic_batch(data, max_token_len: int, dp_group=None, num_batches_divided_by=None,
                          same_micro_num_in_dp=True, min_num_micro_batch=None, use_dynamic_bsz_balance=True,
                          strict_equal=False):
    """DataProto -> (list of micro DataProtos, index lists) under the token cap."""
    mbs, idx = rearrange_micro_batches(data.batch, max_token_len, dp_group, num_batches_divided_by,
                                       same_micro_num_in_dp, min_num_micro_batch, use_dynamic_bsz_balance, strict_equal)
    out = []
    for p in idx:
        d = data.select_idxs(torch.tensor(p, dtype=torch.long))
        d.meta_info = data.meta_info
        out.append(d)
    return out, idx


def restore_dynamic_batch(data: torch.Tensor, batch_idx_list) -> torch.Tensor:
    """Undo the row permutation of ``prepare_dynamic_batch`` on a concatenated per-row result."""
    flat = [i for p in batch_idx_list for i in p]
    assert len(flat) == data.shape[0], f"{len(flat)} indices vs {data.shape[0]} rows"
    return data[torch.tensor(get_reverse_idx(flat), dtype=torch.long, device=data.device)]
