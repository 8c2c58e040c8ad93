"""Sampler-side ops: paged KV-cache write, paged decode attention, token sampling with log-probs.

Native sm_100a kernels on CUDA; straightforward PyTorch on CPU (the oracle and the CPU config).
Cache layout per layer: ``K, V: [num_pages, Hkv, 128, D]``; ``block_table[seq, i]`` is the page
that holds positions ``[128*i, 128*i+128)`` of sequence ``seq``.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from . import _common as C

PAGE = 128
# Decode attention kernels: "persistent" (default) runs one warp-specialised CTA per SM that pulls (sequence or group,
# kv head, key split) work units from a counter and keeps its TMA tile ring running across them
# (csrc/paged_attention_persist.cu); "classic" launches one CTA per unit. Same arguments, same results.
DECODE_IMPL = os.environ.get("AXON_PAGED_DECODE", "persistent")
_PLAIN_ITEMS: dict = {}


def _plain_items(B: int, device) -> dict:
    """Item arrays that describe a batch without shared prefixes: one item per sequence over all of its pages."""
    key = (B, str(device))
    it = _PLAIN_ITEMS.get(key)
    if it is None:
        z = torch.zeros(B, dtype=torch.int32, device=device)
        it = _PLAIN_ITEMS[key] = dict(seq_first=torch.arange(B, dtype=torch.int32, device=device),
                                      seq_one=torch.ones(B, dtype=torch.int32, device=device), seq_page0=z, zero=z)
    return it


def _decode_persistent(qkv_r, kcache, vcache, block_table, seq_lens, shared, Hq, Hkv, D, scale):
    lib = C.lib()
    B = qkv_r.shape[0]
    max_pages = block_table.shape[1]
    ns = lib.axb_paged_decode_splits(B, Hkv, max_pages)
    if shared is None:
        it = _plain_items(B, qkv_r.device)
        first, one, page0, keys = it["seq_first"], it["seq_one"], it["seq_page0"], seq_lens
        gf = gs = gz = gk = it["zero"]
        n_groups, nsp = 0, 1
    else:
        first, one, page0, keys = shared["seq_first"], shared["seq_one"], shared["seq_page0"], shared["seq_keys"]
        gf, gs, gz, gk = shared["grp_first"], shared["grp_size"], shared["grp_zero"], shared["grp_keys"]
        n_groups = gf.numel()
        nsp = lib.axb_paged_decode_splits(int(shared.get("typical_groups", max(1, B // 8))), Hkv, int(shared.get("max_shared_pages", 8)))
    nslots = ns if n_groups == 0 else ns + nsp
    scratch = C.workspace(qkv_r.device, B * Hq * nslots * (D + 2) * 4, "paged")
    counters = C.workspace(qkv_r.device, 64, "paged_counters")
    out = torch.empty(B, Hq * D, dtype=qkv_r.dtype, device=qkv_r.device)
    rc = lib.axb_paged_decode_shared_persist(C.ptr(qkv_r), ctypes.c_longlong(qkv_r.stride(0)), C.ptr(kcache), C.ptr(vcache),
                                             kcache.shape[0], C.ptr(block_table), max_pages, C.ptr(first), C.ptr(one), C.ptr(page0),
                                             C.ptr(keys), C.ptr(gf), C.ptr(gs), C.ptr(gz), C.ptr(gk), n_groups, C.ptr(out), B, Hq, Hkv,
                                             D, ctypes.c_float(scale), ns, nsp, C.ptr(scratch), C.ptr(counters),
                                             C.ptr(C.status(qkv_r.device)), C.stream())
    C.launched(rc, "paged_decode_persist", 1 if (n_groups == 0 and ns == 1) else (2 if n_groups == 0 else 3))
    return out


def kv_write(qkv_r, kcache, vcache, tok_seq, tok_pos, block_table, Hq, Hkv, D):
    """Copy the (rotated) K and V head rows of every packed token into its cache page."""
    T = qkv_r.shape[0]
    if not C.use_native(qkv_r):
        x = qkv_r.view(T, Hq + 2 * Hkv, D)
        pages = block_table[tok_seq.long(), (tok_pos // PAGE).long()].long()
        off = (tok_pos % PAGE).long()
        kcache[pages, :, off] = x[:, Hq:Hq + Hkv].to(kcache.dtype)
        vcache[pages, :, off] = x[:, Hq + Hkv:].to(vcache.dtype)
        return
    rc = C.lib().axb_kv_write(C.ptr(qkv_r), C.ptr(kcache), C.ptr(vcache), C.ptr(tok_seq), C.ptr(tok_pos),
                              C.ptr(block_table), block_table.shape[1], ctypes.c_longlong(T), Hq, Hkv, D,
                              kcache.shape[0], C.stream())
    C.launched(rc, "kv_write")


def paged_decode(qkv_r, kcache, vcache, block_table, seq_lens, Hq, Hkv, D, scale=None):
    """One query token per sequence against its paged KV (which already includes that token).
    qkv_r: [B, (Hq+2Hkv)*D]; returns o [B, Hq*D]."""
    B = qkv_r.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not C.use_native(qkv_r):
        q = qkv_r.view(B, Hq + 2 * Hkv, D)[:, :Hq].float()
        out = torch.zeros(B, Hq, D)
        rep = Hq // Hkv
        for b in range(B):
            n = int(seq_lens[b])
            if n == 0:
                continue
            npg = (n + PAGE - 1) // PAGE
            pg = block_table[b, :npg].long()
            k = kcache[pg].float().permute(1, 0, 2, 3).reshape(Hkv, npg * PAGE, D)[:, :n]
            v = vcache[pg].float().permute(1, 0, 2, 3).reshape(Hkv, npg * PAGE, D)[:, :n]
            k = k.repeat_interleave(rep, 0)
            v = v.repeat_interleave(rep, 0)
            s = torch.einsum("hd,hnd->hn", q[b], k) * scale
            out[b] = torch.einsum("hn,hnd->hd", s.softmax(-1), v)
        return out.reshape(B, Hq * D).to(qkv_r.dtype)
    if DECODE_IMPL == "persistent":
        return _decode_persistent(qkv_r, kcache, vcache, block_table, seq_lens, None, Hq, Hkv, D, scale)
    lib = C.lib()
    max_pages = block_table.shape[1]
    ns = lib.axb_paged_decode_splits(B, Hkv, max_pages)
    scratch = C.workspace(qkv_r.device, B * Hq * ns * (D + 2) * 4, "paged") if ns > 1 else None
    out = torch.empty(B, Hq * D, dtype=qkv_r.dtype, device=qkv_r.device)
    rc = lib.axb_paged_decode(C.ptr(qkv_r), ctypes.c_longlong(qkv_r.stride(0)), C.ptr(kcache), C.ptr(vcache),
                              kcache.shape[0], C.ptr(block_table), max_pages, C.ptr(seq_lens), C.ptr(out), B,
                              Hq, Hkv, D, ctypes.c_float(scale), ns, C.ptr(scratch),
                              C.ptr(C.status(qkv_r.device)), C.stream())
    C.launched(rc, "paged_decode", 2 if ns > 1 else 1)
    return out


def paged_decode_shared(qkv_r, kcache, vcache, block_table, seq_lens, shared: dict, Hq, Hkv, D, scale=None):
    """``paged_decode`` for a batch in which groups of consecutive sequences share their first pages (the n
    samples of one prompt): the shared pages are attended to once per group, every sequence's private
    pages once per sequence, and the partial results are merged. ``shared`` holds int32 device tensors:
    ``seq_first`` (arange), ``seq_one`` (1 per row), ``seq_page0`` / ``seq_keys`` (first private page and the
    keys from there on), ``grp_first`` / ``grp_size`` / ``grp_zero`` / ``grp_keys`` (first member, member count
    - 0 for unused entries -, zeros, shared keys). Same result as ``paged_decode`` with ``seq_lens``."""
    if not C.use_native(qkv_r):
        return paged_decode(qkv_r, kcache, vcache, block_table, seq_lens, Hq, Hkv, D, scale)
    B = qkv_r.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if DECODE_IMPL == "persistent":
        return _decode_persistent(qkv_r, kcache, vcache, block_table, seq_lens, shared, Hq, Hkv, D, scale)
    lib = C.lib()
    max_pages = block_table.shape[1]
    n_groups = shared["grp_first"].numel()
    ns = lib.axb_paged_decode_splits(B, Hkv, max_pages)
    # splits of the prefix items: sized for the usual group count (8 samples per prompt), not for the array length
    nsp = lib.axb_paged_decode_splits(int(shared.get("typical_groups", max(1, B // 8))), Hkv, int(shared.get("max_shared_pages", 8)))
    scratch = C.workspace(qkv_r.device, B * Hq * (ns + nsp) * (D + 2) * 4, "paged")
    out = torch.empty(B, Hq * D, dtype=qkv_r.dtype, device=qkv_r.device)
    rc = lib.axb_paged_decode_shared(C.ptr(qkv_r), ctypes.c_longlong(qkv_r.stride(0)), C.ptr(kcache), C.ptr(vcache), kcache.shape[0],
                                     C.ptr(block_table), max_pages, C.ptr(shared["seq_first"]), C.ptr(shared["seq_one"]),
                                     C.ptr(shared["seq_page0"]), C.ptr(shared["seq_keys"]), C.ptr(shared["grp_first"]),
                                     C.ptr(shared["grp_size"]), C.ptr(shared["grp_zero"]), C.ptr(shared["grp_keys"]), n_groups,
                                     C.ptr(out), B, Hq, Hkv, D, ctypes.c_float(scale), ns, nsp, C.ptr(scratch),
                                     C.ptr(C.status(qkv_r.device)), C.stream())
    C.launched(rc, "paged_decode_shared", 3)
    return out


def _ref_process(logits, temperature, top_k, top_p):
    """Processed log-probs (after temperature / top-k / top-p), fp32 [B,V]; rows with T<=0 get argmax one-hot."""
    B, V = logits.shape
    z = logits.float().clone()
    out = torch.empty_like(z)
    for b in range(B):
        t = float(temperature[b]) if temperature is not None else 1.0
        if t <= 0:
            out[b] = torch.log_softmax(z[b], -1)
            continue
        zb = z[b] / t
        k = int(top_k[b]) if top_k is not None else 0
        if 0 < k < V:
            kth = torch.topk(zb, k).values[-1]
            zb = zb.masked_fill(zb < kth, float("-inf"))
        p = float(top_p[b]) if top_p is not None else 1.0
        if p < 1.0:
            probs = torch.softmax(zb, -1)
            sp, si = probs.sort(descending=True)
            keep_sorted = (sp.cumsum(0) - sp) < p
            thr = sp[keep_sorted].min()
            zb = zb.masked_fill(probs < thr, float("-inf"))
        out[b] = torch.log_softmax(zb, -1)
    return out


def sample(logits, temperature=None, top_k=None, top_p=None, seed: int = 0, counters=None,
           logprobs_mode: str = "processed"):
    """Returns (tokens int32 [B], logprobs fp32 [B]). ``logprobs_mode``: ``"processed"`` reports the log-prob
    under the processed distribution (after temperature / top-k / top-p, renormalised over the kept set - the
    reference's vLLM fork, install/vllm/axon.patch:635-680); ``"full"`` reports the temperature-scaled
    log-softmax over the whole vocabulary, which is what the trainer's ``old_log_probs`` hold, so that
    importance-sampling corrections stay unbiased when top-k / top-p truncate the draw."""
    assert logprobs_mode in ("processed", "full")
    B, V = logits.shape
    if not C.use_native(logits):
        lp = _ref_process(logits, temperature, top_k, top_p)
        toks = torch.empty(B, dtype=torch.int32)
        for b in range(B):
            t = float(temperature[b]) if temperature is not None else 1.0
            if t <= 0:
                toks[b] = int(lp[b].argmax())
            else:
                # with counters the draw depends on (seed, counter) only, not on the row the sequence occupies
                g = torch.Generator().manual_seed((seed * 1000003 + (int(counters[b]) if counters is not None else b * 7919)) % (2 ** 63))
                toks[b] = int(torch.multinomial(lp[b].exp(), 1, generator=g))
        if logprobs_mode == "full":
            lp = _ref_process(logits, temperature, None, None)
        return toks, lp.gather(1, toks.long()[:, None])[:, 0]
    toks = torch.empty(B, dtype=torch.int32, device=logits.device)
    lps = torch.empty(B, dtype=torch.float32, device=logits.device)
    rc = C.lib().axb_sample_ex(C.ptr(logits), ctypes.c_longlong(logits.stride(0)), B, V, C.ptr(temperature),
                               C.ptr(top_k), C.ptr(top_p), ctypes.c_ulonglong(seed & (2 ** 64 - 1)), C.ptr(counters),
                               C.ptr(toks), C.ptr(lps), 1 if logprobs_mode == "full" else 0, C.stream())
    C.launched(rc, "sample")
    return toks, lps


def repetition_penalty_(logits, seen, penalty):
    """In place: logits of already-seen tokens are divided (if > 0) or multiplied (if < 0) by the penalty."""
    B, V = logits.shape
    if not C.use_native(logits):
        pen = penalty[:, None]
        adj = torch.where(logits > 0, logits / pen, logits * pen)
        logits.copy_(torch.where(seen.bool(), adj, logits))
        return logits
    rc = C.lib().axb_repetition_penalty(C.ptr(logits), ctypes.c_longlong(logits.stride(0)), B, V, C.ptr(seen),
                                        C.ptr(penalty), C.stream())
    C.launched(rc, "repetition_penalty")
    return logits
