"""Named single-kernel workloads for timing and for ``ncu`` captures.

    python -m axon_b200.utils.profiler.kernel_cases <case> [--iters N] [--small]

Each case builds inputs larger than L2 where the kernel is memory-bound, runs warm-up iterations,
times ``iters`` launches with CUDA events (L2 is flushed between timed launches by writing a 256 MB
buffer) and prints one JSON line with the achieved rate and its fraction of the peaks. The peaks come
from ``--peak-gbs`` / ``--peak-tflops``, else from the environment (``AXON_PEAK_GBS``, ``AXON_PEAK_TFLOPS``,
or ``AXON_PEAKS_JSON`` naming a file with ``hbm_gbs`` / ``bf16_tflops``), else 6650 GB/s and 1590 TFLOP/s.
``--small`` shrinks the case so that a full-metric ``ncu`` capture of a few launches ends quickly.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

PEAK_GBS, PEAK_TFLOPS = 6650.0, 1590.0


_PEAK_OVERRIDE: dict = {}


def _peaks():
    """(copy GB/s, bf16 TFLOP/s, where the numbers came from)."""
    if _PEAK_OVERRIDE:
        return _PEAK_OVERRIDE.get("gbs", PEAK_GBS), _PEAK_OVERRIDE.get("tflops", PEAK_TFLOPS), "measured"
    if os.environ.get("AXON_PEAK_GBS") or os.environ.get("AXON_PEAK_TFLOPS"):
        return float(os.environ.get("AXON_PEAK_GBS", PEAK_GBS)), float(os.environ.get("AXON_PEAK_TFLOPS", PEAK_TFLOPS)), "measured"
    p = os.environ.get("AXON_PEAKS_JSON")
    if p and os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d.get("hbm_gbs", PEAK_GBS)), float(d.get("bf16_tflops", PEAK_TFLOPS)), "measured"
    return PEAK_GBS, PEAK_TFLOPS, "fallback"


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def case_gemm_train(small):
    from ...ops import gemm as G
    M, N, K = (2048, 6144, 4096) if small else (8192, 6144, 4096)
    a, b = bf(M, K), bf(N, K)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    return (lambda: G.gemm_nt(a, b, out=out)), dict(flops=2.0 * M * N * K, bytes=2.0 * (M * K + N * K + M * N), shape=[M, N, K])


def case_gemm_wgrad(small):
    from ...ops import gemm as G
    T, N, K = (2048, 4096, 4096) if small else (8192, 12288, 4096)
    dy, x = bf(T, N), bf(T, K)
    out = torch.zeros(N, K, device="cuda", dtype=torch.float32)
    return (lambda: G.gemm_tn(dy, x, out=out, accumulate=True)), dict(flops=2.0 * T * N * K, bytes=2.0 * T * (N + K) + 8.0 * N * K, shape=[T, N, K])


def case_gemm_decode(small):
    from ...ops import gemm as G
    M, N, K = 256, 6144, 4096
    a = bf(M, K)
    ws = [bf(N, K) for _ in range(2 if small else 8)]       # rotate weights: 8 x 50 MB exceeds L2
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    st = {"i": 0}

    def run():
        st["i"] = (st["i"] + 1) % len(ws)
        G.gemm_nt(a, ws[st["i"]], out=out)
    return run, dict(flops=2.0 * M * N * K, bytes=2.0 * (M * K + N * K + M * N), shape=[M, N, K])


def case_gemm_stream(small):
    """Weight-streaming decode GEMM (64 tokens x 6144 features x K 4096), weights rotated so that they come from HBM."""
    from ...ops import gemm as G
    M, N, K = 64, 6144, 4096
    a = bf(M, K)
    ws = [bf(N, K) for _ in range(3 if small else 8)]
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    st = {"i": 0}

    def run():
        st["i"] = (st["i"] + 1) % len(ws)
        G.gemm_nt(a, ws[st["i"]], out=out)
    return run, dict(flops=2.0 * M * N * K, bytes=2.0 * (M * K + N * K + M * N), shape=[M, N, K])


def case_gemm_decode_chain(small):
    """The four projections of a Qwen3-8B layer at decode batch 64, 8 layers' worth of distinct weights (3 GB, so L2
    is cold for weights by construction), replayed as one CUDA graph: the per-launch figure is per LAYER
    (qkv + o + gate_up + down = 385 MB of weights); launch gaps and dependent-launch overlap are included."""
    from ...ops import gemm as G
    L, M = (2, 64) if small else (8, 64)
    shapes = [(6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288)]
    Ws = [[bf(n, k, scale=0.02) for (n, k) in shapes] for _ in range(L)]
    xs = [bf(M, k) for (_, k) in shapes]
    outs = [torch.empty(M, n, device="cuda", dtype=torch.bfloat16) for (n, _) in shapes]

    def body():
        for l in range(L):
            for i in range(4):
                G.gemm_nt(xs[i], Ws[l][i], out=outs[i])
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        body()
        body()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        body()
    byts = sum(2.0 * n * k for n, k in shapes)
    return (lambda: graph.replay()), dict(flops=2.0 * M * sum(n * k for n, k in shapes) * L, bytes=byts * L, shape=[M, L, "layers"])


def case_train_microbatch(small):
    """One training micro-batch (forward + backward) of the dense model: Qwen3-8B on 8192 packed tokens (``--small``:
    the tiny GPU preset on 1024 tokens), random weights, activations kept (recompute "none")."""
    from ...models.config import get_config
    from ...models.dense import DenseModel, PackedBatch
    cfg = get_config("tiny-gpu" if small else "qwen3-8b")
    model = DenseModel(cfg, device="cuda")
    model.params.init_random(seed=0)
    model.recompute = "none"
    model.params.alloc_grads()
    g = torch.Generator().manual_seed(0)
    lens = (320, 256, 288, 160) if small else (2560, 2048, 2304, 1280)
    batch = PackedBatch.from_sequences([torch.randint(0, cfg.vocab_size, (n,), generator=g, dtype=torch.int32) for n in lens], "cuda")
    T = batch.input_ids.numel()

    def run():
        lp, _ = model.forward(batch, 1.0, save_for_backward=True)
        model.backward(torch.ones_like(lp) / T, None)
    return run, dict(flops=model.flops_per_token(max(lens)) * T, bytes=0.0, shape=[T, cfg.num_hidden_layers, "layers"])


def _qkv(lens, Hq, Hkv, D=128):
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    return bf(T, (Hq + 2 * Hkv) * D, scale=0.5), cu, T


def _attn_flops(lens, Hq, D=128):
    return sum(4.0 * L * L / 2 * Hq * D for L in lens)


def case_attn_fwd(small):
    from ...ops import attention as AT
    lens = [1024] * 2 if small else [2731, 2731, 2730]
    qkv, cu, T = _qkv(lens, 32, 8)
    return (lambda: AT.attn_fwd(qkv, cu, 32, 8, 128)), dict(flops=_attn_flops(lens, 32), bytes=2.0 * T * (48 + 32) * 128, shape=lens)


def case_attn_bwd(small):
    from ...ops import attention as AT
    lens = [1024] * 2 if small else [2731, 2731, 2730]
    qkv, cu, T = _qkv(lens, 32, 8)
    o, lse = AT.attn_fwd(qkv, cu, 32, 8, 128)
    do = bf(T, 32 * 128)
    return (lambda: AT.attn_bwd(do, qkv, o, lse, cu, 32, 8, 128)), dict(flops=3.5 * _attn_flops(lens, 32), bytes=2.0 * T * (48 * 2 + 64) * 128, shape=lens)


def case_paged_decode(small):
    from ...ops import paged as P
    B, ctx, Hq, Hkv, D = (32, 1024, 32, 8, 128) if small else (256, 1536, 32, 8, 128)
    pages_per = (ctx + 127) // 128
    n_pages = B * pages_per
    kc, vc = bf(n_pages, Hkv, 128, D, scale=0.3), bf(n_pages, Hkv, 128, D, scale=0.3)
    bt = torch.randperm(n_pages, device="cuda").to(torch.int32).view(B, pages_per)
    lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    q = bf(B, (Hq + 2 * Hkv) * D, scale=0.3)
    return (lambda: P.paged_decode(q, kc, vc, bt, lens, Hq, Hkv, D)), dict(flops=4.0 * B * ctx * Hq * D, bytes=4.0 * B * ctx * Hkv * D, shape=[B, ctx])


def _grpo_decode_batch(small):
    """B sequences = groups of 8 samples sharing a 1024-token prompt (8 pages), each with a private tail."""
    B, shared, tail, Hq, Hkv, D = (64, 8, 300, 32, 8, 128) if small else (256, 8, 500, 32, 8, 128)
    tail_pages = (tail + 127) // 128
    n_groups = B // 8
    n_pages = n_groups * shared + B * tail_pages
    kc, vc = bf(n_pages, Hkv, 128, D, scale=0.3), bf(n_pages, Hkv, 128, D, scale=0.3)
    perm = torch.randperm(n_pages).to(torch.int32)
    bt = torch.full((B, shared + tail_pages + 1), -1, dtype=torch.int32)
    for b in range(B):
        g = b // 8
        bt[b, :shared] = perm[g * shared:(g + 1) * shared]
        o = n_groups * shared + b * tail_pages
        bt[b, shared:shared + tail_pages] = perm[o:o + tail_pages]
    lens = torch.full((B,), shared * 128 + tail, dtype=torch.int32, device="cuda")
    q = bf(B, (Hq + 2 * Hkv) * D, scale=0.3)
    return B, shared, tail, Hq, Hkv, D, kc, vc, bt.cuda(), lens, q


def case_paged_decode_grpo_plain(small):
    """The plain decode kernel on a GRPO-shaped batch (every sample streams the shared prompt pages itself)."""
    from ...ops import paged as P
    B, shared, tail, Hq, Hkv, D, kc, vc, bt, lens, q = _grpo_decode_batch(small)
    ctx = shared * 128 + tail
    return (lambda: P.paged_decode(q, kc, vc, bt, lens, Hq, Hkv, D)), dict(flops=4.0 * B * ctx * Hq * D, bytes=4.0 * B * ctx * Hkv * D, shape=[B, ctx])


def case_paged_decode_grpo_shared(small):
    """Shared-prefix decode attention on the same batch: prompt pages once per group of 8, tails per sequence."""
    from ...ops import paged as P
    B, shared, tail, Hq, Hkv, D, kc, vc, bt, lens, q = _grpo_decode_batch(small)
    ng = B // 2
    zi = lambda n: torch.zeros(n, dtype=torch.int32, device="cuda")      # noqa: E731
    sh = dict(seq_first=torch.arange(B, dtype=torch.int32, device="cuda"), seq_one=torch.ones(B, dtype=torch.int32, device="cuda"),
              seq_page0=torch.full((B,), shared, dtype=torch.int32, device="cuda"), seq_keys=torch.full((B,), tail, dtype=torch.int32, device="cuda"),
              grp_first=zi(ng), grp_size=zi(ng), grp_zero=zi(ng), grp_keys=zi(ng), max_shared_pages=shared)
    sh["grp_first"][: B // 8] = torch.arange(0, B, 8, dtype=torch.int32, device="cuda")
    sh["grp_size"][: B // 8] = 8
    sh["grp_keys"][: B // 8] = shared * 128
    ctx = shared * 128 + tail
    unique = (B // 8) * shared * 128 + B * tail          # keys that have to be read at least once
    return (lambda: P.paged_decode_shared(q, kc, vc, bt, lens, sh, Hq, Hkv, D)), dict(flops=4.0 * B * ctx * Hq * D, bytes=4.0 * unique * Hkv * D, shape=[B, ctx])


def case_lmhead_fwd(small):
    from ...ops import lm_head as L
    T, H, V = (1024, 4096, 151936) if small else (8192, 4096, 151936)
    h, w = bf(T, H), bf(V, H, scale=0.02)
    lab = torch.randint(0, V, (T,), dtype=torch.int32, device="cuda")
    return (lambda: L.lmhead_fwd(h, w, lab, 1.0)), dict(flops=2.0 * T * H * V, bytes=2.0 * (T * H + V * H), shape=[T, H, V])


def case_rmsnorm(small):
    from ...ops import norm as N
    T, H = (16384, 4096) if small else (65536, 4096)
    x, d, w = bf(T, H), bf(T, H), bf(H)
    return (lambda: N.rmsnorm_fwd(x, w, 1e-6, delta=d)), dict(flops=0.0, bytes=2.0 * T * H * 4, shape=[T, H])


def case_adamw(small):
    from ...ops import optim as O
    n = (1 << 26) if small else (1 << 28)
    master, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    p = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    return (lambda: O.adamw_step(master, p, g, m, v, 1e-5, 0.9, 0.95, 1e-8, 0.1, 3)), dict(flops=0.0, bytes=n * (4 * 7 + 2.0), shape=[n])


def case_gemm_ag(small):
    """All-gather -> GEMM kernel with both "ranks" on this GPU (two local shards stand in for the peers):
    same kernel, same TMA traffic pattern, no NVLink."""
    import ctypes
    from ...ops import _common as C
    rows, N, K, W = (1024, 6144, 4096, 2) if small else (4096, 6144, 4096, 2)
    shards = [bf(rows, K) for _ in range(W)]
    w = bf(N, K)
    out = torch.empty(W * rows, N, device="cuda", dtype=torch.bfloat16)
    ptrs = (ctypes.c_ulonglong * W)(*[t.data_ptr() for t in shards])
    lib = C.lib()

    def run():
        rc = lib.axb_gemm_allgather_a(ptrs, W, 0, C.ptr(w), C.ptr(out), rows, N, K, ctypes.c_longlong(K), ctypes.c_longlong(K),
                                      ctypes.c_longlong(N), 0, 0, C.ptr(C.status(w.device)), C.stream())
        C.launched(rc, "gemm_allgather_a")
    T = W * rows
    return run, dict(flops=2.0 * T * N * K, bytes=2.0 * (T * K + N * K + T * N), shape=[T, N, K])


def case_gemm_gather_w(small):
    """Weight all-gather -> GEMM (sharded parameters) with both weight shards on this GPU: same kernel and TMA
    traffic pattern as across NVLink."""
    import ctypes
    from ...ops import _common as C
    T, F, K, W = (2048, 6144, 4096, 2) if small else (8192, 6144, 4096, 2)
    shards = [bf(F // W, K) for _ in range(W)]
    x = bf(T, K)
    out = torch.empty(T, F, device="cuda", dtype=torch.bfloat16)
    ptrs = (ctypes.c_ulonglong * W)(*[t.data_ptr() for t in shards])
    lib = C.lib()

    def run():
        rc = lib.axb_gemm_gather_weights(ptrs, W, 0, C.ptr(x), C.ptr(out), F // W, T, K, ctypes.c_longlong(K), ctypes.c_longlong(K),
                                         ctypes.c_longlong(F), 0, C.ptr(C.status(x.device)), C.stream())
        C.launched(rc, "gemm_gather_weights")
    return run, dict(flops=2.0 * T * F * K, bytes=2.0 * (T * K + F * K + T * F), shape=[T, F, K])


def case_gemm_rs(small):
    """GEMM -> reduce-scatter (scatter part) with both staging areas on this GPU."""
    import ctypes
    from ...ops import _common as C
    T, N, K, W = (2048, 4096, 2048, 2) if small else (8192, 4096, 2048, 2)
    x, w = bf(T, K), bf(N, K)
    stage = [torch.empty(W * (T // W) * N, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    ptrs = (ctypes.c_ulonglong * W)(*[t.data_ptr() for t in stage])
    out = torch.empty(T // W, N, device="cuda", dtype=torch.bfloat16)
    lib = C.lib()

    def run():
        rc = lib.axb_gemm_scatter(C.ptr(x), C.ptr(w), ptrs, W, 0, T, N, K, ctypes.c_longlong(K), ctypes.c_longlong(K),
                                  ctypes.c_longlong(N), 0, C.ptr(C.status(w.device)), C.stream())
        C.launched(rc, "gemm_scatter")
        rc = lib.axb_rs_reduce(C.ptr(stage[0]), None, C.ptr(out), W, ctypes.c_longlong(T // W), N, ctypes.c_longlong(N),
                               ctypes.c_longlong(N), C.stream())
        C.launched(rc, "rs_reduce")
    return run, dict(flops=2.0 * T * N * K, bytes=2.0 * (T * K + N * K + T * N), shape=[T, N, K])


def case_indexer_fwd(small):
    """Lightning indexer logits: 32 heads x 128 dims, S queries against Skv keys (one GEMM with the head sum
    in the epilogue). Bytes: q, k once, fp32 logits written once."""
    from ...ops import dsa
    S, Skv, Hi, D = (1024, 4096, 32, 128) if small else (4096, 8192, 32, 128)
    q, k = bf(S, Hi, D, scale=0.3), bf(Skv, D, scale=0.3)
    w = torch.randn(S, Hi, device="cuda")
    ks = torch.zeros(S, dtype=torch.int32, device="cuda")
    ke = torch.full((S,), Skv, dtype=torch.int32, device="cuda")

    def run():
        dsa.indexer_logits(q, k, w, ks, ke)
    return run, dict(flops=2.0 * S * Hi * Skv * D, bytes=2.0 * (S * Hi * D + Skv * D) + 4.0 * S * Skv, shape=[S, Hi, Skv, D])


def case_indexer_bwd(small):
    """Lightning indexer backward at 2048 selected keys per query (one block per query, warp per key)."""
    from ...ops import dsa
    S, Skv, Hi, D, topk = (512, 4096, 32, 128, 2048) if small else (2048, 8192, 32, 128, 2048)
    q, k = bf(S, Hi, D, scale=0.3), bf(Skv, D, scale=0.3)
    w = torch.randn(S, Hi, device="cuda")
    idx = torch.stack([torch.randperm(Skv, device="cuda")[:topk] for _ in range(S)]).int()
    g = torch.randn(S, topk, device="cuda")

    def run():
        dsa.indexer_bwd(g, idx, q, k, w)
    return run, dict(flops=6.0 * S * topk * Hi * D, bytes=2.0 * S * topk * D + 4.0 * S * topk * D, shape=[S, Hi, topk, D])


def case_sparse_mla_fwd(small):
    """Sparse latent attention forward, dense-masked on the GEMM kernels: 64 heads, 576-dim rows, top-2048 of Skv
    keys. FLOPs counted for the selected keys only (what a gathering kernel would spend)."""
    from ...ops import dsa
    S, Skv, H, Dk, d_v, topk = (512, 4096, 64, 576, 512, 2048) if small else (2048, 8192, 64, 576, 512, 2048)
    q, kv = bf(S, H, Dk, scale=0.2), bf(Skv, Dk, scale=0.2)
    idx = torch.stack([torch.randperm(Skv, device="cuda")[:topk] for _ in range(S)]).int()

    def run():
        dsa.sparse_mla_fwd(q, kv, idx, Dk ** -0.5, d_v)
    return run, dict(flops=2.0 * S * H * topk * (Dk + d_v), bytes=2.0 * (S * H * (Dk + d_v) + Skv * Dk), shape=[S, H, Skv, topk])


def case_zero1_reduce(small):
    """Gradient reduce of the fused ZeRO-1 step with both "ranks" on this GPU: this rank's shard of every rank's fp32
    gradient buffer is read once and summed (plus the sum of squares for the clipping norm)."""
    import ctypes
    from ...ops import _common as C
    W = 2
    n = (16 << 20) if small else (128 << 20)                  # elements of this rank's shard
    grads = [torch.randn(W * n, device="cuda") for _ in range(W)]
    ptrs = (ctypes.c_ulonglong * W)(*[g.data_ptr() for g in grads])
    lib = C.lib()
    reduced = torch.empty(n, device="cuda")
    partials = torch.zeros(lib.axb_zero1_partials(), device="cuda")

    def run():
        rc = lib.axb_zero1_reduce(ptrs, 0, W, ctypes.c_longlong(0), ctypes.c_longlong(n), C.ptr(reduced), C.ptr(partials), C.stream())
        C.launched(rc, "zero1_reduce")
    return run, dict(flops=float(W * n), bytes=4.0 * n * (W + 1), shape=[W, n])


def case_zero1_adamw_bcast(small):
    """AdamW on this rank's shard whose epilogue stores the new bf16 values into every rank's parameter buffer
    (both "ranks" on this GPU): fp32 master / m / v read and written, gradient read, W bf16 copies written."""
    import ctypes
    from ...ops import _common as C
    W = 2
    n = (16 << 20) if small else (128 << 20)
    master, g, m, v = (torch.randn(n, device="cuda") * 0.01 for _ in range(4))
    v = v.abs()
    params = [torch.empty(W * n, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    ptrs = (ctypes.c_ulonglong * W)(*[t.data_ptr() for t in params])
    state = torch.tensor([1.0, 1.0, 1.0, 0.0], device="cuda")       # [sumsq, norm, clip coefficient, skip]
    lib = C.lib()
    f = ctypes.c_float

    def run():
        rc = lib.axb_zero1_adamw_bcast(C.ptr(master), C.ptr(g), C.ptr(m), C.ptr(v), ptrs, W, ctypes.c_longlong(0), ctypes.c_longlong(n),
                                       f(1e-5), f(0.9), f(0.95), f(1e-8), f(0.01), f(0.1), f(0.05), C.ptr(state), C.stream())
        C.launched(rc, "zero1_adamw_bcast")
    return run, dict(flops=12.0 * n, bytes=n * (4.0 * 7 + 2.0 * W), shape=[W, n])


def _sync_plan(small, quant):
    from ...utils.p2p.plan import copy_desc, plan_from_descs
    R, Cc, L, W = (4096, 4096, 8, 2) if small else (4096, 4096, 48, 2)          # L matrices, split by rows over W destinations
    src = bf(L * R * Cc, scale=0.05)
    rows = []
    per = R // W
    for l in range(L):
        for d in range(W):
            desc = copy_desc((l * R + d * per) * Cc, l * per * Cc, per, Cc, Cc, Cc, d)
            if quant:
                desc["quant"], desc["scale_cols"] = 1, Cc // 128
                desc["dst_scale_off"] = l * (per // 128) * (Cc // 128)
            rows.append(desc)
    return src, plan_from_descs(rows), L * per * Cc, L * (per // 128) * (Cc // 128), W, L * R * Cc


def case_p2p_copy_plan(small):
    """Weight-sync plan kernel, bf16 copies: one launch moves every routed slice (row shards of L matrices to two
    destinations, both on this GPU)."""
    from ...utils.p2p.plan import execute_plan
    src, plan, dst_n, _, W, total = _sync_plan(small, False)
    dst = [torch.empty(dst_n, device="cuda", dtype=torch.bfloat16) for _ in range(W)]

    def run():
        execute_plan(plan, src, dst)
    return run, dict(flops=0.0, bytes=4.0 * total, shape=[total])


def case_p2p_quant_plan(small):
    """Weight-sync plan kernel with the bf16 -> fp8 (128 x 128 block scales) quantisation fused into the copy."""
    from ...utils.p2p.plan import execute_plan
    src, plan, dst_n, sc_n, W, total = _sync_plan(small, True)
    dst = [torch.empty(dst_n, device="cuda", dtype=torch.uint8) for _ in range(W)]
    scales = [torch.empty(sc_n, device="cuda") for _ in range(W)]

    def run():
        execute_plan(plan, src, dst, scale_flats=scales)
    return run, dict(flops=0.0, bytes=3.0 * total, shape=[total])


def case_moe_grouped(small):
    from ...ops import moe as M
    T, E, k, H, F = (2048, 128, 8, 2048, 768) if small else (8192, 128, 8, 2048, 768)
    logits = torch.randn(T, E, device="cuda")
    x = bf(T, H)
    w13 = bf(E, 2 * F, H, scale=0.05)
    ids, w = M.route(logits, k)
    lay = M.align(ids, E)
    xs = M.gather(x, lay)
    return (lambda: M.grouped_fwd(xs, w13, lay)), dict(flops=2.0 * T * k * 2 * F * H, bytes=2.0 * (T * k * H + E * 2 * F * H + T * k * 2 * F),
                                                     shape=[T * k, 2 * F, H, E])


CASES = {"zero1_reduce": case_zero1_reduce, "zero1_adamw_bcast": case_zero1_adamw_bcast, "p2p_copy_plan": case_p2p_copy_plan, "p2p_quant_plan": case_p2p_quant_plan, "indexer_fwd": case_indexer_fwd, "indexer_bwd": case_indexer_bwd, "sparse_mla_fwd": case_sparse_mla_fwd, "gemm_train": case_gemm_train, "gemm_wgrad": case_gemm_wgrad, "gemm_decode": case_gemm_decode, "gemm_stream": case_gemm_stream,
         "gemm_decode_chain": case_gemm_decode_chain, "train_microbatch": case_train_microbatch,
         "attn_fwd": case_attn_fwd, "attn_bwd": case_attn_bwd, "paged_decode": case_paged_decode, "paged_decode_grpo_plain": case_paged_decode_grpo_plain,
         "paged_decode_grpo_shared": case_paged_decode_grpo_shared,
         "lmhead_fwd": case_lmhead_fwd, "rmsnorm": case_rmsnorm, "adamw": case_adamw, "gemm_ag": case_gemm_ag, "gemm_gather_w": case_gemm_gather_w,
         "gemm_rs": case_gemm_rs, "moe_grouped": case_moe_grouped}


_NOT_IN_ALL = {"train_microbatch"}      # whole-model cases (tens of GB): run by name


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=sorted(CASES) + ["all"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--peak-gbs", type=float, default=None, help="measured copy bandwidth to report fractions against")
    ap.add_argument("--peak-tflops", type=float, default=None, help="measured bf16 GEMM rate to report fractions against")
    args = ap.parse_args()
    if args.peak_gbs:
        _PEAK_OVERRIDE["gbs"] = args.peak_gbs
    if args.peak_tflops:
        _PEAK_OVERRIDE["tflops"] = args.peak_tflops
    from ...ops import _common as C
    gbs, tfl, src = _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for name in ([n for n in sorted(CASES) if n not in _NOT_IN_ALL] if args.case == "all" else [args.case]):
        fn, info = CASES[name](args.small)
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        ms = []
        for _ in range(args.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
        C.check_status()
        t = sorted(ms)[len(ms) // 2] * 1e-3
        out = {"case": name, "shape": info["shape"], "ms": t * 1e3, "tflops": info["flops"] / t / 1e12,
               "gbs": info["bytes"] / t / 1e9, "frac_of_" + src + "_tflops": info["flops"] / t / 1e12 / tfl,
               "frac_of_" + src + "_hbm": info["bytes"] / t / 1e9 / gbs, "l2": "flushed between timed launches"}
        print(json.dumps(out))
        del fn
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
