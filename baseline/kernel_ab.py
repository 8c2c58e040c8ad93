"""Kernel-level A/B on one GPU: this repository's kernels against the libraries of the image and against the
reference's own kernels, on identical inputs and shapes.

    python -m baseline.kernel_ab [case ...] [--iters N] [--warmup W] [--out FILE]

Every case builds its inputs once, checks that the two sides agree numerically (the comparison is void if they
compute different things), times each side with CUDA events after warm-up with a 256 MB write between timed
launches (L2 flushed) and prints one JSON line:

    {"case": ..., "shape": ..., "ours_ms": a, "other": "<library or reference kernel>", "other_ms": b,
     "speedup": b / a, "max_abs_diff": d}

Sides. ``other`` is one of
  * a library of the image called the way the reference calls it: ``torch.matmul`` (cuBLAS),
    ``flash_attn_varlen_func`` (flash-attn 2.8), FlashInfer's paged decode (the wrapper the reference's sampler
    back end plans per batch, and the TRT-LLM generated kernels where their cubins are present);
  * a kernel file of the reference, loaded UNMODIFIED by path from ``baseline/_ref``: the Triton log-prob/entropy
    head (axon/utils/kernel/linear_cross_entropy.py, kernels.py), the Triton fused experts
    (axon/utils/kernel/fused_experts.py:352) and the Triton 128x128 fp8 cast (axon/utils/sglang/fp8.py:60-114).
A side that cannot be built or run here is reported as ``{"case": ..., "other_unavailable": "<why>"}`` with this
repository's time alone; nothing is skipped silently.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")


def _ref_module(name: str):
    """Import ``axon.<...>`` from the untouched install without running the package ``__init__`` files."""
    for pkg, rel in (("axon", "axon"), ("axon.utils", "axon/utils"), ("axon.utils.kernel", "axon/utils/kernel"),
                     ("axon.utils.sglang", "axon/utils/sglang")):
        if pkg not in sys.modules:
            m = types.ModuleType(pkg)
            m.__path__ = [os.path.join(REF_ROOT, rel)]
            sys.modules[pkg] = m
    return importlib.import_module(name)


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


_FLUSH = None


def timed(fn, iters: int, warmup: int) -> float:
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        _FLUSH.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def _diff(x, y) -> float:
    return float((x.float() - y.float()).abs().max())


# ----------------------------------------------------------------------------------------------- cases
# Each returns (shape, ours_fn, other_name, other_fn_or_exception, check) where check() -> max abs difference.

def case_gemm_train():
    from axon_b200.ops import gemm as G
    M, N, K = 8192, 6144, 4096
    a, w = bf(M, K), bf(N, K, scale=0.05)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    out2 = torch.empty_like(out)
    ours = lambda: G.gemm_nt(a, w, out=out)
    other = lambda: torch.matmul(a, w.t(), out=out2)
    return [M, N, K], ours, "torch.matmul (cuBLAS bf16)", other, lambda: _diff(ours(), other())


def case_gemm_wgrad():
    from axon_b200.ops import gemm as G
    T, N, K = 8192, 12288, 4096
    dy, x = bf(T, N, scale=0.05), bf(T, K)
    out = torch.zeros(N, K, device="cuda", dtype=torch.float32)
    ours = lambda: G.gemm_tn(dy, x, out=out, accumulate=False)
    other = lambda: torch.matmul(dy.t(), x)                 # bf16 result, as autograd of nn.Linear produces it
    return [T, N, K], ours, "torch.matmul (cuBLAS bf16, transposed A)", other, lambda: _diff(ours(), other())


def _attn_inputs():
    lens = [2731, 2731, 2730]
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    qkv = bf(T, 48 * 128, scale=0.5)
    return lens, T, cu, qkv


def case_attn_fwd():
    from axon_b200.ops import attention as AT
    from flash_attn import flash_attn_varlen_func
    lens, T, cu, qkv = _attn_inputs()
    x = qkv.view(T, 48, 128)
    q, k, v = x[:, :32], x[:, 32:40], x[:, 40:]
    ours = lambda: AT.attn_fwd(qkv, cu, 32, 8, 128)[0]
    other = lambda: flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True)
    return lens, ours, "flash_attn_varlen_func 2.8 (mma.sync path on this GPU)", other, \
        lambda: _diff(ours().view(T, 32, 128), other())


def case_attn_bwd():
    from axon_b200.ops import attention as AT
    from flash_attn import flash_attn_varlen_func
    lens, T, cu, qkv = _attn_inputs()
    o, lse = AT.attn_fwd(qkv, cu, 32, 8, 128)
    do = bf(T, 32 * 128)
    x = qkv.view(T, 48, 128)
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (x[:, :32], x[:, 32:40], x[:, 40:]))
    o2 = flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True)
    do2 = do.view(T, 32, 128)
    ours = lambda: AT.attn_bwd(do, qkv, o, lse, cu, 32, 8, 128)

    def other():
        return torch.autograd.grad(o2, (q, k, v), do2, retain_graph=True)

    def check():
        dqkv = ours().view(T, 48, 128)
        dq, dk, dv = other()
        return max(_diff(dqkv[:, :32], dq), _diff(dqkv[:, 32:40], dk), _diff(dqkv[:, 40:], dv))
    return lens, ours, "flash-attn 2.8 backward (autograd of flash_attn_varlen_func)", other, check


def _decode_inputs():
    B, ctx, Hq, Hkv, D = 256, 1536, 32, 8, 128
    pages_per = (ctx + 127) // 128
    n_pages = B * pages_per
    kc, vc = bf(n_pages, Hkv, 128, D, scale=0.3), bf(n_pages, Hkv, 128, D, scale=0.3)
    bt = torch.randperm(n_pages, device="cuda").to(torch.int32).view(B, pages_per)
    lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    q = bf(B, (Hq + 2 * Hkv) * D, scale=0.3)
    return B, ctx, Hq, Hkv, D, pages_per, kc, vc, bt, lens, q


def case_paged_decode_flashinfer():
    import flashinfer
    from axon_b200.ops import paged as P
    B, ctx, Hq, Hkv, D, pages_per, kc, vc, bt, lens, q = _decode_inputs()
    ours = lambda: P.paged_decode(q, kc, vc, bt, lens, Hq, Hkv, D)
    ws = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    wrap = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "HND", use_tensor_cores=True)
    indptr = torch.arange(0, B + 1, dtype=torch.int32, device="cuda") * pages_per
    last = torch.full((B,), ctx - (pages_per - 1) * 128, dtype=torch.int32, device="cuda")
    wrap.plan(indptr, bt.reshape(-1).contiguous(), last, Hq, Hkv, D, 128, q_data_type=torch.bfloat16, kv_data_type=torch.bfloat16)
    qh = q.view(B, Hq + 2 * Hkv, D)[:, :Hq].contiguous()
    other = lambda: wrap.run(qh, (kc, vc))
    return [B, ctx], ours, "flashinfer BatchDecodeWithPagedKVCacheWrapper (tensor cores, page 128, planned once)", other, \
        lambda: _diff(ours().view(B, Hq, D), other())


def case_paged_decode_trtllm():
    from flashinfer.decode import trtllm_batch_decode_with_kv_cache
    from axon_b200.ops import paged as P
    B, ctx, Hq, Hkv, D, pages_per, kc, vc, bt, lens, q = _decode_inputs()
    ours = lambda: P.paged_decode(q, kc, vc, bt, lens, Hq, Hkv, D)
    ws = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")
    qh = q.view(B, Hq + 2 * Hkv, D)[:, :Hq].contiguous()
    scale = 1.0 / (D ** 0.5)
    other = lambda: trtllm_batch_decode_with_kv_cache(qh, (kc, vc), ws, bt, lens, ctx, bmm1_scale=scale, bmm2_scale=1.0,
                                                      kv_layout="HND")
    return [B, ctx], ours, "flashinfer trtllm_batch_decode_with_kv_cache (TRT-LLM generated sm_100 kernels)", other, \
        lambda: _diff(ours().view(B, Hq, D), other())


def case_lmhead():
    from axon_b200.ops import lm_head as L
    mod = _ref_module("axon.utils.kernel.linear_cross_entropy")
    T, H, V = 8192, 4096, 151936
    h, w = bf(T, H), bf(V, H, scale=0.02)
    lab = torch.randint(0, V, (T,), device="cuda")
    lab32 = lab.to(torch.int32)
    ours = lambda: L.lmhead_fwd(h, w, lab32, 1.0)
    other = lambda: mod.linear_cross_entropy(h, w, lab, 1.0, "none")

    def check():
        a, b = ours(), other()
        return max(_diff(a[0], b[0]), _diff(a[1], b[1]))          # log-probs, entropy
    return [T, H, V], ours, "reference Triton linear_cross_entropy forward (axon/utils/kernel/kernels.py)", other, check


def case_lmhead_fwd_bwd():
    from axon_b200.ops import lm_head as L
    mod = _ref_module("axon.utils.kernel.linear_cross_entropy")
    T, H, V = 8192, 4096, 151936
    w = bf(V, H, scale=0.02).requires_grad_(True)
    h = bf(T, H).requires_grad_(True)
    lab = torch.randint(0, V, (T,), device="cuda")
    lab32 = lab.to(torch.int32)
    g = torch.randn(T, device="cuda")
    ge = torch.full((T,), 0.01, device="cuda")        # a tensor, so that both incoming gradients are contiguous (the reference asserts it)

    def ours():
        lp, ent = L.linear_logprob_entropy(h, w, lab32, 1.0)
        return torch.autograd.grad((lp * g).sum() + (ent * ge).sum(), (h, w))

    def other():
        lp, ent = mod.linear_cross_entropy(h, w, lab, 1.0, "none")
        return torch.autograd.grad((lp * g).sum() + (ent * ge).sum(), (h, w))

    def check():
        a, b = ours(), other()
        return max(_diff(a[0], b[0]), _diff(a[1], b[1]))
    return [T, H, V], ours, "reference Triton linear_cross_entropy forward + backward", other, check


def case_moe_experts():
    from axon_b200.ops import moe as M
    from axon_b200.ops import activation as A
    fe = _ref_module("axon.utils.kernel.fused_experts")
    T, E, k, H, F = 8192, 128, 8, 2048, 768
    x = bf(T, H)
    w13, w2 = bf(E, 2 * F, H, scale=0.03), bf(E, H, F, scale=0.03)
    logits = torch.randn(T, E, device="cuda")
    ids, wts = M.route(logits, k)

    def ours():
        lay = M.align(ids, E)
        xs = M.gather(x, lay)
        hmid = A.swiglu_fwd(M.grouped_fwd(xs, w13, lay))
        return M.combine(M.grouped_fwd(hmid, w2, lay), wts, lay)
    other = lambda: fe.fused_experts_forward(x, w13, w2, wts.float(), ids.to(torch.int32))
    return [T * k, 2 * F, H, E], ours, "reference Triton fused_experts_forward (axon/utils/kernel/fused_experts.py:352)", other, \
        lambda: _diff(ours(), other())


def case_fp8_cast():
    from axon_b200.ops import quant as Q
    mod = _ref_module("axon.utils.sglang.fp8")
    w = bf(8 * 4096, 4096)
    ours = lambda: Q.fp8_block_quant(w)
    other = lambda: mod.blockwise_cast_to_fp8_triton(w)

    def check():
        (q1, s1), (q2, s2) = ours(), other()
        return max(_diff(q1.float() * s1.repeat_interleave(128, 0).repeat_interleave(128, 1),
                         q2.float() * s2.repeat_interleave(128, 0).repeat_interleave(128, 1)), _diff(s1, s2))
    return list(w.shape), ours, "reference Triton blockwise_cast_to_fp8_triton (axon/utils/sglang/fp8.py:60-114)", other, check


CASES = {"gemm_train": case_gemm_train, "gemm_wgrad": case_gemm_wgrad, "attn_fwd": case_attn_fwd, "attn_bwd": case_attn_bwd,
         "paged_decode_flashinfer": case_paged_decode_flashinfer, "paged_decode_trtllm": case_paged_decode_trtllm,
         "lmhead": case_lmhead, "lmhead_fwd_bwd": case_lmhead_fwd_bwd, "moe_experts": case_moe_experts, "fp8_cast": case_fp8_cast}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("cases", nargs="*", default=[])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    sys.path.insert(0, os.path.dirname(HERE))
    names = args.cases or list(CASES)
    lines = []
    for name in names:
        rec = {"case": name}
        ours = None
        try:
            shape, ours, other_name, other, check = CASES[name]()
            rec.update(shape=shape, other=other_name)
            rec["max_abs_diff"] = check()
            rec["ours_ms"] = timed(ours, args.iters, args.warmup)
            rec["other_ms"] = timed(other, args.iters, args.warmup)
            rec["speedup"] = rec["other_ms"] / rec["ours_ms"]
        except Exception as e:                                  # the other side (or its import) is what can fail here
            rec["other_unavailable"] = f"{type(e).__name__}: {e}"[:300]
            if ours is not None and "ours_ms" not in rec:
                try:
                    rec["ours_ms"] = timed(ours, args.iters, args.warmup)
                except Exception as e2:
                    rec["ours_error"] = f"{type(e2).__name__}: {e2}"[:300]
        print(json.dumps(rec), flush=True)
        lines.append(rec)
        torch.cuda.empty_cache()
    if args.out:
        with open(args.out, "w") as f:
            json.dump(lines, f, indent=1)


if __name__ == "__main__":
    main()
