"""Decoder families beyond the in-house dense / sparse Qwen-style models: DeepSeek-V3 (latent attention,
sigmoid group-limited routing, shared experts), GPT-OSS (attention sinks, alternating sliding windows, clamped
SwiGLU experts with biases), Gemma-2/3 (GeGLU, (1 + w) norms, sandwich norms, soft-capping, sliding windows),
GLM-4.5 / GLM-4.6 sparse models, and Qwen3-Next / Qwen3.5 (gated delta-rule linear attention mixed with gated
full attention). These are the families the reference reaches through its HF patches, Megatron model specs and
weight bridges (axon/models/mcore/models/{gemma4,gpt_oss,qwen3_next,qwen3_5,glm5}.py,
axon/models/mbridge/{deepseek_v3,gpt_oss,glm4_moe_lite,qwen3_next,qwen3_5}.py,
axon/monkey_patches/transformers/).

Design: one ``FamilyModel`` class holds the parameters in the same flat buffer (``FlatParams``) as every other
model here, under the checkpoint's own tensor names, and exposes the interface the policy engine and the
generation engine expect (``forward`` / ``backward`` over packed batches, ``prefill`` / ``decode`` over the
paged KV cache). The layer mathematics is written once per family as PyTorch functions over that buffer and
differentiated by autograd (per-layer recomputation with ``recompute = "full"``); dense projections run on the
tcgen05 GEMM on CUDA through ``NativeLinear``. The families share nothing hot with the flagship benchmark path:
they trade the hand-scheduled backward of ``DenseModel`` for breadth, and every one of them is checked
against the HF implementation of the same architecture on CPU (tests/test_families.py).
"""
from __future__ import annotations

import math
import re
from collections import OrderedDict

import torch
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .config import ModelConfig
from .params import FlatParams

FAMILY_TYPES = ("deepseek_v3", "glm4_moe", "glm4_moe_lite", "gpt_oss", "gemma2", "gemma3_text", "qwen3_next", "qwen3_5_text",
                "qwen3_5_moe_text", "glm_moe_dsa", "gemma4_text", "qwen2_vl", "qwen2_5_vl", "qwen3_vl", "qwen3_vl_moe", "glm4v")
VISION_LANGUAGE_TYPES = ("qwen2_vl", "qwen2_5_vl", "qwen3_vl", "qwen3_vl_moe", "glm4v")
# Multimodal checkpoints whose decoder is one of the text families above: they are trained text-only, as the reference does
# for Gemma-4 (axon/models/transformers/gemma4.py: ``patch_gemma4_for_text_only_training``) - the decoder's configuration
# and weights are taken, the towers are left alone.
TEXT_ONLY_OF = {"gemma3": "gemma3_text", "gemma4": "gemma4_text", "qwen3_5": "qwen3_5_text", "qwen3_5_moe": "qwen3_5_moe_text"}


# ------------------------------------------------------------------------------------------ small pieces
class NativeLinear(torch.autograd.Function):
    """y = x W^T on the tcgen05 GEMM (CUDA bf16 operands with 8-element aligned sizes); dgrad and wgrad likewise."""

    @staticmethod
    def forward(ctx, x, w):
        from ..ops import gemm as G
        ctx.save_for_backward(x, w)
        return G.gemm_nt(x, w)

    @staticmethod
    def backward(ctx, dy):
        from ..ops import gemm as G
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        return G.gemm_nn(dy, w), G.gemm_tn(dy, x, out_dtype=w.dtype)


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    """x [..., K] @ w[N, K]^T (+ b)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0:
        lead = x.shape[:-1]
        y = NativeLinear.apply(x.reshape(-1, x.shape[-1]).contiguous(), w).view(*lead, w.shape[0])
    else:
        y = F.linear(x, w)
    return y if b is None else y + b


def rms_norm(x, w, eps: float, plus_one: bool = False):
    """RMSNorm in fp32; ``plus_one``: the stored weight is an offset from 1 (Gemma, Qwen3-Next)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if w is not None:
        y = y * ((1.0 + w.float()) if plus_one else w.float())
    return y.to(x.dtype)


def rotate_half(x):
    a, b = x.chunk(2, dim=-1)
    return torch.cat((-b, a), dim=-1)


def apply_rope(x, cos, sin, interleaved: bool = False):
    """x [T, heads, D]; cos / sin [T, R] with R <= D: the first R dims turn (half-split pairs), the rest pass.
    ``interleaved``: the checkpoint pairs dims (2i, 2i + 1); they are regrouped to half-split order first."""
    R = cos.shape[-1]
    xr, xp = x[..., :R], x[..., R:]
    if interleaved:
        xr = xr.reshape(*xr.shape[:-1], R // 2, 2).transpose(-1, -2).reshape(*xr.shape[:-1], R)
    c, s = cos[:, None, :].to(x.dtype), sin[:, None, :].to(x.dtype)
    out = xr * c + rotate_half(xr) * s
    return torch.cat([out, xp], dim=-1) if xp.shape[-1] else out


def yarn_mscale(scale: float = 1.0, mscale: float = 1.0) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


def rope_frequencies(rope: dict, dim: int, max_pos_default: int) -> tuple[torch.Tensor, float]:
    """(inverse frequencies [dim / 2], factor applied to cos / sin) for the rope types ``default``, ``linear`` and
    ``yarn`` (the blend of interpolated and extrapolated frequencies with its attention temperature)."""
    theta = float(rope.get("rope_theta", 10000.0))
    kind = rope.get("rope_type", rope.get("type", "default")) or "default"
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
    if kind == "default":
        return inv.float(), 1.0
    factor = float(rope.get("factor", 1.0))
    if kind == "linear":
        return (inv / factor).float(), 1.0
    if kind == "yarn":
        orig = float(rope.get("original_max_position_embeddings") or max_pos_default)
        beta_fast, beta_slow = float(rope.get("beta_fast") or 32), float(rope.get("beta_slow") or 1)
        ms, ms_all = rope.get("mscale"), rope.get("mscale_all_dim")
        att = rope.get("attention_factor")
        if att is None:
            att = yarn_mscale(factor, ms) / yarn_mscale(factor, ms_all) if (ms and ms_all) else yarn_mscale(factor)

        def corr_dim(rot):
            return dim * math.log(orig / (rot * 2 * math.pi)) / (2 * math.log(theta))
        low, high = corr_dim(beta_fast), corr_dim(beta_slow)
        if rope.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(dim // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        extrap_weight = 1.0 - ramp
        inv_y = (inv / factor) * (1 - extrap_weight) + inv * extrap_weight
        return inv_y.float(), float(att)
    raise NotImplementedError(f"rope type '{kind}'")


def attention_packed(q, k, v, cu, scale: float, window: int | None = None, sinks: torch.Tensor | None = None,
                     softcap: float | None = None, allowed: list | None = None):
    """Causal attention over packed sequences. q [T, Hq, Dk], k [T, Hkv, Dk], v [T, Hkv, Dv]; ``cu`` = sequence
    boundaries (python ints). ``window``: a key is visible while ``q_pos - k_pos < window``. ``sinks`` [Hq]: one
    extra logit per head that takes probability mass and contributes nothing. ``softcap``: logits pass through
    ``cap * tanh(x / cap)``. ``allowed``: per sequence a bool [n, n] matrix of keys each query may see (sparse
    attention by selected indices), applied on top of causality. Returns [T, Hq, Dv]."""
    Hq, Hkv = q.shape[1], k.shape[1]
    rep = Hq // Hkv
    outs = []
    plain = sinks is None and softcap is None
    for si, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        n = b - a
        if n == 0:
            continue
        qs, ks, vs = q[a:b].transpose(0, 1), k[a:b].transpose(0, 1), v[a:b].transpose(0, 1)      # [H, n, D]
        if plain and window is None and allowed is None:
            o = F.scaled_dot_product_attention(qs[None], ks[None], vs[None], is_causal=True, scale=scale, enable_gqa=rep > 1)[0]
            outs.append(o.transpose(0, 1))
            continue
        idx = torch.arange(n, device=q.device)
        ok = idx[None, :] <= idx[:, None]
        if window is not None:
            ok = ok & (idx[:, None] - idx[None, :] < window)
        if allowed is not None:
            ok = ok & allowed[si]
        if plain:
            o = F.scaled_dot_product_attention(qs[None], ks[None], vs[None], attn_mask=ok[None, None], scale=scale, enable_gqa=rep > 1)[0]
            outs.append(o.transpose(0, 1))
            continue
        if rep > 1:
            ks, vs = ks.repeat_interleave(rep, dim=0), vs.repeat_interleave(rep, dim=0)
        s = torch.matmul(qs, ks.transpose(1, 2)).float() * scale
        if softcap is not None:
            s = torch.tanh(s / softcap) * softcap
        s = s.masked_fill(~ok[None], float("-inf"))
        if sinks is not None:
            s = torch.cat([s, sinks.float()[:, None, None].expand(Hq, n, 1)], dim=-1)
            p = torch.softmax(s, dim=-1)[..., :-1]
        else:
            p = torch.softmax(s, dim=-1)
        outs.append(torch.matmul(p.to(vs.dtype), vs).transpose(0, 1))
    return torch.cat(outs, dim=0)


def attention_cached(q, kc, vc, lens, scale, window=None, sinks=None, softcap=None, select=None):
    """One query token per sequence against that sequence's cached keys. q [B, Hq, Dk]; kc / vc: lists of
    [n_b, Hkv, D] tensors (the first ``lens[b]`` positions, the query's own key included)."""
    outs = []
    Hq = q.shape[1]
    for b in range(q.shape[0]):
        k, v = kc[b], vc[b]
        n = k.shape[0]
        lo = max(0, n - window) if window is not None else 0
        k, v = k[lo:], v[lo:]
        if select is not None:                       # sparse attention: only the chosen cache positions
            k, v = k[select[b]], v[select[b]]
        rep = Hq // k.shape[1]
        ks, vs = k.transpose(0, 1), v.transpose(0, 1)
        if rep > 1:
            ks, vs = ks.repeat_interleave(rep, dim=0), vs.repeat_interleave(rep, dim=0)
        s = torch.matmul(q[b][:, None, :], ks.transpose(1, 2)).float() * scale        # [Hq, 1, n]
        if softcap is not None:
            s = torch.tanh(s / softcap) * softcap
        if sinks is not None:
            s = torch.cat([s, sinks.float()[:, None, None]], dim=-1)
            p = torch.softmax(s, dim=-1)[..., :-1]
        else:
            p = torch.softmax(s, dim=-1)
        outs.append(torch.matmul(p.to(vs.dtype), vs)[:, 0])
    return torch.stack(outs)


def experts_forward(x, idx, wts, apply_expert, n_experts: int):
    """Token-choice expert mixture: row t goes through experts ``idx[t, :]`` with weights ``wts[t, :]``.
    ``apply_expert(e, rows)`` -> rows' outputs. Experts are visited in order (deterministic accumulation)."""
    out = torch.zeros_like(x)
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=n_experts).tolist()
    tok = (order // idx.shape[1])
    w_sorted = wts.reshape(-1)[order]
    pos = 0
    for e, c in enumerate(counts):
        if c == 0:
            continue
        rows = tok[pos:pos + c]
        y = apply_expert(e, x[rows]) * w_sorted[pos:pos + c, None].to(x.dtype)
        out = out.index_add(0, rows, y.to(out.dtype))
        pos += c
    return out


def gated_delta_rule(q, k, v, g, beta, state=None):
    """Gated delta rule, one sequence: q, k [n, H, Dk] (already L2-normalised), v [n, H, Dv], g [n, H] (log decay),
    beta [n, H]. S <- S * exp(g) ; S <- S + k (beta (v - S^T k))^T ; o = S^T q / sqrt(Dk). Returns (o [n, H, Dv],
    final state [H, Dk, Dv]). Recurrent form in fp32 (the oracle of the chunked kernels)."""
    n, H, Dk = k.shape
    Dv = v.shape[-1]
    if q.is_cuda and q.dtype == torch.bfloat16 and Dk in (64, 128, 256) and n > 0:
        # the recurrent CUDA kernels (forward and reverse sweep), differentiable through their autograd wrapper
        from ..ops.gdn import gated_delta_rule as native_rule
        cu = torch.tensor([0, n], dtype=torch.int32, device=q.device)
        o, st = native_rule(q.contiguous(), k.to(q.dtype).contiguous(), v.to(q.dtype).contiguous(), g.float(), beta.float(), cu,
                            scale=1.0 / math.sqrt(Dk), initial_state=None if state is None else state.float()[None])
        return o.to(v.dtype), st[0]
    qf, kf, vf = q.float() / math.sqrt(Dk), k.float(), v.float()
    S = torch.zeros(H, Dk, Dv, dtype=torch.float32, device=q.device) if state is None else state.float()
    outs = []
    for t in range(n):
        S = S * g[t].float().exp()[:, None, None]
        mem = torch.einsum("hkv,hk->hv", S, kf[t])
        delta = (vf[t] - mem) * beta[t].float()[:, None]
        S = S + kf[t][:, :, None] * delta[:, None, :]
        outs.append(torch.einsum("hkv,hk->hv", S, qf[t]))
    return torch.stack(outs).to(v.dtype), S


def l2norm(x, eps: float = 1e-6):
    return x * torch.rsqrt(x.float().pow(2).sum(-1, keepdim=True) + eps).to(x.dtype)


# ------------------------------------------------------------------------------------------ parameters
class FamilyParams(FlatParams):
    """Flat parameter buffer under the checkpoint's tensor names, with the HF import / export the rest of the framework
    calls (``load_hf_state_dict`` / ``to_hf_state_dict`` / ``init_random``)."""

    def __init__(self, cfg, device, dtype, layout, spec):
        super().__init__(cfg, device, dtype, layout=layout)
        self.spec = spec

    def init_random(self, std: float = 0.02, seed: int = 0) -> None:
        g = torch.Generator(device="cpu").manual_seed(seed)
        for name, v in self.views.items():
            kind = self.spec.init_kind(name)
            if kind == "ones":
                v.fill_(1.0)
            elif kind == "zeros":
                v.zero_()
            elif kind == "a_log":
                v.copy_(torch.log(torch.empty(v.shape).uniform_(1.0, 16.0, generator=g)).to(v.dtype))
            else:
                v.copy_((torch.randn(v.shape, generator=g) * std).to(v.dtype))

    def load_hf_state_dict(self, sd: dict, strict: bool = True) -> list[str]:
        """Copies tensors by name. Checkpoints that store every expert separately
        (``mlp.experts.<e>.{gate,up,down}_proj.weight``) are stacked into the ``[E, ...]`` tensors used here."""
        sd = dict(sd)
        if not any(".language_model." in n for n in self.layout):
            # a multimodal checkpoint read by its text family: the decoder's tensors sit under ``...language_model.``
            for k in [k for k in sd if ".language_model." in k]:
                sd.setdefault(k.replace("language_model.", "", 1), sd[k])
        missing = []
        for name in self.layout:
            t = sd.get(name)
            if t is None and name.endswith(("mlp.experts.gate_up_proj", "mlp.experts.down_proj")):
                base = name[: name.rindex(".experts.") + len(".experts.")]
                E = self.layout[name][0]
                if f"{base}0.down_proj.weight" in sd:
                    if name.endswith("gate_up_proj"):
                        t = torch.stack([torch.cat([sd[f"{base}{e}.gate_proj.weight"], sd[f"{base}{e}.up_proj.weight"]], 0) for e in range(E)])
                    else:
                        t = torch.stack([sd[f"{base}{e}.down_proj.weight"] for e in range(E)])
            if t is None:
                missing.append(name)
                continue
            self.views[name].copy_(t.to(self.views[name].dtype).reshape(self.views[name].shape))
        if strict and missing:
            raise KeyError(f"checkpoint lacks {missing[:5]} ... ({len(missing)} tensors)")
        return missing

    def to_hf_state_dict(self) -> "OrderedDict[str, torch.Tensor]":
        shape_of = getattr(self.spec, "checkpoint_shape", lambda n: None)
        return OrderedDict((n, self.views[n] if shape_of(n) is None else self.views[n].view(shape_of(n))) for n in self.layout)


# ------------------------------------------------------------------------------------------ the model
class FamilyModel:
    """A decoder of one of ``FAMILY_TYPES`` built from its HF config dictionary ``hf``."""

    def __init__(self, cfg: ModelConfig, device="cuda", dtype=torch.bfloat16, hf: dict | None = None):
        self.cfg = cfg
        self.hf = dict(cfg.extra.get("hf_config") or hf or {})      # the flattened form (vision-language configs nest the decoder)
        self.kind = self.hf.get("model_type", cfg.model_type)
        assert self.kind in FAMILY_TYPES, f"'{self.kind}' is not one of {FAMILY_TYPES}"
        self.device, self.dtype = torch.device(device), dtype
        self.spec = _SPECS[self.kind](self.hf)
        self.layout = self.spec.layout()
        self.params = self._make_params()
        self.buffers: dict[str, torch.Tensor] = self.spec.buffers(self.device)      # non-trainable tensors of the checkpoint
        self.recompute = "full"
        self._saved = None
        self._rope_cache: dict = {}
        self.recurrent_state: dict = {}       # sampler: per-sequence state of linear-attention layers, keyed by the first page
        # linear-attention state is per sequence and keyed by its first cache page: samples of one prompt must not share pages
        self.has_recurrent_state = any(t == "linear_attention" for t in getattr(self.spec, "types", [])) or self.kind == "glm_moe_dsa"

    # ---- parameters
    def _make_params(self):
        """Storage for ``self.layout`` (a model with parameter shards allocates its pieces instead)."""
        return FamilyParams(self.cfg, self.device, self.dtype, self.layout, self.spec)

    def _layer_call(self, W, l: int, h, ctx):
        """Decoder layer ``l`` on the weights ``W`` (a model with parameter shards gathers the layer first)."""
        return self.spec.layer(W, l, h, ctx)

    def init_random(self, std: float = 0.02, seed: int = 0) -> None:
        self.params.init_random(std, seed)

    def load_state_dict(self, sd: dict, strict: bool = True) -> None:
        """Tensors by checkpoint name (the HF names of the family); buffers of the checkpoint are taken along."""
        self.params.load_hf_state_dict(sd, strict=strict)
        for n in list(self.buffers):
            if n in sd:
                self.buffers[n] = sd[n].to(self.device)

    def state_dict(self) -> "OrderedDict[str, torch.Tensor]":
        out = OrderedDict((n, self.params[n]) for n in self.layout)
        out.update(self.buffers)
        return out

    # ---- rope tables
    def _rope(self, which: str, positions: torch.Tensor):
        key = which
        if key not in self._rope_cache:
            self._rope_cache[key] = self.spec.rope(which)
        inv, att = self._rope_cache[key]
        ang = positions.to(torch.float32)[:, None] * inv.to(positions.device)[None, :]
        emb = torch.cat([ang, ang], dim=-1)
        return emb.cos() * att, emb.sin() * att

    # ---- training interface (DenseModel's)
    def _leaves(self, grad: bool) -> dict:
        if not grad:
            return dict(self.params.views)
        return {n: v.detach().requires_grad_(self.spec.trainable(n)) for n, v in self.params.views.items()}

    def hidden_states(self, W: dict, input_ids, position_ids, cu: list[int], ckpt: bool, multimodal: dict | None = None):
        """``multimodal`` (vision-language families): ``pixel_values`` [patches, patch_dim] and ``image_grid_thw`` [images, 3]
        of every image of the packed batch in token order, and optionally ``mrope_positions`` [3, T] (else the packed
        ``position_ids`` serve all three rotary rows, which is exact for text-only sequences)."""
        if multimodal:
            x = self.spec.embed(W, input_ids, multimodal)
            if multimodal.get("mrope_positions") is not None:
                position_ids = multimodal["mrope_positions"].to(input_ids.device)
        else:
            x = self.spec.embed(W, input_ids)
        ctx = {"positions": position_ids, "cu": cu, "model": self}
        for l in range(self.cfg.num_hidden_layers):
            fn = lambda h, l=l: self._layer_call(W, l, h, ctx)      # noqa: E731
            x = checkpoint(fn, x, use_reentrant=False) if ckpt else fn(x)
        return self.spec.final_norm(W, x)

    def logprob_entropy(self, W: dict, h, labels, temperature: float, ckpt: bool, chunk: int = 2048):
        """Per-token log-prob of ``labels`` and entropy from hidden states, vocabulary in fp32, token chunks recomputed
        in backward so that no [T, V] tensor outlives its chunk."""
        head = self.spec.head_weight(W)
        cap = self.spec.final_softcap

        def piece(hc, lc):
            z = F.linear(hc, head).float()
            if cap:
                z = torch.tanh(z / cap) * cap
            z = z / temperature
            lse = torch.logsumexp(z, dim=-1)
            p = torch.softmax(z, dim=-1)
            ent = lse - (p * z).sum(-1)
            lp = z.gather(1, lc.clamp_min(0)[:, None].long())[:, 0] - lse
            return torch.where(lc >= 0, lp, torch.zeros_like(lp)), ent
        lps, ents = [], []
        for s in range(0, h.shape[0], chunk):
            hc, lc = h[s:s + chunk], labels[s:s + chunk]
            a, b = checkpoint(piece, hc, lc, use_reentrant=False) if (ckpt and torch.is_grad_enabled()) else piece(hc, lc)
            lps.append(a)
            ents.append(b)
        return torch.cat(lps), torch.cat(ents)

    def forward(self, batch, temperature: float = 1.0, save_for_backward: bool = False):
        cu = batch.cu_seqlens.tolist()
        with torch.set_grad_enabled(save_for_backward):
            W = self._leaves(save_for_backward)
            ck = save_for_backward and self.recompute == "full"
            h = self.hidden_states(W, batch.input_ids.long(), batch.position_ids, cu, ck, getattr(batch, "multimodal", None))
            lp, ent = self.logprob_entropy(W, h, batch.labels, temperature, ck)
        if save_for_backward:
            self._saved = (W, lp, ent)
        return lp.detach(), ent.detach()

    def backward(self, g_logprob, g_entropy=None) -> None:
        assert self._saved is not None, "forward(save_for_backward=True) must come first"
        W, lp, ent = self._saved
        self._saved = None
        self.params.alloc_grads()
        outs, grads = [lp], [g_logprob.to(lp.dtype)]
        if g_entropy is not None:
            outs.append(ent)
            grads.append(g_entropy.to(ent.dtype))
        torch.autograd.backward(outs, grads)
        for n, leaf in W.items():
            if leaf.grad is not None:
                self.params.grads[n].add_(leaf.grad.float())

    def logits(self, input_ids: torch.Tensor, position_ids: torch.Tensor | None = None, multimodal: dict | None = None) -> torch.Tensor:
        """fp32 logits [T, V] of one sequence (tests, evaluation)."""
        T = input_ids.numel()
        pos = position_ids if position_ids is not None else torch.arange(T, device=input_ids.device)
        with torch.no_grad():
            W = self._leaves(False)
            h = self.hidden_states(W, input_ids.long(), pos, [0, T], False, multimodal)
            z = F.linear(h, self.spec.head_weight(W)).float()
            if self.spec.final_softcap:
                z = torch.tanh(z / self.spec.final_softcap) * self.spec.final_softcap
        return z

    # ---- sampler interface
    @torch.no_grad()
    def prefill(self, batch, cache, tok_seq, tok_pos, block_table, last_index):
        W = self._leaves(False)
        cu = batch.cu_seqlens.tolist()
        mm = getattr(batch, "multimodal", None)
        x = self.spec.embed(W, batch.input_ids.long(), mm) if mm else self.spec.embed(W, batch.input_ids.long())
        rope_pos = mm["mrope_positions"].to(x.device) if mm and mm.get("mrope_positions") is not None else batch.position_ids
        ctx = {"positions": rope_pos, "cu": cu, "model": self, "cache": cache, "tok_seq": tok_seq.long(),
               "tok_pos": tok_pos.long(), "block_table": block_table, "mode": "prefill"}
        for l in range(self.cfg.num_hidden_layers):
            x = self.spec.layer(W, l, x, ctx)
        h = self.spec.final_norm(W, x[last_index])
        z = F.linear(h, self.spec.head_weight(W)).float()
        return torch.tanh(z / self.spec.final_softcap) * self.spec.final_softcap if self.spec.final_softcap else z

    @torch.no_grad()
    def decode(self, tokens, positions, cache, block_table, seq_lens, shared=None, rope_positions=None):
        """``rope_positions``: rotary position of every token where it differs from its place in the cache (sequences
        whose prompt held images: the rotary count resumes after the prompt's largest row)."""
        W = self._leaves(False)
        B = tokens.numel()
        x = self.spec.embed(W, tokens.long())
        ctx = {"positions": positions if rope_positions is None else rope_positions, "cu": list(range(B + 1)), "model": self, "cache": cache,
               "tok_seq": torch.arange(B, device=tokens.device), "tok_pos": positions.long(), "block_table": block_table,
               "mode": "decode", "seq_lens": seq_lens}
        for l in range(self.cfg.num_hidden_layers):
            x = self.spec.layer(W, l, x, ctx)
        h = self.spec.final_norm(W, x)
        z = F.linear(h, self.spec.head_weight(W)).float()
        return torch.tanh(z / self.spec.final_softcap) * self.spec.final_softcap if self.spec.final_softcap else z

    def flops_per_token(self, seqlen: int) -> float:
        return 6.0 * self.params.numel

    supports_cuda_graph = False         # decode reads sequence lengths on the host (per-sequence gathers from the pages)

    def rotary_rows(self, prompt_ids, image_data: dict) -> torch.Tensor:
        """Three rotary rows [3, n] of a prompt whose placeholder tokens stand for ``image_data`` (vision-language families)."""
        assert self.kind in VISION_LANGUAGE_TYPES, f"'{self.kind}' takes no vision inputs"
        from types import SimpleNamespace
        from .vision import mrope_position_ids
        sp = self.spec
        proc = SimpleNamespace(image_token_id=sp.image_token, video_token_id=sp.video_token,
                               image_processor=SimpleNamespace(merge_size=sp.merge))
        ids = torch.as_tensor(list(prompt_ids), dtype=torch.long)
        g = lambda k: torch.as_tensor(image_data[k]).reshape(-1, 3) if image_data.get(k) is not None else None      # noqa: E731
        return mrope_position_ids(proc, ids, None, g("image_grid_thw"), g("video_grid_thw"), image_data.get("second_per_grid_ts")).reshape(3, -1)


# ------------------------------------------------------------------------------------------ KV cache helpers
PAGE = 128


def cache_write(cache, l: int, k, v, ctx) -> None:
    """Store k [T, Hkv, Dk] / v [T, Hkv, Dv] of the packed tokens at (row ``tok_seq``, position ``tok_pos``) of the
    paged pool; narrower heads than the pool's ``head_dim`` are zero-padded."""
    bt, seq, pos = ctx["block_table"], ctx["tok_seq"], ctx["tok_pos"]
    page = bt[seq, pos // PAGE].long()
    slot = pos % PAGE
    cache.k[l][page, : k.shape[1], slot, : k.shape[-1]] = k.to(cache.k[l].dtype)
    cache.v[l][page, : v.shape[1], slot, : v.shape[-1]] = v.to(cache.v[l].dtype)


def cache_read(cache, l: int, ctx, dk: int, dv: int, heads: int | None = None):
    """Per sequence of a decode batch: (keys [n, heads, dk], values [n, heads, dv]) for the first ``seq_lens[b]`` positions."""
    bt, lens = ctx["block_table"], ctx["seq_lens"].tolist()
    ks, vs = [], []
    hk = heads if heads is not None else cache.k[l].shape[1]
    for b, n in enumerate(lens):
        pages = bt[b, : (n + PAGE - 1) // PAGE].long()
        k = cache.k[l][pages].permute(0, 2, 1, 3).reshape(-1, cache.k[l].shape[1], cache.k[l].shape[3])[:n, :hk, :dk]
        v = cache.v[l][pages].permute(0, 2, 1, 3).reshape(-1, cache.v[l].shape[1], cache.v[l].shape[3])[:n, :hk, :dv]
        ks.append(k)
        vs.append(v)
    return ks, vs


def attend(q, k, v, ctx, l: int, scale: float, window=None, sinks=None, softcap=None, allowed=None, select=None,
           write: bool = True):
    """Attention of a layer in whichever mode the context is in: packed training / prefill (writing the cache in
    prefill) or single-token decode against the cache. ``write = False``: the layer reuses keys / values that layer
    ``l`` has already stored (layers that share another layer's keys and values)."""
    mode = ctx.get("mode")
    if mode is not None and write:
        cache_write(ctx["cache"], l, k, v, ctx)
    if mode == "decode":
        ks, vs = cache_read(ctx["cache"], l, ctx, k.shape[-1], v.shape[-1], k.shape[1])
        return attention_cached(q, ks, vs, ctx["seq_lens"], scale, window, sinks, softcap, select)
    return attention_packed(q, k, v, ctx["cu"], scale, window, sinks, softcap, allowed)


# ------------------------------------------------------------------------------------------ family specs
class _Spec:
    """What a family defines: parameter layout, initialisation kinds, rope, embedding, one layer, final norm, head."""
    final_softcap: float | None = None

    def __init__(self, hf: dict):
        self.hf = hf
        self.H = hf["hidden_size"]
        self.L = hf["num_hidden_layers"]
        self.V = hf["vocab_size"]
        self.eps = hf.get("rms_norm_eps", 1e-6)
        self.tied = bool(hf.get("tie_word_embeddings", False))
        rp = hf.get("rope_parameters") or hf.get("rope_scaling") or {}
        self.rope_params = dict(rp)
        self.rope_params.setdefault("rope_theta", hf.get("rope_theta", 10000.0))

    # layout helpers
    def base_layout(self) -> "OrderedDict[str, tuple]":
        lay = OrderedDict()
        lay["model.embed_tokens.weight"] = (self.V, self.H)
        for l in range(self.L):
            for n, s in self.layer_layout(l).items():
                lay[f"model.layers.{l}.{n}"] = s
        lay["model.norm.weight"] = (self.H,)
        if not self.tied:
            lay["lm_head.weight"] = (self.V, self.H)
        return lay

    def layout(self):
        return self.base_layout()

    def buffers(self, device) -> dict:
        return {}

    def aliases(self, sd: dict) -> dict:
        return {}

    def trainable(self, name: str) -> bool:
        return True

    def init_kind(self, name: str) -> str:
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            return "ones"
        if name.endswith(".bias") or name.endswith("_bias"):
            return "zeros"
        return "normal"

    def embed(self, W, ids):
        return W["model.embed_tokens.weight"][ids]

    def final_norm(self, W, x):
        return rms_norm(x, W["model.norm.weight"], self.eps)

    def head_weight(self, W):
        return W["model.embed_tokens.weight"] if self.tied else W["lm_head.weight"]

    def rope(self, which: str):
        raise NotImplementedError

    def P(self, W, l: int, name: str):
        return W[f"model.layers.{l}.{name}"]

    def swiglu(self, W, l, prefix, x):
        g = linear(x, self.P(W, l, f"{prefix}.gate_proj.weight"))
        u = linear(x, self.P(W, l, f"{prefix}.up_proj.weight"))
        return linear(F.silu(g) * u, self.P(W, l, f"{prefix}.down_proj.weight"))


class _DeepseekV3(_Spec):
    """DeepSeek-V3 / GLM-4.x "lite": multi-head latent attention + sigmoid routing over expert groups with a
    correction bias, shared experts, the first layers dense."""

    mla = True

    def __init__(self, hf):
        super().__init__(hf)
        self.nh = hf["num_attention_heads"]
        self.q_lora, self.kv_lora = hf.get("q_lora_rank"), hf["kv_lora_rank"]
        self.d_nope, self.d_rope, self.d_v = hf["qk_nope_head_dim"], hf["qk_rope_head_dim"], hf["v_head_dim"]
        self.d_qk = self.d_nope + self.d_rope
        self.E, self.k = hf["n_routed_experts"], hf["num_experts_per_tok"]
        self.n_group, self.topk_group = hf.get("n_group", 1), hf.get("topk_group", 1)
        self.first_dense = hf.get("first_k_dense_replace", 0)
        self.Fm, self.F = hf["moe_intermediate_size"], hf["intermediate_size"]
        self.n_shared = hf.get("n_shared_experts", 0) or 0
        self.route_scale = hf.get("routed_scaling_factor", 1.0)
        self.norm_topk = hf.get("norm_topk_prob", True)
        self.interleave = bool(hf.get("rope_interleave", True))
        self.bias = bool(hf.get("attention_bias", False))
        self.scale = self.d_qk ** -0.5
        if self.rope_params.get("rope_type", "default") == "yarn" and self.rope_params.get("mscale_all_dim"):
            m = yarn_mscale(self.rope_params["factor"], self.rope_params["mscale_all_dim"])
            self.scale *= m * m

    def is_moe(self, l):
        return l >= self.first_dense

    def layer_layout(self, l):
        H, nh = self.H, self.nh
        lay = OrderedDict()
        lay["input_layernorm.weight"] = (H,)
        if self.q_lora:
            lay["self_attn.q_a_proj.weight"] = (self.q_lora, H)
            lay["self_attn.q_a_layernorm.weight"] = (self.q_lora,)
            lay["self_attn.q_b_proj.weight"] = (nh * self.d_qk, self.q_lora)
        else:
            lay["self_attn.q_proj.weight"] = (nh * self.d_qk, H)
        lay["self_attn.kv_a_proj_with_mqa.weight"] = (self.kv_lora + self.d_rope, H)
        lay["self_attn.kv_a_layernorm.weight"] = (self.kv_lora,)
        lay["self_attn.kv_b_proj.weight"] = (nh * (self.d_nope + self.d_v), self.kv_lora)
        lay["self_attn.o_proj.weight"] = (H, nh * self.d_v)
        lay["post_attention_layernorm.weight"] = (H,)
        lay.update(self.mlp_layout(l))
        return lay

    def mlp_layout(self, l):
        H = self.H
        lay = OrderedDict()
        if self.is_moe(l):
            lay["mlp.gate.weight"] = (self.E, H)
            lay["mlp.gate.e_score_correction_bias"] = (self.E,)
            lay["mlp.experts.gate_up_proj"] = (self.E, 2 * self.Fm, H)
            lay["mlp.experts.down_proj"] = (self.E, H, self.Fm)
            if self.n_shared:
                for n, s in (("gate_proj", (self.Fm * self.n_shared, H)), ("up_proj", (self.Fm * self.n_shared, H)),
                             ("down_proj", (H, self.Fm * self.n_shared))):
                    lay[f"mlp.shared_experts.{n}.weight"] = s
        else:
            for n, s in (("gate_proj", (self.F, H)), ("up_proj", (self.F, H)), ("down_proj", (H, self.F))):
                lay[f"mlp.{n}.weight"] = s
        return lay

    def trainable(self, name):
        return not name.endswith("e_score_correction_bias")      # updated by the load-balancing rule, not by gradients

    def init_kind(self, name):
        return "zeros" if name.endswith("e_score_correction_bias") else super().init_kind(name)

    def rope(self, which):
        return rope_frequencies(self.rope_params, self.d_rope, self.hf.get("max_position_embeddings", 4096))

    def attention(self, W, l, h, ctx):
        T = h.shape[0]
        nh = self.nh
        if self.q_lora:
            qa = rms_norm(linear(h, self.P(W, l, "self_attn.q_a_proj.weight")), self.P(W, l, "self_attn.q_a_layernorm.weight"), self.eps)
            q = linear(qa, self.P(W, l, "self_attn.q_b_proj.weight"))
        else:
            q = linear(h, self.P(W, l, "self_attn.q_proj.weight"))
        q = q.view(T, nh, self.d_qk)
        ckv = linear(h, self.P(W, l, "self_attn.kv_a_proj_with_mqa.weight"))
        c, k_rot = ckv[:, : self.kv_lora], ckv[:, self.kv_lora:]
        kv = linear(rms_norm(c, self.P(W, l, "self_attn.kv_a_layernorm.weight"), self.eps), self.P(W, l, "self_attn.kv_b_proj.weight"))
        kv = kv.view(T, nh, self.d_nope + self.d_v)
        k_nope, v = kv[..., : self.d_nope], kv[..., self.d_nope:]
        cos, sin = ctx["model"]._rope("main", ctx["positions"])
        q_rot = apply_rope(q[..., self.d_nope:], cos, sin, self.interleave)
        k_rot = apply_rope(k_rot[:, None, :], cos, sin, self.interleave).expand(T, nh, self.d_rope)
        qf = torch.cat([q[..., : self.d_nope], q_rot], dim=-1)
        kf = torch.cat([k_nope, k_rot], dim=-1)
        sparse = self.select_keys(W, l, h, qa if self.q_lora else None, cos, sin, ctx)
        o = attend(qf, kf, v, ctx, l, self.scale, **sparse)
        return linear(o.reshape(T, nh * self.d_v), self.P(W, l, "self_attn.o_proj.weight"))

    def select_keys(self, W, l, h, q_resid, cos, sin, ctx) -> dict:
        """Hook for sparse attention: keyword arguments for ``attend`` (none: every causal key is visible)."""
        return {}

    def route(self, W, l, h):
        scores = F.linear(h.float(), self.P(W, l, "mlp.gate.weight").float()).sigmoid()
        choice = scores + self.P(W, l, "mlp.gate.e_score_correction_bias").float()
        if self.n_group > 1:
            grp = choice.view(-1, self.n_group, self.E // self.n_group).topk(2, dim=-1)[0].sum(-1)
            keep = torch.zeros_like(grp).scatter_(1, grp.topk(self.topk_group, dim=-1)[1], 1.0)
            mask = keep[:, :, None].expand(-1, self.n_group, self.E // self.n_group).reshape(-1, self.E)
            choice = choice.masked_fill(mask == 0, 0.0)
        idx = choice.topk(self.k, dim=-1)[1]
        w = scores.gather(1, idx)
        if self.norm_topk:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        return idx, w * self.route_scale

    def moe(self, W, l, h):
        idx, w = self.route(W, l, h)
        gu, dn = self.P(W, l, "mlp.experts.gate_up_proj"), self.P(W, l, "mlp.experts.down_proj")

        def expert(e, rows):
            g, u = F.linear(rows, gu[e]).chunk(2, dim=-1)
            return F.linear(F.silu(g) * u, dn[e])
        out = experts_forward(h, idx, w, expert, self.E)
        if self.n_shared:
            out = out + self.swiglu(W, l, "mlp.shared_experts", h)
        return out

    def layer(self, W, l, x, ctx):
        x = x + self.attention(W, l, rms_norm(x, self.P(W, l, "input_layernorm.weight"), self.eps), ctx)
        h = rms_norm(x, self.P(W, l, "post_attention_layernorm.weight"), self.eps)
        return x + (self.moe(W, l, h) if self.is_moe(l) else self.swiglu(W, l, "mlp", h))


class _GlmMoeDsa(_DeepseekV3):
    """GLM-5 (DeepSeek-V3.2 style sparse attention): latent attention in which every query attends only to the
    ``index_topk`` keys a light indexer ranks highest. The indexer has its own query heads (from the compressed query),
    one shared key per token (LayerNorm, partly rotated) and per-head weights:
    ``score[s, t] = sum_h w[s, h] * relu(q[s, h] . k[t]) * d^-1/2 * H^-1/2``; its choice is not differentiated."""

    def __init__(self, hf):
        super().__init__(hf)
        self.ih, self.idim, self.topk = hf["index_n_heads"], hf["index_head_dim"], hf["index_topk"]
        self.interleave = bool(hf.get("rope_interleave", False))

    def layer_layout(self, l):
        lay = super().layer_layout(l)
        out = OrderedDict()
        for n, shp in lay.items():
            out[n] = shp
            if n == "self_attn.o_proj.weight":
                out["self_attn.indexer.wq_b.weight"] = (self.ih * self.idim, self.q_lora)
                out["self_attn.indexer.wk.weight"] = (self.idim, self.H)
                out["self_attn.indexer.k_norm.weight"] = (self.idim,)
                out["self_attn.indexer.k_norm.bias"] = (self.idim,)
                out["self_attn.indexer.weights_proj.weight"] = (self.ih, self.H)
        return out

    def trainable(self, name):
        return super().trainable(name) and ".indexer." not in name       # the selection carries no gradient

    def init_kind(self, name):
        return "ones" if name.endswith("indexer.k_norm.weight") else super().init_kind(name)

    @torch.no_grad()
    def select_keys(self, W, l, h, q_resid, cos, sin, ctx):
        T = h.shape[0]
        r = self.d_rope
        q = F.linear(q_resid, self.P(W, l, "self_attn.indexer.wq_b.weight")).view(T, self.ih, self.idim)
        q = torch.cat([apply_rope(q[..., :r], cos, sin), q[..., r:]], dim=-1)
        k = F.layer_norm(F.linear(h, self.P(W, l, "self_attn.indexer.wk.weight")), (self.idim,),
                         self.P(W, l, "self_attn.indexer.k_norm.weight"), self.P(W, l, "self_attn.indexer.k_norm.bias"), 1e-6)
        k = torch.cat([apply_rope(k[:, None, :r], cos, sin)[:, 0], k[:, r:]], dim=-1)
        w = F.linear(h, self.P(W, l, "self_attn.indexer.weights_proj.weight")).float() * (self.ih ** -0.5)
        mode, model, cu = ctx.get("mode"), ctx["model"], ctx["cu"]
        allowed, select = [], []
        for s0, s1 in zip(cu[:-1], cu[1:]):
            if s1 == s0:
                continue
            keys = k[s0:s1]
            if mode is not None:
                key = ("index", l, int(ctx["block_table"][int(ctx["tok_seq"][s0])][0]))
                if mode == "decode":
                    keys = torch.cat([model.recurrent_state[key], keys], dim=0)
                model.recurrent_state[key] = keys
            sc = torch.relu(torch.einsum("shd,td->sht", q[s0:s1].float(), keys.float()) * (self.idim ** -0.5))
            score = torch.einsum("sht,sh->st", sc, w[s0:s1])
            n_q, n_k = score.shape
            if mode != "decode":
                causal = torch.arange(n_k, device=h.device)[None, :] <= torch.arange(n_q, device=h.device)[:, None]
                score = score.masked_fill(~causal, float("-inf"))
            # exact ties (keys whose every head was cut to zero by the ReLU) go to the later position, so that a decode step
            # and the full forward choose the same set whatever order the library's top-k visits equal values in
            score = score.double() + torch.arange(n_k, device=h.device, dtype=torch.float64)[None, :] * 1e-15
            top = score.topk(min(self.topk, n_k), dim=-1).indices
            if mode == "decode":
                select.append(top[0])
            else:
                allowed.append(torch.zeros(n_q, n_k, dtype=torch.bool, device=h.device).scatter_(1, top, True))
        return {"select": select} if mode == "decode" else {"allowed": allowed}


class _Glm4Moe(_DeepseekV3):
    """GLM-4.5 / 4.6: grouped-query attention (half of each head rotates, optional per-head q/k norm, q/k/v bias)
    with the DeepSeek-style routed + shared experts."""
    mla = False

    def __init__(self, hf):
        _Spec.__init__(self, hf)
        self.nh, self.nkv = hf["num_attention_heads"], hf["num_key_value_heads"]
        self.D = hf.get("head_dim") or self.H // self.nh
        self.rot = int(self.D * hf.get("partial_rotary_factor", 0.5))
        self.qk_norm = bool(hf.get("use_qk_norm", False))
        self.bias = bool(hf.get("attention_bias", False))
        self.E, self.k = hf["n_routed_experts"], hf["num_experts_per_tok"]
        self.n_group, self.topk_group = hf.get("n_group", 1), hf.get("topk_group", 1)
        self.first_dense = hf.get("first_k_dense_replace", 0)
        self.Fm, self.F = hf["moe_intermediate_size"], hf["intermediate_size"]
        self.n_shared = hf.get("n_shared_experts", 0) or 0
        self.route_scale = hf.get("routed_scaling_factor", 1.0)
        self.norm_topk = hf.get("norm_topk_prob", True)
        self.scale = self.D ** -0.5

    def layer_layout(self, l):
        H = self.H
        lay = OrderedDict()
        lay["input_layernorm.weight"] = (H,)
        for n, rows in (("q_proj", self.nh * self.D), ("k_proj", self.nkv * self.D), ("v_proj", self.nkv * self.D)):
            lay[f"self_attn.{n}.weight"] = (rows, H)
            if self.bias:
                lay[f"self_attn.{n}.bias"] = (rows,)
        lay["self_attn.o_proj.weight"] = (H, self.nh * self.D)
        if self.qk_norm:
            lay["self_attn.q_norm.weight"] = (self.D,)
            lay["self_attn.k_norm.weight"] = (self.D,)
        lay["post_attention_layernorm.weight"] = (H,)
        lay.update(self.mlp_layout(l))
        return lay

    def rope(self, which):
        return rope_frequencies(self.rope_params, self.rot, self.hf.get("max_position_embeddings", 4096))

    def attention(self, W, l, h, ctx):
        T = h.shape[0]
        b = (lambda n: self.P(W, l, f"self_attn.{n}.bias")) if self.bias else (lambda n: None)
        q = linear(h, self.P(W, l, "self_attn.q_proj.weight"), b("q_proj")).view(T, self.nh, self.D)
        k = linear(h, self.P(W, l, "self_attn.k_proj.weight"), b("k_proj")).view(T, self.nkv, self.D)
        v = linear(h, self.P(W, l, "self_attn.v_proj.weight"), b("v_proj")).view(T, self.nkv, self.D)
        if self.qk_norm:
            q = rms_norm(q, self.P(W, l, "self_attn.q_norm.weight"), self.eps)
            k = rms_norm(k, self.P(W, l, "self_attn.k_norm.weight"), self.eps)
        cos, sin = ctx["model"]._rope("main", ctx["positions"])
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        o = attend(q, k, v, ctx, l, self.scale)
        return linear(o.reshape(T, self.nh * self.D), self.P(W, l, "self_attn.o_proj.weight"))


class _GptOss(_Spec):
    """GPT-OSS: every layer sparse; attention with a learned sink logit per head, sliding-window layers alternate
    with full-attention layers, biases on every projection; experts use a clamped SwiGLU with interleaved gate / up
    columns and the router softmaxes over the chosen experts only."""

    def __init__(self, hf):
        super().__init__(hf)
        self.nh, self.nkv = hf["num_attention_heads"], hf["num_key_value_heads"]
        self.D = hf.get("head_dim") or self.H // self.nh
        self.E, self.k, self.F = hf["num_local_experts"], hf["num_experts_per_tok"], hf["intermediate_size"]
        self.window = hf.get("sliding_window", 128)
        self.types = hf.get("layer_types") or ["sliding_attention" if i % 2 == 0 else "full_attention" for i in range(self.L)]
        self.alpha, self.limit = 1.702, float(hf.get("swiglu_limit", 7.0))
        self.scale = self.D ** -0.5

    def layer_layout(self, l):
        H = self.H
        lay = OrderedDict()
        lay["input_layernorm.weight"] = (H,)
        for n, rows in (("q_proj", self.nh * self.D), ("k_proj", self.nkv * self.D), ("v_proj", self.nkv * self.D)):
            lay[f"self_attn.{n}.weight"] = (rows, H)
            lay[f"self_attn.{n}.bias"] = (rows,)
        lay["self_attn.o_proj.weight"] = (H, self.nh * self.D)
        lay["self_attn.o_proj.bias"] = (H,)
        lay["self_attn.sinks"] = (self.nh,)
        lay["post_attention_layernorm.weight"] = (H,)
        lay["mlp.router.weight"] = (self.E, H)
        lay["mlp.router.bias"] = (self.E,)
        lay["mlp.experts.gate_up_proj"] = (self.E, H, 2 * self.F)
        lay["mlp.experts.gate_up_proj_bias"] = (self.E, 2 * self.F)
        lay["mlp.experts.down_proj"] = (self.E, self.F, H)
        lay["mlp.experts.down_proj_bias"] = (self.E, H)
        return lay

    def rope(self, which):
        return rope_frequencies(self.rope_params, self.D, self.hf.get("max_position_embeddings", 4096))

    def layer(self, W, l, x, ctx):
        T = x.shape[0]
        h = rms_norm(x, self.P(W, l, "input_layernorm.weight"), self.eps)
        q = linear(h, self.P(W, l, "self_attn.q_proj.weight"), self.P(W, l, "self_attn.q_proj.bias")).view(T, self.nh, self.D)
        k = linear(h, self.P(W, l, "self_attn.k_proj.weight"), self.P(W, l, "self_attn.k_proj.bias")).view(T, self.nkv, self.D)
        v = linear(h, self.P(W, l, "self_attn.v_proj.weight"), self.P(W, l, "self_attn.v_proj.bias")).view(T, self.nkv, self.D)
        cos, sin = ctx["model"]._rope("main", ctx["positions"])
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        win = self.window if self.types[l] == "sliding_attention" else None
        o = attend(q, k, v, ctx, l, self.scale, window=win, sinks=self.P(W, l, "self_attn.sinks"))
        x = x + linear(o.reshape(T, self.nh * self.D), self.P(W, l, "self_attn.o_proj.weight"), self.P(W, l, "self_attn.o_proj.bias"))
        h = rms_norm(x, self.P(W, l, "post_attention_layernorm.weight"), self.eps)
        logits = F.linear(h, self.P(W, l, "mlp.router.weight"), self.P(W, l, "mlp.router.bias"))
        top, idx = logits.topk(self.k, dim=-1)
        w = torch.softmax(top, dim=-1, dtype=top.dtype)
        gu, gub = self.P(W, l, "mlp.experts.gate_up_proj"), self.P(W, l, "mlp.experts.gate_up_proj_bias")
        dn, dnb = self.P(W, l, "mlp.experts.down_proj"), self.P(W, l, "mlp.experts.down_proj_bias")

        def expert(e, rows):
            y = rows @ gu[e] + gub[e]
            g, u = y[..., ::2].clamp(max=self.limit), y[..., 1::2].clamp(-self.limit, self.limit)
            return ((u + 1) * (g * torch.sigmoid(g * self.alpha))) @ dn[e] + dnb[e]
        return x + experts_forward(h, idx, w, expert, self.E)

    def init_kind(self, name):
        return "zeros" if name.endswith("sinks") else super().init_kind(name)


class _Gemma(_Spec):
    """Gemma-2 / Gemma-3 text: embeddings scaled by sqrt(hidden), (1 + w) RMSNorm before AND after attention and
    MLP, GeGLU, query scale from ``query_pre_attn_scalar``, sliding-window layers by pattern, optional soft-capping
    of attention logits and of the final logits, per-head q/k norm and a separate local rope base (Gemma-3)."""

    def __init__(self, hf):
        super().__init__(hf)
        self.nh, self.nkv = hf["num_attention_heads"], hf["num_key_value_heads"]
        self.D = hf.get("head_dim") or self.H // self.nh
        self.F = hf["intermediate_size"]
        self.tied = bool(hf.get("tie_word_embeddings", True))
        self.window = hf.get("sliding_window")
        self.gemma3 = hf.get("model_type") == "gemma3_text"
        pat = hf.get("sliding_window_pattern", 6 if self.gemma3 else 2)
        self.types = hf.get("layer_types") or [
            "full_attention" if (i + 1) % pat == 0 else "sliding_attention" for i in range(self.L)]
        self.scale = float(hf.get("query_pre_attn_scalar", self.D)) ** -0.5
        self.attn_cap = hf.get("attn_logit_softcapping")
        self.final_softcap = hf.get("final_logit_softcapping")
        self.local_theta = hf.get("rope_local_base_freq", 10000.0)
        rp = hf.get("rope_parameters") or {}
        if "full_attention" in rp:                        # per-layer-type rope parameters
            self.rope_params = dict(rp["full_attention"])
            self.local_rope = dict(rp.get("sliding_attention", {"rope_type": "default", "rope_theta": self.local_theta}))
        else:
            self.local_rope = {"rope_type": "default", "rope_theta": self.local_theta if self.gemma3 else self.rope_params["rope_theta"]}

    def layer_layout(self, l):
        H = self.H
        lay = OrderedDict()
        lay["input_layernorm.weight"] = (H,)
        lay["self_attn.q_proj.weight"] = (self.nh * self.D, H)
        lay["self_attn.k_proj.weight"] = (self.nkv * self.D, H)
        lay["self_attn.v_proj.weight"] = (self.nkv * self.D, H)
        lay["self_attn.o_proj.weight"] = (H, self.nh * self.D)
        if self.gemma3:
            lay["self_attn.q_norm.weight"] = (self.D,)
            lay["self_attn.k_norm.weight"] = (self.D,)
        lay["post_attention_layernorm.weight"] = (H,)
        lay["pre_feedforward_layernorm.weight"] = (H,)
        lay["post_feedforward_layernorm.weight"] = (H,)
        for n, s in (("gate_proj", (self.F, H)), ("up_proj", (self.F, H)), ("down_proj", (H, self.F))):
            lay[f"mlp.{n}.weight"] = s
        return lay

    def init_kind(self, name):       # (1 + w) norms start at w = 0
        return "zeros" if name.endswith("norm.weight") else "normal"

    def rope(self, which):
        rp = self.local_rope if which == "local" else self.rope_params
        return rope_frequencies(rp, self.D, self.hf.get("max_position_embeddings", 8192))

    def embed(self, W, ids):
        e = W["model.embed_tokens.weight"][ids]
        return e * torch.tensor(self.H ** 0.5, dtype=e.dtype)

    def final_norm(self, W, x):
        return rms_norm(x, W["model.norm.weight"], self.eps, plus_one=True)

    def layer(self, W, l, x, ctx):
        T = x.shape[0]
        n1 = lambda t, name: rms_norm(t, self.P(W, l, name), self.eps, plus_one=True)      # noqa: E731
        h = n1(x, "input_layernorm.weight")
        q = linear(h, self.P(W, l, "self_attn.q_proj.weight")).view(T, self.nh, self.D)
        k = linear(h, self.P(W, l, "self_attn.k_proj.weight")).view(T, self.nkv, self.D)
        v = linear(h, self.P(W, l, "self_attn.v_proj.weight")).view(T, self.nkv, self.D)
        if self.gemma3:
            q, k = n1(q, "self_attn.q_norm.weight"), n1(k, "self_attn.k_norm.weight")
        sliding = self.types[l] == "sliding_attention"
        cos, sin = ctx["model"]._rope("local" if sliding else "main", ctx["positions"])
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        o = attend(q, k, v, ctx, l, self.scale, window=self.window if sliding else None, softcap=self.attn_cap)
        x = x + n1(linear(o.reshape(T, self.nh * self.D), self.P(W, l, "self_attn.o_proj.weight")), "post_attention_layernorm.weight")
        h = n1(x, "pre_feedforward_layernorm.weight")
        g = linear(h, self.P(W, l, "mlp.gate_proj.weight"))
        u = linear(h, self.P(W, l, "mlp.up_proj.weight"))
        m = linear(F.gelu(g, approximate="tanh") * u, self.P(W, l, "mlp.down_proj.weight"))
        return x + n1(m, "post_feedforward_layernorm.weight")


class _Gemma4(_Spec):
    """Gemma-4 text: sliding-window layers with the local head size alternate with global layers that use a wider
    head, their own number of KV heads, keys doubling as values (``attention_k_eq_v``) and a rope that turns only a
    share of each head; queries and keys are RMS-normalised per head (weighted), values without weight, and the
    softmax scale is 1. The last ``num_kv_shared_layers`` layers compute no keys / values of their own: each reuses
    those of the last earlier layer of its type. Optional extras: a small per-layer token embedding mixed into every
    layer through a gate, a sparse expert block in parallel with the dense MLP, a learned scalar per layer, and
    soft-capped final logits."""

    def __init__(self, hf):
        super().__init__(hf)
        g = hf.get
        self.nh, self.nkv = hf["num_attention_heads"], hf["num_key_value_heads"]
        self.D, self.Dg = hf["head_dim"], g("global_head_dim") or hf["head_dim"]
        self.k_eq_v = bool(g("attention_k_eq_v", False))
        self.nkv_g = g("num_global_key_value_heads") or self.nkv
        self.F = hf["intermediate_size"]
        self.tied = bool(g("tie_word_embeddings", True))
        self.window = g("sliding_window")
        self.types = hf["layer_types"]
        self.n_shared_kv = g("num_kv_shared_layers", 0) or 0
        self.first_shared = self.L - self.n_shared_kv
        self.double_wide = bool(g("use_double_wide_mlp", False))
        self.Hp = g("hidden_size_per_layer_input", 0) or 0
        self.Vp = g("vocab_size_per_layer_input") or self.V
        self.moe_on = bool(g("enable_moe_block", False))
        self.E, self.k, self.Fm = g("num_experts", 0) or 0, g("top_k_experts", 0) or 0, g("moe_intermediate_size", 0) or 0
        self.final_softcap = g("final_logit_softcapping")
        self.rope_by_type = hf["rope_parameters"]

    def shared(self, l):
        return self.n_shared_kv > 0 and l >= self.first_shared

    def kv_source(self, l):
        prev = self.types[: self.first_shared]
        return len(prev) - 1 - prev[::-1].index(self.types[l])

    def dims(self, l):
        full = self.types[l] != "sliding_attention"
        D = self.Dg if full else self.D
        alt = self.k_eq_v and full
        return D, (self.nkv_g if alt else self.nkv), alt

    def layout(self):
        lay = self.base_layout()
        if self.Hp:
            lay["model.embed_tokens_per_layer.weight"] = (self.Vp, self.L * self.Hp)
            lay["model.per_layer_model_projection.weight"] = (self.L * self.Hp, self.H)
            lay["model.per_layer_projection_norm.weight"] = (self.Hp,)
        return lay

    def buffers(self, device):
        return {f"model.layers.{l}.layer_scalar": torch.ones(1, device=device) for l in range(self.L)}

    def layer_layout(self, l):
        H = self.H
        D, nkv, alt = self.dims(l)
        lay = OrderedDict()
        lay["self_attn.q_norm.weight"] = (D,)
        lay["self_attn.k_norm.weight"] = (D,)
        lay["self_attn.k_proj.weight"] = (nkv * D, H)
        lay["self_attn.q_proj.weight"] = (self.nh * D, H)
        if not alt:
            lay["self_attn.v_proj.weight"] = (nkv * D, H)
        lay["self_attn.o_proj.weight"] = (H, self.nh * D)
        Fl = self.F * (2 if (self.double_wide and self.shared(l)) else 1)
        for n, shp in (("gate_proj", (Fl, H)), ("up_proj", (Fl, H)), ("down_proj", (H, Fl))):
            lay[f"mlp.{n}.weight"] = shp
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            lay[f"{n}.weight"] = (H,)
        if self.Hp:
            lay["per_layer_input_gate.weight"] = (self.Hp, H)
            lay["per_layer_projection.weight"] = (H, self.Hp)
            lay["post_per_layer_input_norm.weight"] = (H,)
        if self.moe_on:
            lay["router.proj.weight"] = (self.E, H)
            lay["router.scale"] = (H,)
            lay["router.per_expert_scale"] = (self.E,)
            lay["experts.gate_up_proj"] = (self.E, 2 * self.Fm, H)
            lay["experts.down_proj"] = (self.E, H, self.Fm)
            for n in ("post_feedforward_layernorm_1", "post_feedforward_layernorm_2", "pre_feedforward_layernorm_2"):
                lay[f"{n}.weight"] = (H,)
        return lay

    def init_kind(self, name):
        if name.endswith(("router.scale", "router.per_expert_scale")):
            return "ones"
        return super().init_kind(name)

    def rope(self, which):
        rp = dict(self.rope_by_type[which])
        if rp.get("rope_type", "default") == "proportional":
            hd = self.Dg
            angles = int(rp.get("partial_rotary_factor", 1.0) * hd // 2)
            inv = 1.0 / (float(rp["rope_theta"]) ** (torch.arange(0, 2 * angles, 2, dtype=torch.float64) / hd))
            inv = torch.cat([inv, torch.zeros(hd // 2 - angles, dtype=torch.float64)]) / float(rp.get("factor", 1.0))
            return inv.float(), 1.0
        return rope_frequencies(rp, self.Dg if which == "full_attention" else self.D, self.hf.get("max_position_embeddings", 8192))

    def embed(self, W, ids):
        e = W["model.embed_tokens.weight"][ids]
        x = e * torch.tensor(self.H ** 0.5, dtype=e.dtype)
        self._per_layer = None
        if self.Hp:
            T = ids.shape[0]
            pe = W["model.embed_tokens_per_layer.weight"][ids] * torch.tensor(self.Hp ** 0.5, dtype=e.dtype)
            proj = linear(x, W["model.per_layer_model_projection.weight"]) * (self.H ** -0.5)
            proj = rms_norm(proj.view(T, self.L, self.Hp), W["model.per_layer_projection_norm.weight"], self.eps)
            self._per_layer = (proj + pe.view(T, self.L, self.Hp)) * (2.0 ** -0.5)
        self._kv = {}
        return x

    def layer(self, W, l, x, ctx):
        T = x.shape[0]
        D, nkv, alt = self.dims(l)
        N = lambda t, name: rms_norm(t, self.P(W, l, name), self.eps)      # noqa: E731
        sliding = self.types[l] == "sliding_attention"
        h = N(x, "input_layernorm.weight")
        cos, sin = ctx["model"]._rope(self.types[l], ctx["positions"])
        q = apply_rope(N(linear(h, self.P(W, l, "self_attn.q_proj.weight")).view(T, self.nh, D), "self_attn.q_norm.weight"), cos, sin)
        if self.shared(l):
            src = self.kv_source(l)
            k, v = self._kv[src]
            o = attend(q, k, v, ctx, src, 1.0, window=self.window if sliding else None, write=False)
        else:
            kr = linear(h, self.P(W, l, "self_attn.k_proj.weight")).view(T, nkv, D)
            vr = kr if alt else linear(h, self.P(W, l, "self_attn.v_proj.weight")).view(T, nkv, D)
            k = apply_rope(N(kr, "self_attn.k_norm.weight"), cos, sin)
            v = rms_norm(vr, None, self.eps)
            self._kv[l] = (k, v)
            o = attend(q, k, v, ctx, l, 1.0, window=self.window if sliding else None)
        x = x + N(linear(o.reshape(T, self.nh * D), self.P(W, l, "self_attn.o_proj.weight")), "post_attention_layernorm.weight")
        res = x
        h = N(x, "pre_feedforward_layernorm.weight")
        g = linear(h, self.P(W, l, "mlp.gate_proj.weight"))
        m = linear(F.gelu(g, approximate="tanh") * linear(h, self.P(W, l, "mlp.up_proj.weight")), self.P(W, l, "mlp.down_proj.weight"))
        if self.moe_on:
            m1 = N(m, "post_feedforward_layernorm_1.weight")
            r = rms_norm(res, None, self.eps) * self.P(W, l, "router.scale") * (self.H ** -0.5)
            probs = torch.softmax(F.linear(r, self.P(W, l, "router.proj.weight")), dim=-1)
            wts, idx = probs.topk(self.k, dim=-1)
            wts = wts / wts.sum(-1, keepdim=True) * self.P(W, l, "router.per_expert_scale")[idx]
            gu, dn = self.P(W, l, "experts.gate_up_proj"), self.P(W, l, "experts.down_proj")

            def expert(e, rows):
                a, b = F.linear(rows, gu[e]).chunk(2, dim=-1)
                return F.linear(F.gelu(a, approximate="tanh") * b, dn[e])
            m2 = experts_forward(N(res, "pre_feedforward_layernorm_2.weight"), idx, wts, expert, self.E)
            m = m1 + N(m2, "post_feedforward_layernorm_2.weight")
        x = res + N(m, "post_feedforward_layernorm.weight")
        if self.Hp:
            gate = F.gelu(linear(x, self.P(W, l, "per_layer_input_gate.weight")), approximate="tanh") * self._per_layer[:, l]
            x = x + N(linear(gate, self.P(W, l, "per_layer_projection.weight")), "post_per_layer_input_norm.weight")
        return x * ctx["model"].buffers[f"model.layers.{l}.layer_scalar"].to(x.dtype)


class _Qwen3Next(_Spec):
    """Qwen3-Next / Qwen3.5: three of four layers mix tokens with a gated delta-rule linear attention (short causal
    convolution over q | k | v, L2-normalised keys and queries, per-head decay and write strength, gated RMSNorm on
    the output); every fourth layer is full attention with a sigmoid output gate, (1 + w) norms and a quarter of each
    head rotated. MLPs are sparse with one always-on shared expert behind its own sigmoid gate."""

    def __init__(self, hf):
        super().__init__(hf)
        self.nh, self.nkv = hf["num_attention_heads"], hf["num_key_value_heads"]
        self.D = hf.get("head_dim") or self.H // self.nh
        self.rot = int(self.D * (hf.get("partial_rotary_factor") or self.rope_params.get("partial_rotary_factor", 0.25)))
        self.types = hf.get("layer_types") or [
            "full_attention" if (i + 1) % hf.get("full_attention_interval", 4) == 0 else "linear_attention" for i in range(self.L)]
        self.nv, self.nk = hf["linear_num_value_heads"], hf["linear_num_key_heads"]
        self.dk, self.dv = hf["linear_key_head_dim"], hf["linear_value_head_dim"]
        self.conv_k = hf.get("linear_conv_kernel_dim", 4)
        self.E, self.k = hf.get("num_experts", 0), hf.get("num_experts_per_tok", 0)
        self.Fm, self.F = hf.get("moe_intermediate_size", 0), hf.get("intermediate_size", 0)
        self.Fs = hf.get("shared_expert_intermediate_size", 0)
        self.sparse_step = hf.get("decoder_sparse_step", 1)
        self.mlp_only = set(hf.get("mlp_only_layers", []) or [])
        self.norm_topk = hf.get("norm_topk_prob", True)
        self.scale = self.D ** -0.5

    def is_moe(self, l):
        return l not in self.mlp_only and self.E > 0 and (l + 1) % self.sparse_step == 0

    def layer_layout(self, l):
        H = self.H
        lay = OrderedDict()
        lay["input_layernorm.weight"] = (H,)
        if self.types[l] == "linear_attention":
            kd, vd = self.nk * self.dk, self.nv * self.dv
            lay["linear_attn.in_proj_qkvz.weight"] = (2 * kd + 2 * vd, H)
            lay["linear_attn.in_proj_ba.weight"] = (2 * self.nv, H)
            lay["linear_attn.conv1d.weight"] = (2 * kd + vd, 1, self.conv_k)
            lay["linear_attn.dt_bias"] = (self.nv,)
            lay["linear_attn.A_log"] = (self.nv,)
            lay["linear_attn.norm.weight"] = (self.dv,)
            lay["linear_attn.out_proj.weight"] = (H, vd)
        else:
            lay["self_attn.q_proj.weight"] = (2 * self.nh * self.D, H)
            lay["self_attn.k_proj.weight"] = (self.nkv * self.D, H)
            lay["self_attn.v_proj.weight"] = (self.nkv * self.D, H)
            lay["self_attn.o_proj.weight"] = (H, self.nh * self.D)
            lay["self_attn.q_norm.weight"] = (self.D,)
            lay["self_attn.k_norm.weight"] = (self.D,)
        lay["post_attention_layernorm.weight"] = (H,)
        if self.is_moe(l):
            lay["mlp.gate.weight"] = (self.E, H)
            lay["mlp.experts.gate_up_proj"] = (self.E, 2 * self.Fm, H)
            lay["mlp.experts.down_proj"] = (self.E, H, self.Fm)
            for n, s in (("gate_proj", (self.Fs, H)), ("up_proj", (self.Fs, H)), ("down_proj", (H, self.Fs))):
                lay[f"mlp.shared_expert.{n}.weight"] = s
            lay["mlp.shared_expert_gate.weight"] = (1, H)
        else:
            for n, s in (("gate_proj", (self.F, H)), ("up_proj", (self.F, H)), ("down_proj", (H, self.F))):
                lay[f"mlp.{n}.weight"] = s
        return lay

    def init_kind(self, name):
        if name.endswith("linear_attn.norm.weight") or name.endswith("dt_bias"):
            return "ones"
        if name.endswith("A_log"):
            return "a_log"
        if name.endswith("norm.weight"):
            return "zeros"                       # (1 + w) norms
        return "normal"

    def rope(self, which):
        return rope_frequencies(self.rope_params, self.rot, self.hf.get("max_position_embeddings", 4096))

    def final_norm(self, W, x):
        return rms_norm(x, W["model.norm.weight"], self.eps, plus_one=True)

    def full_attention(self, W, l, h, ctx):
        T = h.shape[0]
        qg = linear(h, self.P(W, l, "self_attn.q_proj.weight")).view(T, self.nh, 2 * self.D)
        q, gate = qg[..., : self.D], qg[..., self.D:].reshape(T, self.nh * self.D)
        k = linear(h, self.P(W, l, "self_attn.k_proj.weight")).view(T, self.nkv, self.D)
        v = linear(h, self.P(W, l, "self_attn.v_proj.weight")).view(T, self.nkv, self.D)
        q = rms_norm(q, self.P(W, l, "self_attn.q_norm.weight"), self.eps, plus_one=True)
        k = rms_norm(k, self.P(W, l, "self_attn.k_norm.weight"), self.eps, plus_one=True)
        cos, sin = ctx["model"]._rope("main", ctx["positions"])
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        o = attend(q, k, v, ctx, l, self.scale).reshape(T, self.nh * self.D)
        return linear(o * torch.sigmoid(gate), self.P(W, l, "self_attn.o_proj.weight"))

    def project_linear(self, W, l, h):
        """(q | k | v rows [T, C], z [T, nv, dv], b [T, nv], a [T, nv]) from the fused, key-head-grouped projections."""
        T = h.shape[0]
        nk, nv, dk, dv = self.nk, self.nv, self.dk, self.dv
        r = nv // nk
        qkvz = linear(h, self.P(W, l, "linear_attn.in_proj_qkvz.weight")).view(T, nk, 2 * dk + 2 * r * dv)
        ba = linear(h, self.P(W, l, "linear_attn.in_proj_ba.weight")).view(T, nk, 2 * r)
        q, k, v, z = torch.split(qkvz, [dk, dk, r * dv, r * dv], dim=-1)
        b, a = ba[..., :r].reshape(T, nv), ba[..., r:].reshape(T, nv)
        mixed = torch.cat([q.reshape(T, nk * dk), k.reshape(T, nk * dk), v.reshape(T, nv * dv)], dim=-1)
        return mixed, z.reshape(T, nv, dv), b, a

    def linear_attention(self, W, l, h, ctx):
        T = h.shape[0]
        nk, nv, dk, dv = self.nk, self.nv, self.dk, self.dv
        r = nv // nk
        mixed, z, b, a = self.project_linear(W, l, h)                                                         # mixed [T, C]
        wconv = self.P(W, l, "linear_attn.conv1d.weight")[:, 0, :]                                            # [C, K]
        K = self.conv_k
        mode, model = ctx.get("mode"), ctx["model"]
        beta = torch.sigmoid(b)
        g = -self.P(W, l, "linear_attn.A_log").float().exp() * F.softplus(a.float() + self.P(W, l, "linear_attn.dt_bias").float())
        outs = []
        cu = ctx["cu"]
        for s_i, (s0, s1) in enumerate(zip(cu[:-1], cu[1:])):
            if s1 == s0:
                continue
            key = None
            prev_conv = prev_state = None
            if mode is not None:
                key = (l, int(ctx["block_table"][int(ctx["tok_seq"][s0])][0]))
                if mode == "decode":
                    prev_conv, prev_state = model.recurrent_state[key]
            seg = mixed[s0:s1]
            hist = prev_conv if prev_conv is not None else torch.zeros(K - 1, seg.shape[1], dtype=seg.dtype, device=seg.device)
            padded = torch.cat([hist, seg], dim=0)                                                              # [n + K - 1, C]
            win = padded.unfold(0, K, 1)                                                                        # [n, C, K]
            conv = F.silu((win * wconv[None].to(win.dtype)).sum(-1))
            n = s1 - s0
            qs, ks, vs = torch.split(conv, [nk * dk, nk * dk, nv * dv], dim=-1)
            qs, ks = l2norm(qs.reshape(n, nk, dk)), l2norm(ks.reshape(n, nk, dk))
            if r > 1:
                qs, ks = qs.repeat_interleave(r, dim=1), ks.repeat_interleave(r, dim=1)
            o, S = gated_delta_rule(qs, ks, vs.reshape(n, nv, dv), g[s0:s1], beta[s0:s1], prev_state)
            if key is not None:
                model.recurrent_state[key] = (padded[-(K - 1):].clone(), S)
            outs.append(o)
        o = torch.cat(outs, dim=0)                                                                               # [T, nv, dv]
        of = o.float()
        of = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + self.eps)
        o = (self.P(W, l, "linear_attn.norm.weight") * of.to(h.dtype)) * F.silu(z.float()).to(h.dtype)
        return linear(o.reshape(T, nv * dv), self.P(W, l, "linear_attn.out_proj.weight"))

    def moe(self, W, l, h):
        probs = torch.softmax(F.linear(h, self.P(W, l, "mlp.gate.weight")), dim=-1, dtype=torch.float)
        w, idx = probs.topk(self.k, dim=-1)
        if self.norm_topk:
            w = w / w.sum(-1, keepdim=True)
        gu, dn = self.P(W, l, "mlp.experts.gate_up_proj"), self.P(W, l, "mlp.experts.down_proj")

        def expert(e, rows):
            g, u = F.linear(rows, gu[e]).chunk(2, dim=-1)
            return F.linear(F.silu(g) * u, dn[e])
        out = experts_forward(h, idx, w.to(h.dtype), expert, self.E)
        shared = self.swiglu(W, l, "mlp.shared_expert", h)
        return out + torch.sigmoid(F.linear(h, self.P(W, l, "mlp.shared_expert_gate.weight"))) * shared

    def layer(self, W, l, x, ctx):
        h = rms_norm(x, self.P(W, l, "input_layernorm.weight"), self.eps, plus_one=True)
        mix = self.linear_attention if self.types[l] == "linear_attention" else self.full_attention
        x = x + mix(W, l, h, ctx)
        h = rms_norm(x, self.P(W, l, "post_attention_layernorm.weight"), self.eps, plus_one=True)
        return x + (self.moe(W, l, h) if self.is_moe(l) else self.swiglu(W, l, "mlp", h))


class _Qwen35(_Qwen3Next):
    """Qwen3.5 text models: the Qwen3-Next layer with separate, ungrouped q|k|v, z, b and a projections."""

    def layer_layout(self, l):
        lay = super().layer_layout(l)
        if self.types[l] != "linear_attention":
            return lay
        kd, vd = self.nk * self.dk, self.nv * self.dv
        out = OrderedDict()
        for n, shp in lay.items():
            if n == "linear_attn.in_proj_qkvz.weight":
                out["linear_attn.in_proj_qkv.weight"] = (2 * kd + vd, self.H)
                out["linear_attn.in_proj_z.weight"] = (vd, self.H)
            elif n == "linear_attn.in_proj_ba.weight":
                out["linear_attn.in_proj_b.weight"] = (self.nv, self.H)
                out["linear_attn.in_proj_a.weight"] = (self.nv, self.H)
            else:
                out[n] = shp
        return out

    def project_linear(self, W, l, h):
        T = h.shape[0]
        mixed = linear(h, self.P(W, l, "linear_attn.in_proj_qkv.weight"))
        z = linear(h, self.P(W, l, "linear_attn.in_proj_z.weight")).view(T, self.nv, self.dv)
        return mixed, z, F.linear(h, self.P(W, l, "linear_attn.in_proj_b.weight")), F.linear(h, self.P(W, l, "linear_attn.in_proj_a.weight"))


class _Qwen2VL(_Spec):
    """Qwen2-VL: a Qwen2 decoder (q / k / v biases) whose rotary angles come from three position rows (temporal,
    height, width: text tokens carry the same number in all three), fed with the embeddings of a vision transformer
    at the image placeholder tokens. The tower works on flattened patches [N, C * t * p * p] in merge-window order:
    linear patch embedding (the checkpoint's Conv3d kernel flattened), blocks of LayerNorm - full attention inside
    each frame with 2-D rotary angles (half of a head's pairs follow the patch row, half the column) - LayerNorm -
    QuickGELU MLP, then LayerNorm and a two-layer MLP over each window of merge^2 patches.
    Reference: axon/models/transformers/qwen2_vl.py (packed forward of the HF model), HF modeling_qwen2_vl.py."""

    def __init__(self, hf):
        super().__init__(hf)
        self.nh, self.nkv = hf["num_attention_heads"], hf.get("num_key_value_heads", hf["num_attention_heads"])
        self.D = hf.get("head_dim") or self.H // self.nh
        self.F = hf["intermediate_size"]
        self.sections = list(self.rope_params.get("mrope_section") or [self.D // 2, 0, 0])
        v = dict(hf["vision_config"])
        self.v = v
        self.vE, self.vL, self.vH = v["embed_dim"], v["depth"], v["num_heads"]
        self.vF = int(v["embed_dim"] * v.get("mlp_ratio", 4))
        self.merge = v.get("spatial_merge_size", 2)
        self.patch_dim = v.get("in_channels", 3) * v.get("temporal_patch_size", 2) * v["patch_size"] ** 2
        self.image_token, self.video_token = hf.get("image_token_id"), hf.get("video_token_id")

    def layout(self):
        lay = OrderedDict()
        E, m2 = self.vE, self.merge ** 2
        lay["model.visual.patch_embed.proj.weight"] = (E, self.patch_dim)
        for b in range(self.vL):
            p = f"model.visual.blocks.{b}."
            for n in ("norm1", "norm2"):
                lay[p + n + ".weight"], lay[p + n + ".bias"] = (E,), (E,)
            lay[p + "attn.qkv.weight"], lay[p + "attn.qkv.bias"] = (3 * E, E), (3 * E,)
            lay[p + "attn.proj.weight"], lay[p + "attn.proj.bias"] = (E, E), (E,)
            lay[p + "mlp.fc1.weight"], lay[p + "mlp.fc1.bias"] = (self.vF, E), (self.vF,)
            lay[p + "mlp.fc2.weight"], lay[p + "mlp.fc2.bias"] = (E, self.vF), (E,)
        lay["model.visual.merger.ln_q.weight"], lay["model.visual.merger.ln_q.bias"] = (E,), (E,)
        lay["model.visual.merger.mlp.0.weight"], lay["model.visual.merger.mlp.0.bias"] = (E * m2, E * m2), (E * m2,)
        lay["model.visual.merger.mlp.2.weight"], lay["model.visual.merger.mlp.2.bias"] = (self.H, E * m2), (self.H,)
        lay["model.language_model.embed_tokens.weight"] = (self.V, self.H)
        for l in range(self.L):
            p = f"model.language_model.layers.{l}."
            for n, rows in (("q_proj", self.nh * self.D), ("k_proj", self.nkv * self.D), ("v_proj", self.nkv * self.D)):
                lay[p + f"self_attn.{n}.weight"], lay[p + f"self_attn.{n}.bias"] = (rows, self.H), (rows,)
            lay[p + "self_attn.o_proj.weight"] = (self.H, self.nh * self.D)
            lay[p + "mlp.gate_proj.weight"], lay[p + "mlp.up_proj.weight"] = (self.F, self.H), (self.F, self.H)
            lay[p + "mlp.down_proj.weight"] = (self.H, self.F)
            lay[p + "input_layernorm.weight"], lay[p + "post_attention_layernorm.weight"] = (self.H,), (self.H,)
        lay["model.language_model.norm.weight"] = (self.H,)
        if not self.tied:
            lay["lm_head.weight"] = (self.V, self.H)
        return lay

    def checkpoint_shape(self, name):
        # the checkpoint stores the patch embedding as a Conv3d kernel [E, C, t, p, p]; it is used flattened here
        if name == "model.visual.patch_embed.proj.weight":
            return (self.vE, self.v.get("in_channels", 3), self.v.get("temporal_patch_size", 2), self.v["patch_size"], self.v["patch_size"])
        return None

    def init_kind(self, name):
        if ".norm" in name or "ln_q" in name or name.endswith("layernorm.weight"):
            return "zeros" if name.endswith(".bias") else "ones"
        return super().init_kind(name)

    def P(self, W, l, name):
        return W[f"model.language_model.layers.{l}.{name}"]

    def final_norm(self, W, x):
        return rms_norm(x, W["model.language_model.norm.weight"], self.eps)

    def head_weight(self, W):
        return W["model.language_model.embed_tokens.weight"] if self.tied else W["lm_head.weight"]

    # ---- vision tower
    def vision_rotary(self, grid_thw, device):
        hd = self.vE // self.vH
        inv = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, dtype=torch.float32) / (hd // 2)))      # hd / 4 frequencies
        ms, rows = self.merge, []
        for t, h, w in grid_thw.tolist():
            hi = torch.arange(h)[:, None].expand(h, w).reshape(h // ms, ms, w // ms, ms).permute(0, 2, 1, 3).reshape(-1)
            wi = torch.arange(w)[None, :].expand(h, w).reshape(h // ms, ms, w // ms, ms).permute(0, 2, 1, 3).reshape(-1)
            rows.append(torch.cat([hi[:, None].float() * inv[None], wi[:, None].float() * inv[None]], dim=1).repeat(t, 1))
        ang = torch.cat(rows).to(device)
        ang = torch.cat([ang, ang], dim=1)                                                           # [N, hd]
        return ang.cos(), ang.sin()

    def vision(self, W, patches, grid_thw):
        """[N, patch_dim] patches of all images -> [N / merge^2, H] embeddings in token order."""
        E, Hh = self.vE, self.vH
        hd = E // Hh
        x = linear(patches.to(W["model.visual.patch_embed.proj.weight"].dtype), W["model.visual.patch_embed.proj.weight"])
        cos, sin = self.vision_rotary(grid_thw, x.device)
        segs, a = [], 0
        for t, h, w in grid_thw.tolist():
            for _ in range(int(t)):
                segs.append((a, a + int(h) * int(w)))
                a += int(h) * int(w)
        assert a == x.shape[0], f"{x.shape[0]} patches for grids that describe {a}"
        for b in range(self.vL):
            p = f"model.visual.blocks.{b}."
            h1 = F.layer_norm(x, (E,), W[p + "norm1.weight"], W[p + "norm1.bias"], 1e-6)
            q, k, v = (linear(h1, W[p + "attn.qkv.weight"]) + W[p + "attn.qkv.bias"]).view(-1, 3, Hh, hd).unbind(1)
            q = (q.float() * cos[:, None] + rotate_half(q.float()) * sin[:, None]).to(x.dtype)
            k = (k.float() * cos[:, None] + rotate_half(k.float()) * sin[:, None]).to(x.dtype)
            outs = []
            for s0, s1 in segs:                                 # full attention inside each frame
                o = F.scaled_dot_product_attention(q[s0:s1].transpose(0, 1)[None], k[s0:s1].transpose(0, 1)[None],
                                                   v[s0:s1].transpose(0, 1)[None])
                outs.append(o[0].transpose(0, 1).reshape(s1 - s0, E))
            x = x + linear(torch.cat(outs), W[p + "attn.proj.weight"]) + W[p + "attn.proj.bias"]
            h2 = F.layer_norm(x, (E,), W[p + "norm2.weight"], W[p + "norm2.bias"], 1e-6)
            m = linear(h2, W[p + "mlp.fc1.weight"]) + W[p + "mlp.fc1.bias"]
            x = x + linear(m * torch.sigmoid(1.702 * m), W[p + "mlp.fc2.weight"]) + W[p + "mlp.fc2.bias"]
        x = F.layer_norm(x, (E,), W["model.visual.merger.ln_q.weight"], W["model.visual.merger.ln_q.bias"], 1e-6)
        x = x.view(-1, E * self.merge ** 2)
        x = F.gelu(linear(x, W["model.visual.merger.mlp.0.weight"]) + W["model.visual.merger.mlp.0.bias"])
        return linear(x, W["model.visual.merger.mlp.2.weight"]) + W["model.visual.merger.mlp.2.bias"]

    def embed(self, W, ids, multimodal=None):
        x = W["model.language_model.embed_tokens.weight"][ids]
        if multimodal and multimodal.get("pixel_values") is not None and multimodal["pixel_values"].numel():
            vis = self.vision(W, multimodal["pixel_values"].to(x.device), multimodal["image_grid_thw"]).to(x.dtype)
            where = torch.zeros_like(ids, dtype=torch.bool)
            for tok in (self.image_token, self.video_token):
                if tok is not None:
                    where |= ids == tok
            idx = torch.nonzero(where).flatten()
            assert idx.numel() == vis.shape[0], f"{idx.numel()} placeholder tokens for {vis.shape[0]} vision embeddings"
            x = x.index_copy(0, idx, vis)
        return x

    # ---- decoder
    def rope(self, which):
        return rope_frequencies({"rope_theta": self.rope_params["rope_theta"]}, getattr(self, "rot_dim", self.D),
                                self.hf.get("max_position_embeddings", 32768))

    def rotary(self, ctx):
        pos = ctx["positions"]
        if pos.dim() == 1:                                      # text only: the three rows coincide
            return ctx["model"]._rope("default", pos)
        key = ("mrope", id(pos))
        if ctx.get("_mrope_key") != key:
            from .vision import mrope_tables
            c, s = mrope_tables(pos, getattr(self, "rot_dim", self.D), float(self.rope_params["rope_theta"]), self.sections, device=pos.device,
                                interleaved=getattr(self, "mrope_interleaved", False))
            ctx["_mrope"], ctx["_mrope_key"] = (torch.cat([c, c], -1), torch.cat([s, s], -1)), key
        return ctx["_mrope"]

    def layer(self, W, l, x, ctx):
        T = x.shape[0]
        h = rms_norm(x, self.P(W, l, "input_layernorm.weight"), self.eps)
        cos, sin = self.rotary(ctx)
        q = (linear(h, self.P(W, l, "self_attn.q_proj.weight")) + self.P(W, l, "self_attn.q_proj.bias")).view(T, self.nh, self.D)
        k = (linear(h, self.P(W, l, "self_attn.k_proj.weight")) + self.P(W, l, "self_attn.k_proj.bias")).view(T, self.nkv, self.D)
        v = (linear(h, self.P(W, l, "self_attn.v_proj.weight")) + self.P(W, l, "self_attn.v_proj.bias")).view(T, self.nkv, self.D)
        o = attend(apply_rope(q, cos, sin), apply_rope(k, cos, sin), v, ctx, l, self.D ** -0.5)
        x = x + linear(o.reshape(T, self.nh * self.D), self.P(W, l, "self_attn.o_proj.weight"))
        h = rms_norm(x, self.P(W, l, "post_attention_layernorm.weight"), self.eps)
        return x + linear(F.silu(linear(h, self.P(W, l, "mlp.gate_proj.weight"))) * linear(h, self.P(W, l, "mlp.up_proj.weight")),
                          self.P(W, l, "mlp.down_proj.weight"))


class _Qwen25VL(_Qwen2VL):
    """Qwen2.5-VL: the decoder of Qwen2-VL; the vision tower has RMSNorm, a gated SiLU MLP with biases and WINDOWED
    attention - merge-size units of patches are regrouped window by window (``window_size`` pixels a side), most blocks
    attend inside a window only, the blocks in ``fullatt_block_indexes`` inside a whole frame; the merged embeddings are
    put back into raster order at the end. Reference: axon/models/transformers/qwen2_vl.py (shared forward), HF
    modeling_qwen2_5_vl.py."""

    def __init__(self, hf):
        v = dict(hf["vision_config"])
        v.setdefault("embed_dim", v["hidden_size"])
        hf = {**hf, "vision_config": v}
        super().__init__(hf)
        self.vF = int(v["intermediate_size"])
        self.window = int(v.get("window_size", 112))
        self.full_blocks = set(v.get("fullatt_block_indexes") or [])

    def layout(self):
        lay = OrderedDict()
        E, m2 = self.vE, self.merge ** 2
        lay["model.visual.patch_embed.proj.weight"] = (E, self.patch_dim)
        for b in range(self.vL):
            p = f"model.visual.blocks.{b}."
            lay[p + "norm1.weight"], lay[p + "norm2.weight"] = (E,), (E,)
            lay[p + "attn.qkv.weight"], lay[p + "attn.qkv.bias"] = (3 * E, E), (3 * E,)
            lay[p + "attn.proj.weight"], lay[p + "attn.proj.bias"] = (E, E), (E,)
            for n, (o, i) in (("gate_proj", (self.vF, E)), ("up_proj", (self.vF, E)), ("down_proj", (E, self.vF))):
                lay[p + f"mlp.{n}.weight"], lay[p + f"mlp.{n}.bias"] = (o, i), (o,)
        lay["model.visual.merger.ln_q.weight"] = (E,)
        lay["model.visual.merger.mlp.0.weight"], lay["model.visual.merger.mlp.0.bias"] = (E * m2, E * m2), (E * m2,)
        lay["model.visual.merger.mlp.2.weight"], lay["model.visual.merger.mlp.2.bias"] = (self.H, E * m2), (self.H,)
        text = _Qwen2VL.layout(self)
        for n, sh in text.items():
            if not n.startswith("model.visual."):
                lay[n] = sh
        return lay

    def window_order(self, grid_thw):
        """(order of the merge units window by window, segment boundaries in patches of that order)."""
        ms, unit = self.merge, self.merge ** 2
        side = self.window // ms // self.v["patch_size"]
        order, cu, base = [], [0], 0
        for t, h, w in grid_thw.tolist():
            gh, gw = h // ms, w // ms
            idx = torch.arange(t * gh * gw).reshape(t, gh, gw)
            ph, pw = side - gh % side, side - gw % side
            nh, nw = (gh + ph) // side, (gw + pw) // side
            pad = F.pad(idx, (0, pw, 0, ph), value=-1).reshape(t, nh, side, nw, side).permute(0, 1, 3, 2, 4).reshape(t, nh * nw, side, side)
            counts = (pad >= 0).sum((2, 3)).reshape(-1)
            flat = pad.reshape(-1)
            order.append(flat[flat >= 0] + base)
            for c in counts.tolist():
                if c:
                    cu.append(cu[-1] + c * unit)
            base += t * gh * gw
        return torch.cat(order), cu

    def vision(self, W, patches, grid_thw):
        E, Hh, unit = self.vE, self.vH, self.merge ** 2
        hd = E // Hh
        x = linear(patches.to(W["model.visual.patch_embed.proj.weight"].dtype), W["model.visual.patch_embed.proj.weight"])
        cos, sin = self.vision_rotary(grid_thw, x.device)
        order, cu_win = self.window_order(grid_thw)
        order = order.to(x.device)
        N = x.shape[0]
        regroup = lambda t: t.reshape(N // unit, unit, -1)[order].reshape(N, -1)      # noqa: E731
        x, cos, sin = regroup(x), regroup(cos), regroup(sin)
        frames, a = [], 0
        for t, h, w in grid_thw.tolist():
            for _ in range(int(t)):
                frames.append((a, a + int(h) * int(w)))
                a += int(h) * int(w)
        assert a == N, f"{N} patches for grids that describe {a}"
        windows = list(zip(cu_win[:-1], cu_win[1:]))
        for b in range(self.vL):
            p = f"model.visual.blocks.{b}."
            h1 = rms_norm(x, W[p + "norm1.weight"], 1e-6)
            q, k, v = (linear(h1, W[p + "attn.qkv.weight"]) + W[p + "attn.qkv.bias"]).view(-1, 3, Hh, hd).unbind(1)
            q = (q.float() * cos[:, None] + rotate_half(q.float()) * sin[:, None]).to(x.dtype)
            k = (k.float() * cos[:, None] + rotate_half(k.float()) * sin[:, None]).to(x.dtype)
            outs = []
            for s0, s1 in (frames if b in self.full_blocks else windows):
                o = F.scaled_dot_product_attention(q[s0:s1].transpose(0, 1)[None], k[s0:s1].transpose(0, 1)[None],
                                                   v[s0:s1].transpose(0, 1)[None])
                outs.append(o[0].transpose(0, 1).reshape(s1 - s0, E))
            x = x + linear(torch.cat(outs), W[p + "attn.proj.weight"]) + W[p + "attn.proj.bias"]
            h2 = rms_norm(x, W[p + "norm2.weight"], 1e-6)
            g = linear(h2, W[p + "mlp.gate_proj.weight"]) + W[p + "mlp.gate_proj.bias"]
            u = linear(h2, W[p + "mlp.up_proj.weight"]) + W[p + "mlp.up_proj.bias"]
            x = x + linear(F.silu(g) * u, W[p + "mlp.down_proj.weight"]) + W[p + "mlp.down_proj.bias"]
        x = rms_norm(x, W["model.visual.merger.ln_q.weight"], 1e-6).view(-1, E * unit)
        x = F.gelu(linear(x, W["model.visual.merger.mlp.0.weight"]) + W["model.visual.merger.mlp.0.bias"])
        x = linear(x, W["model.visual.merger.mlp.2.weight"]) + W["model.visual.merger.mlp.2.bias"]
        return x[torch.argsort(order)]


class _Qwen3VL(_Qwen2VL):
    """Qwen3-VL: a Qwen3 decoder (no projection biases, RMSNorm on every query / key head before the rotation) with
    INTERLEAVED three-row rotary positions; the vision tower adds bilinearly interpolated learned position embeddings
    to the patches, uses LayerNorm blocks with a tanh-GELU MLP, and besides the final merger taps the outputs of the
    blocks in ``deepstack_visual_indexes``: each tap is merged (LayerNorm AFTER grouping merge^2 patches) and ADDED to
    the decoder's hidden states at the image tokens after decoder layer 0, 1, ... ("DeepStack"). Reference: HF
    modeling_qwen3_vl.py; the reference patches this family in axon/models/transformers/qwen3_vl.py."""
    mrope_interleaved = True

    def __init__(self, hf):
        v = dict(hf["vision_config"])
        v.setdefault("embed_dim", v["hidden_size"])
        v.setdefault("mlp_ratio", v["intermediate_size"] / v["hidden_size"])
        hf = {**hf, "vision_config": v}
        super().__init__(hf)
        self.vF = int(v["intermediate_size"])
        self.taps = list(v.get("deepstack_visual_indexes") or [])
        self.grid_side = int(round(v["num_position_embeddings"] ** 0.5))
        self._deepstack, self._visual_idx = None, None

    def layout(self):
        lay = OrderedDict()
        E, m2 = self.vE, self.merge ** 2
        lay["model.visual.patch_embed.proj.weight"], lay["model.visual.patch_embed.proj.bias"] = (E, self.patch_dim), (E,)
        lay["model.visual.pos_embed.weight"] = (self.grid_side ** 2, E)
        for b in range(self.vL):
            p = f"model.visual.blocks.{b}."
            for n in ("norm1", "norm2"):
                lay[p + n + ".weight"], lay[p + n + ".bias"] = (E,), (E,)
            lay[p + "attn.qkv.weight"], lay[p + "attn.qkv.bias"] = (3 * E, E), (3 * E,)
            lay[p + "attn.proj.weight"], lay[p + "attn.proj.bias"] = (E, E), (E,)
            lay[p + "mlp.linear_fc1.weight"], lay[p + "mlp.linear_fc1.bias"] = (self.vF, E), (self.vF,)
            lay[p + "mlp.linear_fc2.weight"], lay[p + "mlp.linear_fc2.bias"] = (E, self.vF), (E,)
        for p, nd in [("model.visual.merger.", E)] + [(f"model.visual.deepstack_merger_list.{i}.", E * m2) for i in range(len(self.taps))]:
            lay[p + "norm.weight"], lay[p + "norm.bias"] = (nd,), (nd,)
            lay[p + "linear_fc1.weight"], lay[p + "linear_fc1.bias"] = (E * m2, E * m2), (E * m2,)
            lay[p + "linear_fc2.weight"], lay[p + "linear_fc2.bias"] = (self.H, E * m2), (self.H,)
        lay["model.language_model.embed_tokens.weight"] = (self.V, self.H)
        for l in range(self.L):
            p = f"model.language_model.layers.{l}."
            for n, rows in (("q_proj", self.nh * self.D), ("k_proj", self.nkv * self.D), ("v_proj", self.nkv * self.D)):
                lay[p + f"self_attn.{n}.weight"] = (rows, self.H)
            lay[p + "self_attn.o_proj.weight"] = (self.H, self.nh * self.D)
            lay[p + "self_attn.q_norm.weight"], lay[p + "self_attn.k_norm.weight"] = (self.D,), (self.D,)
            lay[p + "mlp.gate_proj.weight"], lay[p + "mlp.up_proj.weight"] = (self.F, self.H), (self.F, self.H)
            lay[p + "mlp.down_proj.weight"] = (self.H, self.F)
            lay[p + "input_layernorm.weight"], lay[p + "post_attention_layernorm.weight"] = (self.H,), (self.H,)
        lay["model.language_model.norm.weight"] = (self.H,)
        if not self.tied:
            lay["lm_head.weight"] = (self.V, self.H)
        return lay

    def init_kind(self, name):
        if name.endswith(("q_norm.weight", "k_norm.weight")) or ".norm." in name:
            return "zeros" if name.endswith(".bias") else "ones"
        return super().init_kind(name)

    def position_embeddings(self, W, grid_thw):
        """Learned [side x side] table sampled bilinearly at every patch of every grid, in merge-window order."""
        table, side, ms = W["model.visual.pos_embed.weight"], self.grid_side, self.merge
        outs = []
        for t, h, w in grid_thw.tolist():
            hs, ws = torch.linspace(0, side - 1, h), torch.linspace(0, side - 1, w)
            h0, w0 = hs.int(), ws.int()
            h1, w1 = (h0 + 1).clip(max=side - 1), (w0 + 1).clip(max=side - 1)
            dh, dw = (hs - h0).to(table.dtype), (ws - w0).to(table.dtype)
            pe = 0
            for hi, wi, wt in ((h0, w0, (1 - dh)[:, None] * (1 - dw)[None]), (h0, w1, (1 - dh)[:, None] * dw[None]),
                               (h1, w0, dh[:, None] * (1 - dw)[None]), (h1, w1, dh[:, None] * dw[None])):
                idx = (hi.long()[:, None] * side + wi.long()[None]).reshape(-1).to(table.device)
                pe = pe + table[idx] * wt.reshape(-1, 1).to(table.device)
            pe = pe.repeat(int(t), 1).view(int(t), h // ms, ms, w // ms, ms, -1).permute(0, 1, 3, 2, 4, 5).reshape(int(t) * h * w, -1)
            outs.append(pe)
        return torch.cat(outs)

    def _merge(self, W, p, x, after_grouping: bool):
        E, m2 = self.vE, self.merge ** 2
        if after_grouping:
            x = F.layer_norm(x.view(-1, E * m2), (E * m2,), W[p + "norm.weight"], W[p + "norm.bias"], 1e-6)
        else:
            x = F.layer_norm(x, (E,), W[p + "norm.weight"], W[p + "norm.bias"], 1e-6).view(-1, E * m2)
        x = F.gelu(linear(x, W[p + "linear_fc1.weight"]) + W[p + "linear_fc1.bias"])
        return linear(x, W[p + "linear_fc2.weight"]) + W[p + "linear_fc2.bias"]

    def vision(self, W, patches, grid_thw):
        """-> (embeddings for the placeholder tokens [N / merge^2, H], list of DeepStack features of the same shape)."""
        E, Hh = self.vE, self.vH
        hd = E // Hh
        x = linear(patches.to(W["model.visual.patch_embed.proj.weight"].dtype), W["model.visual.patch_embed.proj.weight"]) \
            + W["model.visual.patch_embed.proj.bias"]
        x = x + self.position_embeddings(W, grid_thw).to(x.dtype)
        cos, sin = self.vision_rotary(grid_thw, x.device)
        segs, a = [], 0
        for t, h, w in grid_thw.tolist():
            for _ in range(int(t)):
                segs.append((a, a + int(h) * int(w)))
                a += int(h) * int(w)
        assert a == x.shape[0], f"{x.shape[0]} patches for grids that describe {a}"
        taps = []
        for b in range(self.vL):
            p = f"model.visual.blocks.{b}."
            h1 = F.layer_norm(x, (E,), W[p + "norm1.weight"], W[p + "norm1.bias"], 1e-6)
            q, k, v = (linear(h1, W[p + "attn.qkv.weight"]) + W[p + "attn.qkv.bias"]).view(-1, 3, Hh, hd).unbind(1)
            q = (q.float() * cos[:, None] + rotate_half(q.float()) * sin[:, None]).to(x.dtype)
            k = (k.float() * cos[:, None] + rotate_half(k.float()) * sin[:, None]).to(x.dtype)
            outs = []
            for s0, s1 in segs:
                o = F.scaled_dot_product_attention(q[s0:s1].transpose(0, 1)[None], k[s0:s1].transpose(0, 1)[None],
                                                   v[s0:s1].transpose(0, 1)[None])
                outs.append(o[0].transpose(0, 1).reshape(s1 - s0, E))
            x = x + linear(torch.cat(outs), W[p + "attn.proj.weight"]) + W[p + "attn.proj.bias"]
            h2 = F.layer_norm(x, (E,), W[p + "norm2.weight"], W[p + "norm2.bias"], 1e-6)
            m = F.gelu(linear(h2, W[p + "mlp.linear_fc1.weight"]) + W[p + "mlp.linear_fc1.bias"], approximate="tanh")
            x = x + linear(m, W[p + "mlp.linear_fc2.weight"]) + W[p + "mlp.linear_fc2.bias"]
            if b in self.taps:
                taps.append(self._merge(W, f"model.visual.deepstack_merger_list.{self.taps.index(b)}.", x, after_grouping=True))
        return self._merge(W, "model.visual.merger.", x, after_grouping=False), taps

    def embed(self, W, ids, multimodal=None):
        x = W["model.language_model.embed_tokens.weight"][ids]
        self._deepstack, self._visual_idx = None, None
        if multimodal and multimodal.get("pixel_values") is not None and multimodal["pixel_values"].numel():
            vis, taps = self.vision(W, multimodal["pixel_values"].to(x.device), multimodal["image_grid_thw"])
            where = torch.zeros_like(ids, dtype=torch.bool)
            for tok in (self.image_token, self.video_token):
                if tok is not None:
                    where |= ids == tok
            idx = torch.nonzero(where).flatten()
            assert idx.numel() == vis.shape[0], f"{idx.numel()} placeholder tokens for {vis.shape[0]} vision embeddings"
            x = x.index_copy(0, idx, vis.to(x.dtype))
            self._deepstack, self._visual_idx = [t.to(x.dtype) for t in taps], idx
        return x

    def layer(self, W, l, x, ctx):
        T = x.shape[0]
        h = rms_norm(x, self.P(W, l, "input_layernorm.weight"), self.eps)
        cos, sin = self.rotary(ctx)
        q = rms_norm(linear(h, self.P(W, l, "self_attn.q_proj.weight")).view(T, self.nh, self.D), self.P(W, l, "self_attn.q_norm.weight"), self.eps)
        k = rms_norm(linear(h, self.P(W, l, "self_attn.k_proj.weight")).view(T, self.nkv, self.D), self.P(W, l, "self_attn.k_norm.weight"), self.eps)
        v = linear(h, self.P(W, l, "self_attn.v_proj.weight")).view(T, self.nkv, self.D)
        o = attend(apply_rope(q, cos, sin), apply_rope(k, cos, sin), v, ctx, l, self.D ** -0.5)
        x = x + linear(o.reshape(T, self.nh * self.D), self.P(W, l, "self_attn.o_proj.weight"))
        x = x + self.mlp(W, l, rms_norm(x, self.P(W, l, "post_attention_layernorm.weight"), self.eps))
        if self._deepstack is not None and l < len(self._deepstack):
            x = x.index_add(0, self._visual_idx, self._deepstack[l])
        return x

    def mlp(self, W, l, h):
        return linear(F.silu(linear(h, self.P(W, l, "mlp.gate_proj.weight"))) * linear(h, self.P(W, l, "mlp.up_proj.weight")),
                      self.P(W, l, "mlp.down_proj.weight"))


class _Qwen3VLMoe(_Qwen3VL):
    """Qwen3-VL with a sparse decoder: the layers named by ``decoder_sparse_step`` / ``mlp_only_layers`` replace the
    MLP with top-k softmax routing (weights renormalised over the chosen experts) over stacked SwiGLU experts.
    Reference: axon/models/transformers/qwen3_vl.py (its patch of the sparse block), HF modeling_qwen3_vl_moe.py."""

    def __init__(self, hf):
        super().__init__(hf)
        self.E, self.k, self.Fm = int(hf.get("num_experts") or hf["num_local_experts"]), int(hf["num_experts_per_tok"]), int(hf["moe_intermediate_size"])
        step, dense_only = int(hf.get("decoder_sparse_step", 1) or 1), set(hf.get("mlp_only_layers") or [])
        self.sparse = [l not in dense_only and self.E > 0 and (l + 1) % step == 0 for l in range(self.L)]

    def layout(self):
        lay = OrderedDict()
        for name, shape in super().layout().items():
            m = re.match(r"model\.language_model\.layers\.(\d+)\.mlp\.(gate_proj|up_proj|down_proj)\.weight", name)
            if m and self.sparse[int(m.group(1))]:
                if m.group(2) == "gate_proj":
                    p = f"model.language_model.layers.{m.group(1)}.mlp."
                    lay[p + "experts.gate_up_proj"], lay[p + "experts.down_proj"] = (self.E, 2 * self.Fm, self.H), (self.E, self.H, self.Fm)
                    lay[p + "gate.weight"] = (self.E, self.H)
                continue
            lay[name] = shape
        return lay

    def mlp(self, W, l, h):
        if not self.sparse[l]:
            return super().mlp(W, l, h)
        probs = torch.softmax(F.linear(h, self.P(W, l, "mlp.gate.weight")), dim=-1, dtype=torch.float)
        w, idx = probs.topk(self.k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        gu, dn = self.P(W, l, "mlp.experts.gate_up_proj"), self.P(W, l, "mlp.experts.down_proj")

        def expert(e, rows):
            g, u = F.linear(rows, gu[e]).chunk(2, dim=-1)
            return F.linear(F.silu(g) * u, dn[e])
        return experts_forward(h, idx, w.to(h.dtype), expert, self.E)


class _Glm4V(_Qwen2VL):
    """GLM-4.1V: a GLM-4 decoder (q / k / v biases, fused gate|up, an extra RMSNorm on the attention and on the MLP
    output before each residual add, rotary angles from three position rows applied to interleaved pairs of the first
    ``partial_rotary_factor`` share of a head) fed by a vision tower of RMSNorm blocks with SwiGLU MLPs: patch
    embedding (with bias) - RMSNorm - a learned position table sampled bicubically at every patch's place in its
    image - blocks with 2-D rotary attention inside each frame - RMSNorm - a merge x merge strided convolution over
    each window - a merger (linear, LayerNorm, GELU, SwiGLU). Reference: axon/models/transformers/glm4v.py
    (packed forward of the HF model), HF modeling_glm4v.py."""

    def __init__(self, hf):
        v = dict(hf["vision_config"])
        v.setdefault("embed_dim", v["hidden_size"])
        hf = {**hf, "vision_config": v}
        super().__init__(hf)
        self.rot_dim = int(self.D * float(self.rope_params.get("partial_rotary_factor", hf.get("partial_rotary_factor", 1.0)))) // 2 * 2
        self.sections = list(self.rope_params.get("mrope_section") or [self.rot_dim // 2, 0, 0])
        self.vOut, self.vCtx = int(v["out_hidden_size"]), int(v["intermediate_size"])
        self.v_eps = float(v.get("rms_norm_eps", 1e-5))
        self.grid_side = int(v["image_size"]) // int(v["patch_size"])

    def layout(self):
        lay = OrderedDict()
        E, m, O = self.vE, self.merge, self.vOut
        lay["model.visual.embeddings.position_embedding.weight"] = (self.grid_side ** 2, E)
        lay["model.visual.patch_embed.proj.weight"], lay["model.visual.patch_embed.proj.bias"] = (E, self.patch_dim), (E,)
        for b in range(self.vL):
            p = f"model.visual.blocks.{b}."
            lay[p + "norm1.weight"], lay[p + "norm2.weight"] = (E,), (E,)
            lay[p + "attn.qkv.weight"], lay[p + "attn.proj.weight"] = (3 * E, E), (E, E)
            lay[p + "mlp.gate_proj.weight"], lay[p + "mlp.up_proj.weight"], lay[p + "mlp.down_proj.weight"] = (O, E), (O, E), (E, O)
        lay["model.visual.merger.proj.weight"] = (O, O)
        lay["model.visual.merger.post_projection_norm.weight"], lay["model.visual.merger.post_projection_norm.bias"] = (O,), (O,)
        lay["model.visual.merger.gate_proj.weight"], lay["model.visual.merger.up_proj.weight"] = (self.vCtx, O), (self.vCtx, O)
        lay["model.visual.merger.down_proj.weight"] = (O, self.vCtx)
        lay["model.visual.post_conv_layernorm.weight"] = (E,)
        lay["model.visual.downsample.weight"], lay["model.visual.downsample.bias"] = (O, E * m * m), (O,)
        lay["model.visual.post_layernorm.weight"] = (E,)
        lay["model.language_model.embed_tokens.weight"] = (self.V, self.H)
        for l in range(self.L):
            p = f"model.language_model.layers.{l}."
            for n, rows in (("q_proj", self.nh * self.D), ("k_proj", self.nkv * self.D), ("v_proj", self.nkv * self.D)):
                lay[p + f"self_attn.{n}.weight"], lay[p + f"self_attn.{n}.bias"] = (rows, self.H), (rows,)
            lay[p + "self_attn.o_proj.weight"] = (self.H, self.nh * self.D)
            lay[p + "mlp.gate_up_proj.weight"], lay[p + "mlp.down_proj.weight"] = (2 * self.F, self.H), (self.H, self.F)
            for n in ("input_layernorm", "post_attention_layernorm", "post_self_attn_layernorm", "post_mlp_layernorm"):
                lay[p + n + ".weight"] = (self.H,)
        lay["model.language_model.norm.weight"] = (self.H,)
        if not self.tied:
            lay["lm_head.weight"] = (self.V, self.H)
        return lay

    def checkpoint_shape(self, name):
        if name == "model.visual.downsample.weight":         # a Conv2d kernel [out, E, merge, merge] in the checkpoint
            return (self.vOut, self.vE, self.merge, self.merge)
        return super().checkpoint_shape(name)

    def init_kind(self, name):
        if "post_projection_norm" in name or name.endswith(("post_conv_layernorm.weight", "post_layernorm.weight")):
            return "zeros" if name.endswith(".bias") else "ones"
        return super().init_kind(name)

    def patch_places(self, grid_thw):
        """(row, column, image height, image width) of every patch, in merge-window order."""
        ms, hs, ws, th, tw = self.merge, [], [], [], []
        for t, h, w in grid_thw.tolist():
            hi = torch.arange(h)[:, None].expand(h, w).reshape(h // ms, ms, w // ms, ms).permute(0, 2, 1, 3).reshape(-1).repeat(t)
            wi = torch.arange(w)[None, :].expand(h, w).reshape(h // ms, ms, w // ms, ms).permute(0, 2, 1, 3).reshape(-1).repeat(t)
            hs.append(hi), ws.append(wi), th.append(torch.full_like(hi, h)), tw.append(torch.full_like(wi, w))
        return torch.cat(hs).float(), torch.cat(ws).float(), torch.cat(th).float(), torch.cat(tw).float()

    def vision(self, W, patches, grid_thw):
        E, Hh, m = self.vE, self.vH, self.merge
        hd = E // Hh
        x = linear(patches.to(W["model.visual.patch_embed.proj.weight"].dtype), W["model.visual.patch_embed.proj.weight"]) \
            + W["model.visual.patch_embed.proj.bias"]
        x = rms_norm(x, W["model.visual.post_conv_layernorm.weight"], self.v_eps)
        # the position table as a [side x side] image, sampled bicubically at each patch's centre
        hi, wi, th, tw = (t.to(x.device) for t in self.patch_places(grid_thw))
        table = W["model.visual.embeddings.position_embedding.weight"].float().view(self.grid_side, self.grid_side, E).permute(2, 0, 1)[None]
        grid = torch.stack(((wi + 0.5) / tw * 2 - 1, (hi + 0.5) / th * 2 - 1), dim=-1)[None, :, None, :]
        pe = F.grid_sample(table, grid, mode="bicubic", align_corners=False, padding_mode="border")[0, :, :, 0].t()
        x = x + pe.to(x.dtype)
        cos, sin = self.vision_rotary(grid_thw, x.device)
        segs, a = [], 0
        for t, h, w in grid_thw.tolist():
            for _ in range(int(t)):
                segs.append((a, a + int(h) * int(w)))
                a += int(h) * int(w)
        assert a == x.shape[0], f"{x.shape[0]} patches for grids that describe {a}"
        for b in range(self.vL):
            p = f"model.visual.blocks.{b}."
            h1 = rms_norm(x, W[p + "norm1.weight"], self.v_eps)
            q, k, v = linear(h1, W[p + "attn.qkv.weight"]).view(-1, 3, Hh, hd).unbind(1)
            q = (q.float() * cos[:, None] + rotate_half(q.float()) * sin[:, None]).to(x.dtype)
            k = (k.float() * cos[:, None] + rotate_half(k.float()) * sin[:, None]).to(x.dtype)
            outs = []
            for s0, s1 in segs:
                o = F.scaled_dot_product_attention(q[s0:s1].transpose(0, 1)[None], k[s0:s1].transpose(0, 1)[None],
                                                   v[s0:s1].transpose(0, 1)[None])
                outs.append(o[0].transpose(0, 1).reshape(s1 - s0, E))
            x = x + linear(torch.cat(outs), W[p + "attn.proj.weight"])
            h2 = rms_norm(x, W[p + "norm2.weight"], self.v_eps)
            x = x + linear(F.silu(linear(h2, W[p + "mlp.gate_proj.weight"])) * linear(h2, W[p + "mlp.up_proj.weight"]), W[p + "mlp.down_proj.weight"])
        x = rms_norm(x, W["model.visual.post_layernorm.weight"], self.v_eps)
        x = x.view(-1, m * m, E).transpose(1, 2).reshape(-1, E * m * m)          # each window in the kernel's (channel, row, column) order
        x = linear(x, W["model.visual.downsample.weight"]) + W["model.visual.downsample.bias"]
        x = linear(x, W["model.visual.merger.proj.weight"])
        x = F.gelu(F.layer_norm(x, (self.vOut,), W["model.visual.merger.post_projection_norm.weight"],
                                W["model.visual.merger.post_projection_norm.bias"], 1e-5))
        return linear(F.silu(linear(x, W["model.visual.merger.gate_proj.weight"])) * linear(x, W["model.visual.merger.up_proj.weight"]),
                      W["model.visual.merger.down_proj.weight"])

    def layer(self, W, l, x, ctx):
        T = x.shape[0]
        h = rms_norm(x, self.P(W, l, "input_layernorm.weight"), self.eps)
        cos, sin = self.rotary(ctx)
        q = (linear(h, self.P(W, l, "self_attn.q_proj.weight")) + self.P(W, l, "self_attn.q_proj.bias")).view(T, self.nh, self.D)
        k = (linear(h, self.P(W, l, "self_attn.k_proj.weight")) + self.P(W, l, "self_attn.k_proj.bias")).view(T, self.nkv, self.D)
        v = (linear(h, self.P(W, l, "self_attn.v_proj.weight")) + self.P(W, l, "self_attn.v_proj.bias")).view(T, self.nkv, self.D)
        o = attend(apply_rope(q, cos, sin, interleaved=True), apply_rope(k, cos, sin, interleaved=True), v, ctx, l, self.D ** -0.5)
        a = linear(o.reshape(T, self.nh * self.D), self.P(W, l, "self_attn.o_proj.weight"))
        x = x + rms_norm(a, self.P(W, l, "post_self_attn_layernorm.weight"), self.eps)
        h = rms_norm(x, self.P(W, l, "post_attention_layernorm.weight"), self.eps)
        gate, up = linear(h, self.P(W, l, "mlp.gate_up_proj.weight")).chunk(2, dim=-1)
        mo = linear(F.silu(gate) * up, self.P(W, l, "mlp.down_proj.weight"))
        return x + rms_norm(mo, self.P(W, l, "post_mlp_layernorm.weight"), self.eps)


_SPECS = {"qwen2_vl": _Qwen2VL, "qwen2_5_vl": _Qwen25VL, "qwen3_vl": _Qwen3VL, "qwen3_vl_moe": _Qwen3VLMoe, "glm4v": _Glm4V, "deepseek_v3": _DeepseekV3, "glm4_moe_lite": _DeepseekV3, "glm_moe_dsa": _GlmMoeDsa, "gemma4_text": _Gemma4, "glm4_moe": _Glm4Moe, "gpt_oss": _GptOss,
          "gemma2": _Gemma, "gemma3_text": _Gemma, "qwen3_next": _Qwen3Next, "qwen3_5_text": _Qwen35, "qwen3_5_moe_text": _Qwen35}


# ------------------------------------------------------------------------------------------ construction
def family_config(hf: dict) -> ModelConfig:
    """The ``ModelConfig`` view of a family's HF config: the fields the engines read (cache geometry, vocabulary,
    special tokens); everything else stays in ``extra['hf_config']`` for the family's spec."""
    mt = hf["model_type"]
    if mt in TEXT_ONLY_OF and "text_config" in hf:
        # the decoder of a multimodal checkpoint: its own configuration (special tokens of the wrapper are kept when it has none)
        text = dict(hf["text_config"])
        for k in ("eos_token_id", "pad_token_id", "bos_token_id", "tie_word_embeddings"):
            if text.get(k) is None and hf.get(k) is not None:
                text[k] = hf[k]
        text["model_type"] = mt = TEXT_ONLY_OF[mt]
        hf = text
    if mt in VISION_LANGUAGE_TYPES and "text_config" in hf:
        # vision-language checkpoints nest the decoder's fields: lift them, keep the nested form for export
        nested = dict(hf)
        hf = {**{k: v for k, v in hf["text_config"].items() if k != "model_type"}, **{k: v for k, v in hf.items() if k != "text_config"}}
        hf["_nested_config"] = nested
    nh = hf["num_attention_heads"]
    if mt in ("deepseek_v3", "glm4_moe_lite", "glm_moe_dsa"):
        # the paged cache holds expanded keys (nope + rope) and values per head
        nkv, hd = nh, max(hf["qk_nope_head_dim"] + hf["qk_rope_head_dim"], hf["v_head_dim"])
    elif mt == "gemma4_text":            # the pool is sized for the wider of the two layer kinds
        nkv = max(hf.get("num_key_value_heads", nh), hf.get("num_global_key_value_heads") or 0)
        hd = max(hf["head_dim"], hf.get("global_head_dim") or 0)
    else:
        nkv = hf.get("num_key_value_heads", nh)
        hd = hf.get("head_dim") or hf["hidden_size"] // nh
    eos = hf.get("eos_token_id", 1)
    eos = eos[0] if isinstance(eos, list) else eos
    cfg = ModelConfig(model_type=mt, vocab_size=hf["vocab_size"], hidden_size=hf["hidden_size"],
                      num_hidden_layers=hf["num_hidden_layers"], num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd,
                      intermediate_size=hf.get("intermediate_size", 0), rms_norm_eps=hf.get("rms_norm_eps", 1e-6),
                      tie_word_embeddings=bool(hf.get("tie_word_embeddings", mt.startswith("gemma"))),
                      max_position_embeddings=hf.get("max_position_embeddings", 4096), eos_token_id=eos if eos is not None else 1,
                      pad_token_id=hf.get("pad_token_id") if hf.get("pad_token_id") is not None else 0,
                      num_experts=hf.get("n_routed_experts") or hf.get("num_local_experts") or hf.get("num_experts") or 0,
                      num_experts_per_tok=hf.get("num_experts_per_tok", 0) or 0, moe_intermediate_size=hf.get("moe_intermediate_size", 0) or 0)
    cfg.extra["hf_config"] = dict(hf)
    return cfg


def build_family_model(hf: dict, device="cuda", dtype=torch.bfloat16) -> FamilyModel:
    return FamilyModel(family_config(hf), device=device, dtype=dtype, hf=hf)
