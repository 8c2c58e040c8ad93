"""Dense decoder (Qwen3 / Llama-3 style) with an explicit forward and backward over packed
sequences.

The backward pass is hand-scheduled instead of recorded by autograd: every layer keeps only its
input residual stream, recomputes its activations when its backward runs, and accumulates weight
gradients straight into the flat fp32 main-gradient buffer inside the wgrad GEMM epilogue. All
heavy ops are the native sm_100a kernels of ``axon_b200.ops`` (tcgen05 GEMM / attention /
fused vocabulary head); the same calls run PyTorch fp32 math on CPU tensors, which is both the
test oracle and the CPU/gloo configuration.

Plays the role of the HF model + ``fsdp_model_forward`` in the reference
(axon/utils/fsdp/forward_utils.py:185-318): packed (remove-padding) inputs, fused head that
returns per-token log-probs and entropy without materialising logits.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import activation as A
from ..ops import attention as AT
from ..ops import gemm as G
from ..ops import lm_head as LM
from ..ops import norm as N
from ..ops import rope as R
from .config import ModelConfig
from .params import FlatParams


@dataclass
class PackedBatch:
    """Packed (padding-free) token batch. labels[t] is the next token inside the same sequence, -100 at
    the last position of each sequence, so ``head(t)`` scores token t+1."""
    input_ids: torch.Tensor      # int32 [T]
    position_ids: torch.Tensor   # int32 [T]
    cu_seqlens: torch.Tensor     # int32 [B+1]
    labels: torch.Tensor         # int32 [T]
    max_seqlen: int = 0
    routermap: torch.Tensor | None = None   # int [T, n_moe_layers, top_k] expert ids chosen by the sampler (-1: none)
    # vision-language models: pixel_values [patches, patch_dim], image_grid_thw [images, 3], mrope_positions [3, T]
    multimodal: dict | None = None

    @staticmethod
    def from_sequences(seqs: list[torch.Tensor], device) -> "PackedBatch":
        lens = [int(s.numel()) for s in seqs]
        ids = torch.cat([s.to(torch.int32) for s in seqs])
        pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens])
        labels = torch.cat([torch.cat([s[1:].to(torch.int32), torch.tensor([-100], dtype=torch.int32)]) for s in seqs])
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()), dtype=torch.int32)
        return PackedBatch(ids.to(device), pos.to(device), cu.to(device), labels.to(device), max(lens))


def _cached_prefill_plan(batch: "PackedBatch", past_lens, block_table, tok_seq, device) -> dict:
    """Index tensors for attention over [cached prefix | new tokens] of every sequence: where the new rows and the
    prefix rows sit in the packed full-length row set, and which (page, slot) of the cache each prefix row comes from."""
    import numpy as np
    cu = batch.cu_seqlens.tolist()
    rows_of = tok_seq[torch.tensor(cu[:-1], dtype=torch.long, device=tok_seq.device)].tolist() if len(cu) > 1 else []
    bt = block_table.cpu().numpy()
    new_rows, pre_rows, pre_page, pre_slot, cu_full = [], [], [], [], [0]
    off = 0
    for i, past in enumerate(int(p) for p in past_lens):
        n_new = cu[i + 1] - cu[i]
        pre_rows.append(np.arange(off, off + past))
        pos = np.arange(past)
        pre_page.append(bt[rows_of[i], pos // 128])
        pre_slot.append(pos % 128)
        new_rows.append(np.arange(off + past, off + past + n_new))
        off += past + n_new
        cu_full.append(off)
    t = lambda a, dt=torch.long: torch.from_numpy(np.concatenate(a).astype(np.int64)).to(device=device, dtype=dt)      # noqa: E731
    return dict(T_full=off, new_rows=t(new_rows), pre_rows=t(pre_rows), pre_page=t(pre_page), pre_slot=t(pre_slot),
                cu_full=torch.tensor(cu_full, dtype=torch.int32, device=device))


class DenseModel:
    def __init__(self, cfg: ModelConfig, device="cuda", dtype=torch.bfloat16, params: FlatParams | None = None):
        assert cfg.num_experts == 0 or type(self) is not DenseModel, "use MoEModel for sparse configs"
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype
        self.params = params if params is not None else FlatParams(cfg, self.device, dtype)
        self._saved: dict | None = None
        self.recompute = "selective"          # activation recomputation in backward: full | selective | none
        self.offloader = None                 # an ActivationOffloader: kept activations wait in pinned host memory
        self.mtp_scale = 0.0                  # weight of sum_t(-logprob) of the multi-token-prediction module in backward (0 = module idle)
        self.mtp_last = None

    # ------------------------------------------------------------------ helpers
    # ``weights`` is what the forward pass reads and ``_wgrad`` where weight gradients go; both are the
    # trainable ``params`` here. A model with frozen base weights (adapters) overrides them.
    @property
    def weights(self) -> FlatParams:
        return self.params

    def _wgrad(self, name: str):
        return self.params.grads[name]

    def _p(self, l: int, name: str) -> torch.Tensor:
        return self.weights[f"model.layers.{l}.{name}"]

    def _g(self, l: int, name: str) -> torch.Tensor:
        return self._wgrad(f"model.layers.{l}.{name}")

    def head_weight(self) -> torch.Tensor:
        return self.weights["model.embed_tokens.weight" if self.cfg.tie_word_embeddings else "lm_head.weight"]

    def head_grad(self) -> torch.Tensor:
        return self._wgrad("model.embed_tokens.weight" if self.cfg.tie_word_embeddings else "lm_head.weight")

    def _lin(self, l: int, name: str, x: torch.Tensor) -> torch.Tensor:
        """y = x W^T (+ bias) for the layer's linear ``name`` (adapter models add their low-rank path here)."""
        return self._bias_fwd(l, name, G.gemm_nt(x, self._p(l, name)))

    def _lin_bwd(self, l: int, name: str, dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        """Input gradient of ``_lin``; accumulates the weight (and bias) gradient."""
        dx = G.gemm_nn(dy, self._p(l, name))
        G.gemm_tn(dy, x, out=self._g(l, name), accumulate=True)
        self._bias_bwd(l, name, dy)
        return dx

    def _has_bias(self, name: str) -> bool:
        return self.cfg.attention_bias and name == "self_attn.qkv_proj.weight"

    def _bias_fwd(self, l: int, name: str, y: torch.Tensor) -> torch.Tensor:
        if self._has_bias(name):
            y += self._p(l, name[:-len("weight")] + "bias")
        return y

    def _bias_bwd(self, l: int, name: str, dy: torch.Tensor) -> None:
        if self._has_bias(name):
            g = self._g(l, name[:-len("weight")] + "bias")
            if g is not None:                       # frozen-base models hand out no matrix / bias gradients
                g += dy.float().sum(0)

    def _attn_fwd(self, qkv_r: torch.Tensor, batch: "PackedBatch", need_lse: bool):
        """Causal attention over the packed sequences: qkv_r [T, (Hq + 2 Hkv) D] (rotated) -> (o [T, Hq D], lse).
        Sequence-parallel models override this pair with the head <-> token exchange around the kernel."""
        c = self.cfg
        return AT.attn_fwd(qkv_r, batch.cu_seqlens, c.num_attention_heads, c.num_key_value_heads, c.head_dim, need_lse=need_lse)

    def _attn_bwd(self, do, qkv_r, o, lse, batch: "PackedBatch"):
        c = self.cfg
        return AT.attn_bwd(do, qkv_r, o, lse, batch.cu_seqlens, c.num_attention_heads, c.num_key_value_heads, c.head_dim)

    def _embed_bwd(self, batch: "PackedBatch", dx: torch.Tensor) -> None:
        A.embedding_bwd(batch.input_ids, dx, self._wgrad("model.embed_tokens.weight"))

    def _tables(self, max_pos: int):
        return R.rope_tables(max(max_pos, 8), self.cfg.head_dim, self.cfg.rope_theta, self.device, self.cfg.rotary_dim)

    # ------------------------------------------------------------------ one layer
    # What the forward pass keeps per layer for backward, by ``self.recompute``:
    #   "full"       xin only: backward re-runs the layer up to the SwiGLU (everything but the down GEMM)
    #   "selective"  xin, qkv, o, lse, x1: backward re-runs the two norms, RoPE, the gate/up GEMM and SwiGLU
    #   "none"       additionally gu: backward re-runs only norms, RoPE and SwiGLU (no GEMM, no attention)
    # Bytes kept per token and layer (bf16, H = hidden): full 2H; selective 2(3H + qkv); none adds 4F.
    _KEEP = {"full": ("xin",), "selective": ("xin", "qkv", "o", "lse", "x1"), "none": ("xin", "qkv", "o", "lse", "x1", "gu")}

    def layer_fwd(self, l: int, x, delta, batch: PackedBatch, tables, keep: bool):
        """x (+ delta) is the residual stream entering the layer. Returns (x1, mlp_out, saved): the
        stream after attention, the not-yet-added MLP output (fused into the next norm) and, with
        ``keep``, the tensors backward wants (see ``_KEEP``)."""
        c = self.cfg
        qw = self._p(l, "self_attn.q_norm.weight") if c.qk_norm else None
        kw = self._p(l, "self_attn.k_norm.weight") if c.qk_norm else None
        h, rstd1, xin = N.rmsnorm_fwd(x, self._p(l, "input_layernorm.weight"), c.rms_norm_eps, delta=delta)
        qkv = self._lin(l, "self_attn.qkv_proj.weight", h)
        qkv_r = R.qknorm_rope_fwd(qkv, batch.position_ids, tables[0], tables[1], c.num_attention_heads,
                                  c.num_key_value_heads, c.head_dim, qw, kw, c.rms_norm_eps)
        want = self._KEEP[self.recompute] if keep else ()
        o, lse = self._attn_fwd(qkv_r, batch, need_lse="lse" in want)
        ao = self._post_norm(l, "post_self_attn_layernorm.weight", self._lin(l, "self_attn.o_proj.weight", o))
        h2, rstd2, x1 = N.rmsnorm_fwd(xin, self._p(l, "post_attention_layernorm.weight"), c.rms_norm_eps, delta=ao)
        mo, mlp_saved = self.mlp_fwd(l, h2, batch, want)
        mo = self._post_norm(l, "post_mlp_layernorm.weight", mo)
        local = dict(xin=xin, qkv=qkv, o=o, lse=lse, x1=x1, **mlp_saved)
        return x1, mo, ({k: local[k] for k in local if k in want or k in mlp_saved} if keep else xin)

    def _post_norm(self, l: int, name: str, y: torch.Tensor) -> torch.Tensor:
        """Sandwich-norm families (GLM-4) normalise a sub-layer's output before it joins the residual stream."""
        if not self.cfg.sandwich_norm:
            return y
        return N.rmsnorm_fwd(y, self._p(l, name), self.cfg.rms_norm_eps)[0]

    # ---- MLP hooks (dense SwiGLU here; the mixture-of-experts model overrides the three of them)
    def mlp_fwd(self, l: int, h2, batch: PackedBatch, want=()):
        """Returns (mlp output, tensors to keep for backward)."""
        gu = self._lin(l, "mlp.gate_up_proj.weight", h2)
        a = A.swiglu_fwd(gu)
        mo = self._lin(l, "mlp.down_proj.weight", a)
        return mo, ({"gu": gu} if "gu" in want else {})

    def mlp_infer(self, l: int, h2):
        """MLP of the sampler path (no state kept)."""
        return self.mlp_fwd(l, h2, None, ())[0]

    def mlp_rebuild(self, l: int, k: dict, batch: PackedBatch) -> None:
        if "gu" not in k:
            k["gu"] = self._lin(l, "mlp.gate_up_proj.weight", k["h2"])
        k["a"] = A.swiglu_fwd(k["gu"])

    def mlp_bwd(self, l: int, k: dict, dx_out):
        """Grad wrt the MLP input h2; accumulates the MLP weight gradients."""
        da = self._lin_bwd(l, "mlp.down_proj.weight", dx_out, k["a"])
        dgu = A.swiglu_bwd(da, k["gu"])
        del da
        dh2 = self._lin_bwd(l, "mlp.gate_up_proj.weight", dgu, k["h2"])
        return dh2

    def _rebuild(self, l: int, saved: dict, batch: PackedBatch, tables) -> dict:
        """Recompute, from what forward kept, every tensor backward reads."""
        c = self.cfg
        qw = self._p(l, "self_attn.q_norm.weight") if c.qk_norm else None
        kw = self._p(l, "self_attn.k_norm.weight") if c.qk_norm else None
        k = dict(saved)
        k["h"], k["rstd1"], _ = N.rmsnorm_fwd(k["xin"], self._p(l, "input_layernorm.weight"), c.rms_norm_eps)
        if "qkv" not in k:
            k["qkv"] = self._lin(l, "self_attn.qkv_proj.weight", k["h"])
        k["qkv_r"] = R.qknorm_rope_fwd(k["qkv"], batch.position_ids, tables[0], tables[1], c.num_attention_heads,
                                       c.num_key_value_heads, c.head_dim, qw, kw, c.rms_norm_eps)
        if "o" not in k:
            k["o"], k["lse"] = self._attn_fwd(k["qkv_r"], batch, need_lse=True)
        if c.sandwich_norm:       # backward of the output norms needs their inputs: the o-projection is re-run in every mode
            k["ao_raw"] = self._lin(l, "self_attn.o_proj.weight", k["o"])
            ao, k["rstd_a"], _ = N.rmsnorm_fwd(k["ao_raw"], self._p(l, "post_self_attn_layernorm.weight"), c.rms_norm_eps)
        if "x1" not in k:
            if not c.sandwich_norm:
                ao = self._lin(l, "self_attn.o_proj.weight", k["o"])
            k["h2"], k["rstd2"], k["x1"] = N.rmsnorm_fwd(k["xin"], self._p(l, "post_attention_layernorm.weight"),
                                                         c.rms_norm_eps, delta=ao)
        else:
            k["h2"], k["rstd2"], _ = N.rmsnorm_fwd(k["x1"], self._p(l, "post_attention_layernorm.weight"), c.rms_norm_eps)
        self.mlp_rebuild(l, k, batch)
        if c.sandwich_norm:       # ... and so is the down projection
            k["mo_raw"] = self._lin(l, "mlp.down_proj.weight", k["a"])
            k["rstd_m"] = N.rmsnorm_fwd(k["mo_raw"], self._p(l, "post_mlp_layernorm.weight"), c.rms_norm_eps)[1]
        return k

    def layer_bwd(self, l: int, saved, dx_out, batch: PackedBatch, tables):
        """dx_out: grad of the stream leaving the layer (x1 + mlp_out). Returns grad of the stream entering."""
        c = self.cfg
        if not isinstance(saved, dict):
            saved = {"xin": saved}
        k = self._rebuild(l, saved, batch, tables)
        qw = self._p(l, "self_attn.q_norm.weight") if c.qk_norm else None
        kw = self._p(l, "self_attn.k_norm.weight") if c.qk_norm else None
        d_mo = dx_out
        if c.sandwich_norm:
            d_mo = N.rmsnorm_bwd(dx_out, k["mo_raw"], self._p(l, "post_mlp_layernorm.weight"), k["rstd_m"],
                                 self._g(l, "post_mlp_layernorm.weight"))
        dh2 = self.mlp_bwd(l, k, d_mo)
        dx1 = N.rmsnorm_bwd(dh2, k["x1"], self._p(l, "post_attention_layernorm.weight"), k["rstd2"],
                            self._g(l, "post_attention_layernorm.weight"), dres=dx_out)
        del dh2, d_mo
        # attention
        d_ao = dx1
        if c.sandwich_norm:
            d_ao = N.rmsnorm_bwd(dx1, k["ao_raw"], self._p(l, "post_self_attn_layernorm.weight"), k["rstd_a"],
                                 self._g(l, "post_self_attn_layernorm.weight"))
        do = self._lin_bwd(l, "self_attn.o_proj.weight", d_ao, k["o"])
        dqkv_r = self._attn_bwd(do, k["qkv_r"], k["o"], k["lse"], batch)
        del do
        dqkv = R.qknorm_rope_bwd(dqkv_r, k["qkv"], batch.position_ids, tables[0], tables[1], c.num_attention_heads,
                                 c.num_key_value_heads, c.head_dim, qw, kw,
                                 self._g(l, "self_attn.q_norm.weight") if c.qk_norm else None,
                                 self._g(l, "self_attn.k_norm.weight") if c.qk_norm else None, c.rms_norm_eps)
        del dqkv_r
        dh = self._lin_bwd(l, "self_attn.qkv_proj.weight", dqkv, k["h"])
        del dqkv
        dx = N.rmsnorm_bwd(dh, k["xin"], self._p(l, "input_layernorm.weight"), k["rstd1"],
                           self._g(l, "input_layernorm.weight"), dres=dx1)
        return dx

    # ------------------------------------------------------------------ whole model
    def _trunk_fwd(self, batch: PackedBatch, save_for_backward: bool):
        """Embedding + all layers + final norm. Returns (hf, state) with state holding what backward needs."""
        c = self.cfg
        tables = self._tables(int(batch.max_seqlen) if batch.max_seqlen else c.max_position_embeddings)
        x = A.embedding_fwd(batch.input_ids, self.weights["model.embed_tokens.weight"])
        delta = None
        layer_inputs = []
        for l in range(c.num_hidden_layers):
            x, delta, saved = self.layer_fwd(l, x, delta, batch, tables, keep=save_for_backward)
            if save_for_backward:
                layer_inputs.append(saved if self.offloader is None else self.offloader.stash(l, saved))
            del saved
        hf, rstd_f, xf = N.rmsnorm_fwd(x, self.weights["model.norm.weight"], c.rms_norm_eps, delta=delta)
        state = dict(batch=batch, tables=tables, layer_inputs=layer_inputs, xf=xf, hf=hf, rstd_f=rstd_f) \
            if save_for_backward else None
        return hf, state

    def _trunk_bwd(self, s: dict, dhf: torch.Tensor, extra_dx: torch.Tensor | None = None) -> None:
        """``extra_dx``: a further gradient with respect to the stream before the final norm (the
        multi-token-prediction module reads it)."""
        c = self.cfg
        batch, tables = s["batch"], s["tables"]
        dx = N.rmsnorm_bwd(dhf, s["xf"], self.weights["model.norm.weight"], s["rstd_f"],
                           self._wgrad("model.norm.weight"), dres=extra_dx)
        del dhf
        inputs = s["layer_inputs"]
        for l in reversed(range(c.num_hidden_layers)):
            saved = inputs.pop()
            if self.offloader is not None:
                saved = self.offloader.fetch(saved)          # also starts bringing layer l - 1 back
            dx = self.layer_bwd(l, saved, dx, batch, tables)
            del saved
        if self.offloader is not None:
            self.offloader.end_step()
        self._embed_bwd(batch, dx)

    def forward_values(self, batch: PackedBatch, save_for_backward: bool = False) -> torch.Tensor:
        """Scalar value per packed position from the value head (fp32 [T]); needs ``value_head`` in the config."""
        hf, state = self._trunk_fwd(batch, save_for_backward)
        w = self.params["v_head.weight"]
        values = (hf.float() @ w.float().t()).squeeze(-1)
        if save_for_backward:
            state["kind"] = "values"
            self._saved = state
        return values

    def backward_values(self, g_values: torch.Tensor) -> None:
        s = self._saved
        assert s is not None and s.get("kind") == "values", "call forward_values(save_for_backward=True) first"
        self._saved = None
        self.params.alloc_grads()
        g = g_values.float().contiguous()
        w = self.params["v_head.weight"]
        self.params.grads["v_head.weight"].add_((g[None, :] @ s["hf"].float()))
        dhf = (g[:, None] * w.float()).to(s["hf"].dtype)
        self._trunk_bwd(s, dhf)

    def forward(self, batch: PackedBatch, temperature: float = 1.0, save_for_backward: bool = False):
        """Returns (logprob[T], entropy[T]) of the next token at every packed position (fp32)."""
        hf, state = self._trunk_fwd(batch, save_for_backward)
        lp, ent, lse = LM.lmhead_fwd(hf, self.head_weight(), batch.labels, temperature)
        if save_for_backward:
            state.update(kind="lm", lse=lse, ent=ent, temperature=temperature)
            if self.cfg.num_nextn_predict_layers > 0 and self.mtp_scale:
                from .mtp import mtp_fwd
                self.mtp_last = mtp_fwd(self, state)         # (sum of negative log-probs, positions) of this micro-batch
            self._saved = state
        return lp, ent

    def backward(self, g_logprob: torch.Tensor | None, g_entropy: torch.Tensor | None = None) -> None:
        """Backward from per-position grads of (logprob, entropy); accumulates into params.grads."""
        s = self._saved
        assert s is not None and s.get("kind") == "lm", "call forward(save_for_backward=True) first"
        self._saved = None
        self.params.alloc_grads()
        g_lp = None if g_logprob is None else g_logprob.float().contiguous()
        g_ent = None if g_entropy is None else g_entropy.float().contiguous()
        dhf = LM.lmhead_bwd(s["hf"], self.head_weight(), s["batch"].labels, s["lse"], s["ent"], g_lp, g_ent,
                            s["temperature"], dweight=self.head_grad())
        extra = None
        if "mtp" in s:
            from .mtp import mtp_bwd
            extra = mtp_bwd(self, s, float(self.mtp_scale))
        self._trunk_bwd(s, dhf, extra)

    # ------------------------------------------------------------------ analytic FLOPs (for MFU)
    def flops_per_token(self, seqlen: int) -> float:
        """Forward+backward FLOPs per token (6 x matmul params + attention), as the reference's
        FlopsCounter estimates for dense models (axon/utils/profiler/flops_counter.py)."""
        c = self.cfg
        dense = c.num_hidden_layers * (c.qkv_size * c.hidden_size + c.hidden_size * c.q_size
                                       + 3 * c.hidden_size * c.intermediate_size) + c.vocab_size * c.hidden_size
        attn = 12 * c.num_hidden_layers * c.q_size * seqlen / 2  # causal
        return 6 * dense + attn


# ---------------------------------------------------------------------------------------------
# Sampler-side forward passes (same weights, same kernels as training)
# ---------------------------------------------------------------------------------------------
class _DenseInference:
    """Mixed into DenseModel: prefill over packed prompts and single-token decode against a paged
    KV cache. Both write rotated K / V into the cache and return fp32 logits for sampling."""

    supports_cached_prefill = True

    def prefill(self, batch: PackedBatch, cache, tok_seq, tok_pos, block_table, last_index, past_lens=None):
        """batch: packed NEW tokens of every sequence (``position_ids`` are their positions in the sequence).
        tok_seq/tok_pos: per packed token cache row and position. last_index: int64 [B'] packed indices whose
        next-token logits are wanted. ``past_lens`` (python ints, one per sequence): tokens of the sequence whose keys
        and values are already in its cache pages (a prefix shared with an earlier request, or earlier chunks of a long
        prompt). Returns fp32 logits [B', V].

        With a cached prefix the new tokens' linear layers run on the new tokens only; for attention the prefix keys
        and values are gathered from the pages into a packed [prefix | new] row set and the packed causal kernel runs
        over it (its outputs at the new rows are kept). That reads every cached key once per layer, as a decode step
        would, and needs no attention kernel with separate query and key lengths."""
        from ..ops import paged as P
        c = self.cfg
        Hq, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        plan = None
        if past_lens is not None and any(int(p) > 0 for p in past_lens):
            plan = _cached_prefill_plan(batch, past_lens, block_table, tok_seq, self.device)
        max_pos = int(batch.position_ids.max().item()) + 1 if plan is not None else (int(batch.max_seqlen) if batch.max_seqlen else c.max_position_embeddings)
        tables = self._tables(max_pos)
        x = A.embedding_fwd(batch.input_ids, self.weights["model.embed_tokens.weight"])
        x, delta = self._stage_in(x)
        for l in range(c.num_hidden_layers):
            qw = self._p(l, "self_attn.q_norm.weight") if c.qk_norm else None
            kw = self._p(l, "self_attn.k_norm.weight") if c.qk_norm else None
            h, _, xin = N.rmsnorm_fwd(x, self._p(l, "input_layernorm.weight"), c.rms_norm_eps, delta=delta)
            qkv = self._lin(l, "self_attn.qkv_proj.weight", h)
            if tok_pos is batch.position_ids:      # the usual case: cache positions are the RoPE positions - one launch
                qkv_r = R.qknorm_rope_fwd(qkv, batch.position_ids, tables[0], tables[1], Hq, Hkv, D, qw, kw, c.rms_norm_eps,
                                          kv_cache=(cache.k[l], cache.v[l], tok_seq, block_table))
            else:
                qkv_r = R.qknorm_rope_fwd(qkv, batch.position_ids, tables[0], tables[1], Hq, Hkv, D, qw, kw, c.rms_norm_eps)
                P.kv_write(qkv_r, cache.k[l], cache.v[l], tok_seq, tok_pos, block_table, Hq, Hkv, D)
            if plan is None:
                o, _ = AT.attn_fwd(qkv_r, batch.cu_seqlens, Hq, Hkv, D, need_lse=False)
            else:
                full = torch.zeros(plan["T_full"], (Hq + 2 * Hkv) * D, dtype=qkv_r.dtype, device=qkv_r.device)
                full[plan["new_rows"]] = qkv_r
                kv = full.view(plan["T_full"], Hq + 2 * Hkv, D)
                kv[plan["pre_rows"], Hq:Hq + Hkv] = cache.k[l][plan["pre_page"], :, plan["pre_slot"]]
                kv[plan["pre_rows"], Hq + Hkv:] = cache.v[l][plan["pre_page"], :, plan["pre_slot"]]
                o_full, _ = AT.attn_fwd(full, plan["cu_full"], Hq, Hkv, D, need_lse=False)
                o = o_full[plan["new_rows"]].contiguous()
            ao = self._post_norm(l, "post_self_attn_layernorm.weight", self._lin(l, "self_attn.o_proj.weight", o))
            h2, _, x1 = N.rmsnorm_fwd(xin, self._p(l, "post_attention_layernorm.weight"), c.rms_norm_eps, delta=ao)
            delta = self._post_norm(l, "post_mlp_layernorm.weight", self.mlp_infer(l, h2))
            x = x1
        x, delta = self._stage_out(x, delta)
        xl = x[last_index]
        dl = delta[last_index]
        hf, _, _ = N.rmsnorm_fwd(xl, self.weights["model.norm.weight"], c.rms_norm_eps, delta=dl)
        return G.gemm_nt(hf, self.head_weight(), out_dtype=torch.float32)

    def decode(self, tokens, positions, cache, block_table, seq_lens, shared=None):
        """tokens/positions: int32 [B] (the token to feed and its position); seq_lens = positions + 1.
        ``shared``: prefix-sharing description of the batch (see ``ops.paged.paged_decode_shared``).
        Returns fp32 logits [B, V]."""
        from ..ops import paged as P
        c = self.cfg
        B = tokens.numel()
        tables = self._tables(c.max_position_embeddings)
        x = A.embedding_fwd(tokens, self.weights["model.embed_tokens.weight"])
        x, delta = self._stage_in(x)
        slots = cache.arange(B)
        for l in range(c.num_hidden_layers):
            qw = self._p(l, "self_attn.q_norm.weight") if c.qk_norm else None
            kw = self._p(l, "self_attn.k_norm.weight") if c.qk_norm else None
            h, _, xin = N.rmsnorm_fwd(x, self._p(l, "input_layernorm.weight"), c.rms_norm_eps, delta=delta)
            qkv = self._lin(l, "self_attn.qkv_proj.weight", h)
            qkv_r = R.qknorm_rope_fwd(qkv, positions, tables[0], tables[1], c.num_attention_heads,
                                      c.num_key_value_heads, c.head_dim, qw, kw, c.rms_norm_eps,
                                      kv_cache=(cache.k[l], cache.v[l], slots, block_table))
            if shared is None:
                o = P.paged_decode(qkv_r, cache.k[l], cache.v[l], block_table, seq_lens, c.num_attention_heads,
                                   c.num_key_value_heads, c.head_dim)
            else:
                o = P.paged_decode_shared(qkv_r, cache.k[l], cache.v[l], block_table, seq_lens, shared,
                                          c.num_attention_heads, c.num_key_value_heads, c.head_dim)
            ao = self._post_norm(l, "post_self_attn_layernorm.weight", self._lin(l, "self_attn.o_proj.weight", o))
            h2, _, x1 = N.rmsnorm_fwd(xin, self._p(l, "post_attention_layernorm.weight"), c.rms_norm_eps, delta=ao)
            delta = self._post_norm(l, "post_mlp_layernorm.weight", self.mlp_infer(l, h2))
            x = x1
        x, delta = self._stage_out(x, delta)
        hf, _, _ = N.rmsnorm_fwd(x, self.weights["model.norm.weight"], c.rms_norm_eps, delta=delta)
        return G.gemm_nt(hf, self.head_weight(), out_dtype=torch.float32)

    # A model that holds only a slice of the layers (a stage of a pipelined sampler group, ``models/pp_infer.py``) takes the
    # stream from the stage before it here and hands it on there; a whole model passes it through.
    def _stage_in(self, x):
        return x, None

    def _stage_out(self, x, delta):
        return x, delta


DenseModel.prefill = _DenseInference.prefill
DenseModel._stage_in = _DenseInference._stage_in
DenseModel._stage_out = _DenseInference._stage_out
DenseModel.supports_cached_prefill = True
DenseModel.decode = _DenseInference.decode
