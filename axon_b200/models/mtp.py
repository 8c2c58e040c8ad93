"""Multi-token prediction (depth 1) on top of the dense decoder.

Reference: the MTP patches of the Megatron trainer for packed sequences (axon/monkey_patches/megatron/mtp_training.py:
``roll_tensor`` per sequence, shared embedding and output head, loss added with a scaling factor;
enabled by ``AXON_ENABLE_MTP``) and the MTP loss inside the fused forward
(axon/models/mcore/forward/model_forward_fused.py:167-368). Parameter names follow the DeepSeek-V3
checkpoints: the module is decoder layer ``num_hidden_layers`` with ``enorm``, ``hnorm``, ``eh_proj`` and
``shared_head.norm`` beside the ordinary layer weights; embedding and output head are the model's own.

    z_t   = eh_proj [ enorm(embed(token_{t+1})) ; hnorm(h_t) ]          h_t: hidden state before the final norm
    h'_t  = decoder_layer(z)_t
    loss  = - mean_t log softmax(head(shared_head.norm(h'_t)))[token_{t+2}]

The module trains the draft head a speculative sampler would use; its loss is auxiliary: the engine adds
``coef * loss`` to the objective, the gradient flows into the shared embedding, the head and - through
``hnorm`` - the whole trunk. Everything is built from the kernels of the main model.
"""
from __future__ import annotations

import torch

from ..ops import activation as A
from ..ops import gemm as G
from ..ops import lm_head as LM
from ..ops import norm as N
from .dense import PackedBatch


class SlicedModuleMixin:
    """For the adapters of models whose ranks hold a slice of every batch's tokens: the engine's switch reaches the
    wrapped model, and the module's (sum of negative log-probs, targets) is summed over the ranks of the group."""

    same_rows_ranks = 1          # ranks of the optimizer's group that train on the same rows (the engine counts targets once)

    @property
    def mtp_scale(self):
        return self.inner.mtp_scale

    @mtp_scale.setter
    def mtp_scale(self, v):
        self.inner.mtp_scale = v

    def _wants_mtp(self) -> bool:
        return self.cfg.num_nextn_predict_layers > 0 and bool(self.inner.mtp_scale)

    def _mtp_group(self):
        raise NotImplementedError

    @property
    def mtp_last(self):
        import torch.distributed as dist
        last = self.inner.mtp_last
        if last is None:
            return None
        both = torch.stack([last[0].float(), last[1].float()])
        group = self._mtp_group()
        if group is not None:
            dist.all_reduce(both, group=group)
        return both[0], both[1]


def shifted_inputs(batch: PackedBatch):
    """(ids of token t+1, labels = token t+2 or -100) per packed position."""
    labels = batch.labels
    nxt = labels.clamp_min(0).to(batch.input_ids.dtype)
    lab2 = torch.roll(labels, -1)
    ends = (batch.cu_seqlens[1:].long() - 1).clamp_min(0)
    lab2[ends] = -100                      # the last position of a sequence would look into the next one
    lab2 = torch.where(labels < 0, torch.full_like(lab2, -100), lab2)
    return nxt, lab2


def mtp_fwd(model, s: dict) -> torch.Tensor:
    """Runs the module on the saved trunk state ``s`` (needs ``xf``: the stream before the final norm).
    Adds what backward needs under ``s['mtp']`` and returns (sum of -logprob over valid positions, count)."""
    c, batch, L = model.cfg, s["batch"], model.cfg.num_hidden_layers
    p = f"model.layers.{L}."
    w = model.weights
    # a rank that holds a slice of the tokens (sequence- / context-parallel) gets the slice of the shifted ids with its batch
    nxt, lab2 = getattr(batch, "mtp_inputs", None) or shifted_inputs(batch)
    e = A.embedding_fwd(nxt, w["model.embed_tokens.weight"])
    en, rstd_e, _ = N.rmsnorm_fwd(e, w[p + "enorm.weight"], c.rms_norm_eps)
    hn, rstd_h, _ = N.rmsnorm_fwd(s["xf"], w[p + "hnorm.weight"], c.rms_norm_eps)
    cat = torch.cat([en, hn], dim=1)
    z = G.gemm_nt(cat, w[p + "eh_proj.weight"])
    x2, delta2, saved = model.layer_fwd(L, z, None, batch, s["tables"], keep=True)
    hf2, rstd2, xf2 = N.rmsnorm_fwd(x2, w[p + "shared_head.norm.weight"], c.rms_norm_eps, delta=delta2)
    lp2, ent2, lse2 = LM.lmhead_fwd(hf2, model.head_weight(), lab2, 1.0)
    valid = (lab2 >= 0)
    s["mtp"] = dict(nxt=nxt, lab2=lab2, e=e, rstd_e=rstd_e, rstd_h=rstd_h, cat=cat, saved=saved, hf2=hf2, rstd2=rstd2,
                    xf2=xf2, lse2=lse2, ent2=ent2, valid=valid)
    return -(lp2.float() * valid).sum(), valid.sum()


def mtp_bwd(model, s: dict, scale: float) -> torch.Tensor:
    """Gradient of ``scale * sum_t(-logprob_t)``: accumulates the module's (and the shared embedding's / head's)
    weight gradients and returns the gradient with respect to the stream before the final norm."""
    c, batch, L = model.cfg, s["batch"], model.cfg.num_hidden_layers
    p = f"model.layers.{L}."
    w, m = model.weights, s.pop("mtp")
    H = c.hidden_size
    g_lp = (-scale) * m["valid"].float()
    dhf2 = LM.lmhead_bwd(m["hf2"], model.head_weight(), m["lab2"], m["lse2"], m["ent2"], g_lp, None, 1.0, dweight=model.head_grad())
    dx2 = N.rmsnorm_bwd(dhf2, m["xf2"], w[p + "shared_head.norm.weight"], m["rstd2"], model._wgrad(p + "shared_head.norm.weight"))
    dz = model.layer_bwd(L, m["saved"], dx2, batch, s["tables"])
    dcat = G.gemm_nn(dz, w[p + "eh_proj.weight"])
    G.gemm_tn(dz, m["cat"], out=model._wgrad(p + "eh_proj.weight"), accumulate=True)
    den, dhn = dcat[:, :H].contiguous(), dcat[:, H:].contiguous()
    de = N.rmsnorm_bwd(den, m["e"], w[p + "enorm.weight"], m["rstd_e"], model._wgrad(p + "enorm.weight"))
    A.embedding_bwd(m["nxt"], de, model._wgrad("model.embed_tokens.weight"))
    return N.rmsnorm_bwd(dhn, s["xf"], w[p + "hnorm.weight"], m["rstd_h"], model._wgrad(p + "hnorm.weight"))
