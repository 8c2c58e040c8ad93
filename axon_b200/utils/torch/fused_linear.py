"""Chunked vocabulary head in plain PyTorch: the fallback for the fused native head and the home of
tanh soft-capped logits (reference: axon/utils/torch/fused_linear.py:19-241).

``FusedLinearForPPO()(hidden [T, H], weight [V, H], labels [T], temperature)`` returns per-token
log-prob and entropy, processing ``chunk_size`` tokens at a time so that at most a
``[chunk, V]`` slab of logits is alive; backward recomputes each slab.
"""
from __future__ import annotations

import torch


def _softcap(logits: torch.Tensor, cap: float | None) -> torch.Tensor:
    return logits if not cap else torch.tanh(logits / cap) * cap


def _chunk_fwd(h, w, labels, temperature, softcap):
    logits = _softcap((h @ w.t()).float(), softcap) / temperature
    lse = torch.logsumexp(logits, dim=-1)
    p = torch.softmax(logits, dim=-1)
    lp = logits.gather(-1, labels.clamp_min(0).unsqueeze(-1)).squeeze(-1) - lse
    ent = lse - (p * logits).sum(-1)
    return lp, ent


class FusedLinearForPPOFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, temperature=1.0, chunk_size=512, softcap=None):
        ctx.set_materialize_grads(False)
        T = hidden.shape[0]
        lp = torch.empty(T, dtype=torch.float32, device=hidden.device)
        ent = torch.empty_like(lp)
        for s in range(0, T, chunk_size):
            lp[s:s + chunk_size], ent[s:s + chunk_size] = _chunk_fwd(hidden[s:s + chunk_size], weight, labels[s:s + chunk_size],
                                                                     temperature, softcap)
        ctx.save_for_backward(hidden, weight, labels)
        ctx.args = (temperature, chunk_size, softcap)
        return lp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        hidden, weight, labels = ctx.saved_tensors
        temperature, chunk, softcap = ctx.args
        dh = torch.zeros_like(hidden) if ctx.needs_input_grad[0] else None
        dw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device) if ctx.needs_input_grad[1] else None
        for s in range(0, hidden.shape[0], chunk):
            h = hidden[s:s + chunk]
            raw = (h @ weight.t()).float()
            capped = _softcap(raw, softcap)
            z = capped / temperature
            p = torch.softmax(z, dim=-1)
            dz = torch.zeros_like(z)
            if g_lp is not None:                      # d logprob / dz = onehot - p
                g = g_lp[s:s + chunk].float().unsqueeze(-1)
                dz -= g * p
                dz.scatter_add_(-1, labels[s:s + chunk].clamp_min(0).unsqueeze(-1), g)
            if g_ent is not None:                     # d entropy / dz = -p (z - sum p z)
                ge = g_ent[s:s + chunk].float().unsqueeze(-1)
                dz -= ge * p * (z - (p * z).sum(-1, keepdim=True))
            draw = dz / temperature
            if softcap:
                draw = draw * (1 - (capped / softcap) ** 2)
            draw = draw.to(hidden.dtype)
            if dh is not None:
                dh[s:s + chunk] = draw @ weight
            if dw is not None:
                dw += (draw.t() @ h).float()
        return dh, (dw.to(weight.dtype) if dw is not None else None), None, None, None, None


class FusedLinearForPPO(torch.nn.Module):
    def __init__(self, chunk_size: int = 512, softcap: float | None = None):
        super().__init__()
        self.chunk_size, self.softcap = chunk_size, softcap

    def forward(self, hidden_states, vocab_weights, input_ids, temperature: float = 1.0):
        shape = input_ids.shape
        h = hidden_states.reshape(-1, hidden_states.shape[-1])
        lp, ent = FusedLinearForPPOFunction.apply(h, vocab_weights, input_ids.reshape(-1), temperature, self.chunk_size, self.softcap)
        return lp.view(shape), ent.view(shape)
