"""Vision side of the vision-language families (Qwen2-VL / Qwen2.5-VL / Qwen3-VL layout).

Three pieces:

* ``mrope_position_ids``: the three rotary position rows (temporal, height, width) of a prompt that mixes text
  with image / video placeholders (reference: axon/models/transformers/qwen2_vl.py:63-170, which follows the
  HF ``get_rope_index``). Text tokens advance all three rows together; a vision block of ``t x h x w`` merged
  patches gets its grid coordinates, offset by the position the block starts at; the text after it continues
  from the largest coordinate used so far plus one.
* ``mrope_tables``: per-token cos / sin rows for the language model's rotary kernel. Frequency pair ``i`` of a
  head takes its angle from the row its section names (``mrope_section`` = pairs per row); because the kernel
  reads ``table[position]``, handing it these per-token rows with ``position = arange(T)`` applies the
  three-row rotary embedding without a second kernel.
* ``VisionTower``: a patch-embedding + transformer encoder + 2x2 patch merger in plain PyTorch (autograd), whose
  output rows replace the placeholder tokens' embeddings (reference: the HF vision towers the reference trains
  through axon/models/transformers/qwen2_vl.py:172-566, qwen3_vl.py). Attention runs per image (block-diagonal
  over the packed patch sequence) with 2-D rotary embeddings over the patch grid.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


def _token_id(processor, name: str, default: int | None = None) -> int | None:
    tok = getattr(processor, "tokenizer", processor)
    for owner in (processor, tok):
        v = getattr(owner, f"{name}_id", None)
        if v is not None:
            return int(v)
    conv = getattr(tok, "convert_tokens_to_ids", None)
    if conv is not None:
        try:
            v = conv(f"<|{name}_pad|>" if name in ("image", "video") else f"<|{name}|>")
            if v is not None and v >= 0:
                return int(v)
        except Exception:  # noqa: BLE001
            pass
    return default


def mrope_position_ids(processor, input_ids: torch.Tensor, attention_mask: torch.Tensor | None = None,
                       image_grid_thw: torch.Tensor | None = None, video_grid_thw: torch.Tensor | None = None,
                       second_per_grid_ts: torch.Tensor | None = None) -> torch.Tensor:
    """Rotary rows ``[3, T]`` (temporal, height, width) for ONE prompt. ``image_grid_thw`` / ``video_grid_thw``:
    ``[n, 3]`` patch grids (before the spatial merge) in the order the placeholders appear. Padding positions
    (``attention_mask == 0``) get 0."""
    T = input_ids.numel()
    ids = input_ids.reshape(-1)
    mask = torch.ones(T, dtype=torch.bool) if attention_mask is None else attention_mask.reshape(-1).bool()
    ip = getattr(processor, "image_processor", None)
    merge = int(getattr(ip, "merge_size", 2) or 2)
    tokens_per_second = float(getattr(getattr(processor, "video_processor", None), "tokens_per_second", 2) or 2)
    image_id, video_id = _token_id(processor, "image_token"), _token_id(processor, "video_token")
    if image_id is None:
        image_id = _token_id(processor, "image")
    if video_id is None:
        video_id = _token_id(processor, "video")
    real = ids[mask].tolist()
    rows: list[torch.Tensor] = []
    nxt = 0                    # first position available to the next segment
    i, n = 0, len(real)
    img_i = vid_i = 0
    while i < n:
        tok = real[i]
        is_img, is_vid = tok == image_id and image_grid_thw is not None, tok == video_id and video_grid_thw is not None
        if not (is_img or is_vid):
            j = i
            while j < n and not ((real[j] == image_id and image_grid_thw is not None) or
                                 (real[j] == video_id and video_grid_thw is not None)):
                j += 1
            seg = torch.arange(nxt, nxt + (j - i))
            rows.append(seg.expand(3, -1))
            nxt += j - i
            i = j
            continue
        if is_img:
            t, h, w = (int(x) for x in image_grid_thw[img_i])
            img_i += 1
            dt = 1.0
        else:
            t, h, w = (int(x) for x in video_grid_thw[vid_i])
            dt = float(second_per_grid_ts[vid_i]) * tokens_per_second if second_per_grid_ts is not None else 1.0
            vid_i += 1
        gh, gw = h // merge, w // merge
        count = t * gh * gw
        assert i + count <= n, "placeholder run shorter than its patch grid"
        tt = (torch.arange(t, dtype=torch.float64) * dt).long()[:, None, None].expand(t, gh, gw).reshape(-1)
        hh = torch.arange(gh)[None, :, None].expand(t, gh, gw).reshape(-1)
        ww = torch.arange(gw)[None, None, :].expand(t, gh, gw).reshape(-1)
        block = torch.stack([tt, hh, ww]) + nxt
        rows.append(block)
        nxt = int(block.max()) + 1
        i += count
    out = torch.zeros(3, T, dtype=torch.long)
    if rows:
        out[:, mask] = torch.cat(rows, dim=1)
    return out


def mrope_tables(positions: torch.Tensor, head_dim: int, theta: float, sections: list[int], device=None,
                 interleaved: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-token fp32 cos / sin rows ``[T, head_dim / 2]`` from rotary rows ``positions [3, T]``. ``sections`` =
    number of frequency pairs that follow the temporal, height and width row (sum = head_dim / 2). With
    ``interleaved`` (Qwen3-VL) the rows alternate t, h, w, t, h, w ... over the pairs instead of forming blocks."""
    half = head_dim // 2
    assert sum(sections) == half, f"mrope sections {sections} must add up to {half}"
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    if interleaved:
        which = torch.zeros(half, dtype=torch.long)
        for r in (1, 2):                                      # height, width take every third pair while they last
            idx = torch.arange(r, 3 * sections[r], 3)
            which[idx[idx < half]] = r
    else:
        which = torch.repeat_interleave(torch.arange(3), torch.tensor(sections))
    pos = positions.to(torch.float64).cpu()                    # [3, T]
    ang = pos[which, :].t() * inv[None, :]                     # [T, half]
    dev = device if device is not None else positions.device
    return ang.cos().float().to(dev).contiguous(), ang.sin().float().to(dev).contiguous()


@dataclass
class VisionConfig:
    depth: int = 2
    embed_dim: int = 64
    num_heads: int = 4
    mlp_ratio: float = 4.0
    in_channels: int = 3
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 256          # the language model's hidden size
    rms_norm_eps: float = 1e-6

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size


def _rot_half(x):
    a, b = x.chunk(2, dim=-1)
    return torch.cat([-b, a], dim=-1)


class _VisionBlock(nn.Module):
    def __init__(self, c: VisionConfig):
        super().__init__()
        self.norm1, self.norm2 = nn.LayerNorm(c.embed_dim, eps=c.rms_norm_eps), nn.LayerNorm(c.embed_dim, eps=c.rms_norm_eps)
        self.qkv, self.proj = nn.Linear(c.embed_dim, 3 * c.embed_dim), nn.Linear(c.embed_dim, c.embed_dim)
        hid = int(c.embed_dim * c.mlp_ratio)
        self.fc1, self.fc2 = nn.Linear(c.embed_dim, hid), nn.Linear(hid, c.embed_dim)
        self.heads = c.num_heads

    def forward(self, x, cos, sin, segments):
        T, E = x.shape
        q, k, v = self.qkv(self.norm1(x)).view(T, 3, self.heads, E // self.heads).unbind(1)
        q = q * cos[:, None, :] + _rot_half(q) * sin[:, None, :]
        k = k * cos[:, None, :] + _rot_half(k) * sin[:, None, :]
        outs = []
        for a, b in segments:                                  # full attention inside each image / frame group
            o = F.scaled_dot_product_attention(q[a:b].transpose(0, 1)[None], k[a:b].transpose(0, 1)[None], v[a:b].transpose(0, 1)[None])
            outs.append(o[0].transpose(0, 1).reshape(b - a, E))
        x = x + self.proj(torch.cat(outs))
        return x + self.fc2(F.gelu(self.fc1(self.norm2(x))))


class VisionTower(nn.Module):
    """Flattened patches ``[N, patch_dim]`` + grids ``[n_images, 3]`` -> ``[N / merge^2, out_hidden_size]``."""

    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.cfg = cfg
        self.patch_embed = nn.Linear(cfg.patch_dim, cfg.embed_dim, bias=False)
        self.blocks = nn.ModuleList(_VisionBlock(cfg) for _ in range(cfg.depth))
        m2 = cfg.spatial_merge_size ** 2
        self.merge_norm = nn.LayerNorm(cfg.embed_dim, eps=cfg.rms_norm_eps)
        self.merge_fc1 = nn.Linear(cfg.embed_dim * m2, cfg.embed_dim * m2)
        self.merge_fc2 = nn.Linear(cfg.embed_dim * m2, cfg.out_hidden_size)

    def rotary(self, grid_thw: torch.Tensor, device) -> tuple[torch.Tensor, torch.Tensor]:
        """2-D rotary angles of every patch in merge-window order (the processor lays patches out so that the
        merge^2 patches of a window are adjacent): half of a head's pairs follow the row index, half the column."""
        c = self.cfg
        hd = c.embed_dim // c.num_heads
        quarter = hd // 4
        inv = 1.0 / (10000.0 ** (torch.arange(0, quarter, dtype=torch.float32) / max(quarter, 1)))
        ms = c.spatial_merge_size
        rows = []
        for t, h, w in grid_thw.tolist():
            hi = torch.arange(h)[:, None].expand(h, w).reshape(h // ms, ms, w // ms, ms).permute(0, 2, 1, 3).reshape(-1)
            wi = torch.arange(w)[None, :].expand(h, w).reshape(h // ms, ms, w // ms, ms).permute(0, 2, 1, 3).reshape(-1)
            ang = torch.cat([hi[:, None].float() * inv[None], wi[:, None].float() * inv[None]], dim=1)      # [h*w, hd/2]
            rows.append(ang.repeat(t, 1))
        ang = torch.cat(rows).to(device)
        ang = torch.cat([ang, ang], dim=1)
        return ang.cos(), ang.sin()

    def forward(self, patches: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        x = self.patch_embed(patches.to(self.patch_embed.weight.dtype))
        cos, sin = self.rotary(grid_thw, x.device)
        cos, sin = cos.to(x.dtype), sin.to(x.dtype)
        segs, a = [], 0
        for t, h, w in grid_thw.tolist():
            for _ in range(t):
                segs.append((a, a + h * w))
                a += h * w
        assert a == x.shape[0], f"{x.shape[0]} patches for grids that describe {a}"
        for blk in self.blocks:
            x = blk(x, cos, sin, segs)
        m2 = c.spatial_merge_size ** 2
        x = self.merge_norm(x).view(-1, c.embed_dim * m2)
        return self.merge_fc2(F.gelu(self.merge_fc1(x)))


def merged_token_count(grid_thw: torch.Tensor, merge: int = 2) -> int:
    """Number of placeholder tokens the grids occupy in the prompt."""
    return int(sum(int(t) * (int(h) // merge) * (int(w) // merge) for t, h, w in grid_thw.tolist()))


def scatter_vision_embeddings(text_embeds: torch.Tensor, input_ids: torch.Tensor, vision_embeds: torch.Tensor,
                              placeholder_ids: tuple[int, ...]) -> tuple[torch.Tensor, torch.Tensor]:
    """Rows of ``text_embeds [T, H]`` at placeholder tokens replaced, in order, by ``vision_embeds``. Returns the
    merged embeddings and the row indices that were replaced (backward routes those rows' gradients to the tower)."""
    is_ph = torch.zeros_like(input_ids, dtype=torch.bool)
    for pid in placeholder_ids:
        is_ph |= input_ids == pid
    idx = torch.nonzero(is_ph).flatten()
    assert idx.numel() == vision_embeds.shape[0], f"{idx.numel()} placeholder tokens for {vision_embeds.shape[0]} vision rows"
    out = text_embeds.clone()
    out[idx] = vision_embeds.to(out.dtype)
    return out, idx
