"""Paged KV cache: per-layer ``[num_pages, Hkv, 128, D]`` K and V pools, a host-side free list with
reference counts (sequences sampled from the same prompt share the prompt's full pages), and
per-sequence block tables. Page = 128 tokens (one TMA tile of the decode kernel)."""
from __future__ import annotations

import torch

from ..models.config import ModelConfig

PAGE = 128


class PagedKVCache:
    def __init__(self, cfg: ModelConfig, num_pages: int, device, dtype=torch.bfloat16):
        self.cfg = cfg
        self.num_pages = int(num_pages)
        self.device = torch.device(device)
        shape = (self.num_pages, cfg.num_key_value_heads, PAGE, cfg.head_dim)
        self.k = [torch.zeros(shape, dtype=dtype, device=self.device) for _ in range(cfg.num_hidden_layers)]
        self.v = [torch.zeros(shape, dtype=dtype, device=self.device) for _ in range(cfg.num_hidden_layers)]
        self.free = list(range(self.num_pages - 1, -1, -1))
        self.ref = [0] * self.num_pages
        self.min_free = self.num_pages          # low-water mark of the free list (peak occupancy = num_pages - min_free)
        self._arange = torch.arange(4096, dtype=torch.int32, device=self.device)

    @staticmethod
    def bytes_per_page(cfg: ModelConfig, dtype_bytes: int = 2) -> int:
        return 2 * cfg.num_hidden_layers * cfg.num_key_value_heads * PAGE * cfg.head_dim * dtype_bytes

    def arange(self, n: int) -> torch.Tensor:
        if n > self._arange.numel():
            self._arange = torch.arange(2 * n, dtype=torch.int32, device=self.device)
        return self._arange[:n]

    def num_free(self) -> int:
        return len(self.free)

    def alloc(self, n: int) -> list[int]:
        if n > len(self.free):
            raise MemoryError(f"KV cache exhausted: want {n} pages, {len(self.free)} free")
        out = [self.free.pop() for _ in range(n)]
        for p in out:
            self.ref[p] = 1
        self.min_free = min(self.min_free, len(self.free))
        return out

    def share(self, pages: list[int]) -> list[int]:
        """Another owner for pages that are already full (read-only from now on)."""
        for p in pages:
            assert self.ref[p] > 0, f"page {p} is not allocated"
            self.ref[p] += 1
        return list(pages)

    def release(self, pages: list[int]) -> None:
        for p in pages:
            self.ref[p] -= 1
            if self.ref[p] == 0:
                self.free.append(p)

    def copy_pages(self, src: list[int], dst: list[int]) -> None:
        """Copy whole pages (every layer, K and V): the partly filled last prompt page of a shared prompt."""
        if not src:
            return
        si = torch.tensor(src, dtype=torch.long, device=self.device)
        di = torch.tensor(dst, dtype=torch.long, device=self.device)
        for k, v in zip(self.k, self.v):
            k[di] = k[si]
            v[di] = v[si]

    def drop(self) -> None:
        """Release the device memory (sleep); the cache must be rebuilt before the next use."""
        self.k, self.v = [], []
