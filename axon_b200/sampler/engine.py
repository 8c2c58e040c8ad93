"""In-process generation engine with continuous batching over a paged KV cache.

One ``GenerationEngine`` drives one model replica on one device: requests wait in a queue, are
admitted while KV pages are free, prefilled in packed batches under a token budget, and decoded
one token per running sequence per step. Log-probs are captured under the processed distribution
(after temperature / top-k / top-p). Supports pause / continue with the reference's strategies
(``drain | hold | continue | reset``: axon/sampler/vllm/server.py:653-744), sleep / wake (free and
re-create the KV pool: axon/sampler/vllm/engine.py:240-303) and in-place weight refresh.

The engine shares the model definition — and, when colocated, the very weight buffer — with the
trainer, so sampler and trainer log-probs agree by construction.
"""
from __future__ import annotations

import itertools
import time
from collections import OrderedDict, deque
from dataclasses import dataclass, field

import numpy as np
import torch

from ..models.dense import PackedBatch
from .kv_cache import PAGE, PagedKVCache
from .params import SamplingParams, TokenOutput


@dataclass
class _Seq:
    rid: int
    prompt: list
    params: SamplingParams
    out: TokenOutput = field(default_factory=TokenOutput)
    pages: list = field(default_factory=list)
    length: int = 0            # tokens currently in the KV cache
    last_token: int = 0
    done: bool = False
    leader: object = None      # during admission: the sequence whose prompt pages and prefill this one reuses
    share_key: int = -1        # rid of the sequence whose prompt pages this one shares (its own rid for that sequence)
    shared_pages: int = 0      # number of leading pages shared with the group
    cached: int = 0            # leading tokens whose keys / values are already in the pages (prefix cache hit, earlier chunks)
    chunk_end: int = 0         # the prefill call in progress covers tokens [cached, chunk_end)
    route_chunks: list = field(default_factory=list)    # routed-experts capture: int16 [n, layers, top-k] pieces in token order
    mm: dict | None = None     # vision inputs of the prompt: pixel_values [patches, patch_dim], image_grid_thw [images, 3]
    mrope: object = None       # rotary rows [3, prompt length] of a prompt with vision inputs
    rope_delta: int = 0        # rotary position of generated token i = prompt length + i + rope_delta


class GenerationEngine:
    def __init__(self, model, num_pages: int | None = None, max_num_seqs: int = 256,
                 max_num_batched_tokens: int = 32768, kv_memory_bytes: int | None = None, seed: int = 0):
        self.model = model
        self.cfg = model.cfg
        self.device = model.device
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        if num_pages is None:
            budget = kv_memory_bytes if kv_memory_bytes is not None else 4 << 30
            num_pages = max(8, budget // PagedKVCache.bytes_per_page(self.cfg, model.params.flat.element_size()))
        self._num_pages = int(num_pages)
        self.cache: PagedKVCache | None = PagedKVCache(self.cfg, self._num_pages, self.device, model.params.dtype)
        self.waiting: deque[_Seq] = deque()
        self.running: list[_Seq] = []
        self.finished: dict[int, TokenOutput] = {}
        self._rid = itertools.count()
        self.seed = seed
        self.step_count = 0
        self.paused = False
        self.pause_strategy = "drain"
        self.stats = dict(prefill_tokens=0, decode_tokens=0, decode_steps=0, preempted=0)
        # CUDA-graph decode: one captured graph per batch-size bucket (re-captured after every wake_up,
        # because the KV pool moves). Disabled on CPU.
        self.use_cuda_graph = self.device.type == "cuda" and getattr(model, "supports_cuda_graph", True)
        # n samples of one prompt share its KV pages and its prefill (not for models that keep per-sequence recurrent state)
        self.share_prompts = not getattr(model, "has_recurrent_state", False)
        # "processed": log-prob under the distribution actually drawn from (after top-k / top-p, the reference
        # fork's convention); "full": temperature-scaled log-softmax over the whole vocabulary (what the trainer
        # recomputes), which keeps importance-sampling corrections unbiased under truncation.
        self.logprobs_mode = "processed"
        # Routed-experts capture (sparse models): every token's chosen experts per layer are recorded and returned as
        # ``TokenOutput.moe_routermap`` int16 [prompt + output tokens, moe layers, top-k]; the row of the last sampled
        # token, which never went through the model, is -1 (reference: the vLLM fork's routed_experts output,
        # install/vllm/axon.patch:586-748, consumed at axon/engine/engine.py:1157-1175). The trainer replays it.
        self.capture_routing = False
        # Prefix caching across requests: full pages of finished or prefilled sequences stay in the pool under a hash of
        # the tokens they hold (chained page by page); a new request whose prompt starts with the same tokens shares
        # those pages and prefills only the rest. The cache holds one reference per page and gives pages back, least
        # recently used first, when the pool runs short. Chunked prefill: a prompt longer than ``max_num_batched_tokens``
        # is prefilled in pieces, later pieces attending to the cached keys of the earlier ones.
        self.enable_prefix_caching = False
        self.enable_chunked_prefill = True
        self._cached_ok = bool(getattr(model, "supports_cached_prefill", False))
        self._prefix_pages: "OrderedDict[int, int]" = OrderedDict()      # chain hash -> page
        self._page_hash: dict[int, int] = {}
        self.prefilling: list[_Seq] = []       # sequences whose prompt is partly prefilled (chunked)
        # Decode attention over the shared pages once per group (csrc/paged_attention_shared.cu). Off by default: with
        # one CTA per SM the per-CTA start-up of the extra prefix / suffix items costs as much as the shared tiles
        # save once responses are a few pages long (measured end to end); the kernel pays off for long shared
        # prefixes with short tails and is kept selectable.
        # Speculative decoding with n-gram drafts (prompt lookup): up to this many tokens that followed the latest earlier
        # occurrence of the sequence's last tokens are proposed and verified in one pass over [last token | drafts]
        # against the cached prefix. 0 = off. Needs a model with cached-prefix prefill.
        self.speculative_ngram = 0
        self.speculative_ngram_match = 3          # longest suffix tried first; shorter ones down to one token
        self.cascade_attention = False
        self.cascade_min_batch = 48
        self._graphs: dict[int, dict] = {}
        # batch-size buckets of the captured graphs: the decode GEMM's token width is a run-time value, so
        # finer buckets than powers of two pay off as the batch drains
        self.graph_buckets = (8, 16, 24, 32, 48, 64, 80, 96, 112, 128, 160, 192, 224, 256)
        self.max_pages_per_seq = (self.cfg.max_position_embeddings + PAGE - 1) // PAGE

    # ------------------------------------------------------------------ request API
    def add_request(self, prompt_ids, params: SamplingParams, image_data: dict | None = None) -> int:
        """``image_data`` (vision-language models): the processor's ``pixel_values`` / ``image_grid_thw`` (and the video
        pair) for the placeholder tokens of ``prompt_ids``; requests that pass the SAME dict object share their prompt
        pages (n samples of one prompt)."""
        rid = next(self._rid)
        seq = _Seq(rid, list(map(int, prompt_ids)), params)
        seq.out.prompt_len = len(seq.prompt)
        if image_data:
            assert hasattr(self.model, "rotary_rows"), "this model takes no vision inputs"
            seq.mm = image_data
            seq.mrope = self.model.rotary_rows(seq.prompt, image_data)                   # [3, n]
            seq.rope_delta = int(seq.mrope.max()) + 1 - len(seq.prompt)
        self.waiting.append(seq)
        return rid

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running or self.prefilling)

    def generate(self, prompts, params, image_data=None) -> list[TokenOutput]:
        """Blocking helper: run all prompts to completion; ``params`` is one SamplingParams or a list, ``image_data``
        None or one entry (dict or None) per prompt."""
        plist = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
        ilist = image_data if image_data is not None else [None] * len(prompts)
        rids = [self.add_request(p, sp, im) for p, sp, im in zip(prompts, plist, ilist)]
        while self.has_unfinished():
            self.step()
        return [self.finished.pop(r) for r in rids]

    # ------------------------------------------------------------------ control
    def pause(self, strategy: str = "drain") -> None:
        """drain: finish running sequences, admit nothing new. hold: freeze everything in place.
        continue: keep generating (no-op marker). reset: abort running sequences (their partial
        outputs are returned with finish_reason 'abort') and requeue nothing."""
        assert strategy in ("drain", "hold", "continue", "reset")
        self.pause_strategy = strategy
        self.paused = strategy != "continue"
        if strategy == "drain":
            while self.running:
                self.step()
        elif strategy == "reset":
            for s in self.running:
                self._finish(s, "abort")
            self.running = []

    def resume(self) -> None:
        self.paused = False

    def sleep(self) -> None:
        """Free the KV pool (running sequences are aborted, as a level-1 sleep discards the cache)."""
        for s in self.running:
            self._finish(s, "abort")
        self.running = []
        for s in self.prefilling:
            self._finish(s, "abort")
        self.prefilling = []
        self.reset_prefix_cache()
        if self.cache is not None:
            self.cache.drop()
        self.cache = None
        self._graphs.clear()
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    def wake_up(self, num_pages: int | None = None) -> None:
        if self.cache is None:
            if num_pages is not None:
                self._num_pages = int(num_pages)
            self.cache = PagedKVCache(self.cfg, self._num_pages, self.device, self.model.params.dtype)

    # ------------------------------------------------------------------ internals
    def _finish(self, s: _Seq, reason: str, stop=None) -> None:
        s.done = True
        s.out.finish_reason = reason
        s.out.stop_reason = stop
        if self.capture_routing:
            s.out.moe_routermap = self._routermap(s)
        if self.enable_prefix_caching and self.cache is not None and s.pages and s.length > 0:
            # the keys / values of the first ``length`` tokens are in the pages: later turns that extend this text reuse them
            self._register_prefix(s.prompt + s.out.token_ids, s.pages, s.length)
        if self.cache is not None:
            self.cache.release(s.pages)
        s.pages = []
        self.finished[s.rid] = s.out

    # ------------------------------------------------------------------ prefix cache
    @staticmethod
    def _chain(tokens: list, n_pages: int) -> list[int]:
        keys, h = [], 0
        for k in range(n_pages):
            h = hash((h, tuple(tokens[k * PAGE:(k + 1) * PAGE])))
            keys.append(h)
        return keys

    def reset_prefix_cache(self) -> None:
        """Forget every cached prefix (the weights changed, or the pool is being dropped)."""
        if self.cache is not None and self.cache.k:
            self.cache.release(list(self._prefix_pages.values()))
        self._prefix_pages.clear()
        self._page_hash.clear()

    def _lookup_prefix(self, tokens: list) -> list[int]:
        """Pages holding the longest cached prefix of ``tokens`` that leaves at least one token to compute."""
        pages = []
        for key in self._chain(tokens, (len(tokens) - 1) // PAGE):
            pg = self._prefix_pages.get(key)
            if pg is None:
                break
            self._prefix_pages.move_to_end(key)
            pages.append(pg)
        return pages

    def _register_prefix(self, tokens: list, pages: list[int], n_tokens: int) -> None:
        """Keep the full pages among the first ``n_tokens`` tokens of a sequence findable for later requests."""
        if not self.enable_prefix_caching or not self._cached_ok:
            return
        for k, key in enumerate(self._chain(tokens, n_tokens // PAGE)):
            if key in self._prefix_pages:
                self._prefix_pages.move_to_end(key)
                continue
            if pages[k] in self._page_hash:
                continue
            self.cache.share([pages[k]])
            self._prefix_pages[key] = pages[k]
            self._page_hash[pages[k]] = key

    def _evict_prefixes(self, need: int) -> None:
        """Give back cached pages nobody else holds, oldest first, until ``need`` pages are free."""
        for key in list(self._prefix_pages):
            if self.cache.num_free() >= need:
                break
            pg = self._prefix_pages[key]
            if self.cache.ref[pg] == 1:
                del self._prefix_pages[key]
                del self._page_hash[pg]
                self.cache.release([pg])

    def _admit(self) -> list[_Seq]:
        """Pick waiting sequences that fit the page pool and the token budget. Fresh sequences with the
        same prompt as an earlier one of the batch (n samples per prompt) become its followers: they
        share the prompt's full pages and are not prefilled again. With prefix caching a fresh sequence also
        shares the pages of the longest cached prefix of its prompt. A prompt longer than the token budget is
        admitted alone and prefilled in chunks over several steps."""
        batch, tokens = [], 0
        budget = self.max_num_batched_tokens
        if self.prefilling:                      # the next chunk of a partly prefilled prompt goes first, on its own
            s = self.prefilling.pop(0)
            s.chunk_end = min(len(s.prompt) + len(s.out.token_ids), s.cached + budget)
            return [s]
        leaders: dict[tuple, _Seq] = {}
        while self.waiting and len(self.running) + len(batch) < self.max_num_seqs:
            s = self.waiting[0]
            n = len(s.prompt) + len(s.out.token_ids)  # a preempted sequence re-prefills its output too
            need = (n + 1 + PAGE - 1) // PAGE
            key = (tuple(s.prompt), id(s.mm)) if (self.share_prompts and not s.out.token_ids) else None
            lead = leaders.get(key) if key is not None else None
            held: list[int] = []
            if lead is None and self.enable_prefix_caching and self._cached_ok and not s.out.token_ids:
                held = self.cache.share(self._lookup_prefix(s.prompt))       # hold the hit before anything is evicted
            shared = (len(s.prompt) // PAGE) if lead is not None else len(held)
            # keep one page of head-room per running sequence so decode can always advance
            reserve = len(self.running) + len(batch)
            if need - shared > self.cache.num_free() - reserve and self._prefix_pages:
                self._evict_prefixes(need - shared + reserve)
            if need - shared > self.cache.num_free() - reserve:
                self.cache.release(held)
                break
            fresh = n - shared * PAGE if lead is None else 0
            chunked = lead is None and fresh > budget and self.enable_chunked_prefill and self._cached_ok
            if lead is None and batch and (tokens + fresh > budget or chunked):
                self.cache.release(held)
                break
            self.waiting.popleft()
            if lead is not None:
                s.pages = self.cache.share(lead.pages[:shared]) + self.cache.alloc(need - shared)
                s.leader = lead
                s.share_key, s.shared_pages = lead.rid, shared
                lead.share_key, lead.shared_pages = lead.rid, shared
            else:
                s.pages = held + self.cache.alloc(need - shared)
                s.leader = None
                s.share_key, s.shared_pages = -1, 0
                s.cached = shared * PAGE
                s.chunk_end = s.cached + budget if chunked else n
                if held:
                    self.stats["prefix_cache_hit_tokens"] = self.stats.get("prefix_cache_hit_tokens", 0) + s.cached
                tokens += s.chunk_end - s.cached
                if key is not None and not chunked:
                    leaders[key] = s
            batch.append(s)
            if chunked:
                break
        return batch

    def _block_table(self, seqs) -> torch.Tensor:
        width = max(len(s.pages) for s in seqs)
        bt = np.full((len(seqs), width), -1, dtype=np.int32)
        for i, s in enumerate(seqs):
            bt[i, : len(s.pages)] = s.pages
        return torch.from_numpy(bt).to(self.device, non_blocking=True)

    def _sampling_tensors(self, seqs):
        t = torch.tensor([s.params.temperature for s in seqs], dtype=torch.float32).to(self.device)
        ks = [s.params.top_k for s in seqs]
        ps = [s.params.top_p for s in seqs]
        k = torch.tensor(ks, dtype=torch.int32).to(self.device) if any(x > 0 for x in ks) else None
        p = torch.tensor(ps, dtype=torch.float32).to(self.device) if any(x < 1.0 for x in ps) else None
        ctr = torch.tensor([len(s.out.token_ids) + 7919 * (s.rid + 1) for s in seqs], dtype=torch.int32).to(self.device)
        return t, k, p, ctr

    def _sample_and_record(self, seqs, logits) -> None:
        from ..ops import paged as P
        pens = [s.params.repetition_penalty for s in seqs]
        if any(x != 1.0 for x in pens):
            V = logits.shape[1]
            seen = torch.zeros(len(seqs), V, dtype=torch.uint8)
            for i, s in enumerate(seqs):
                seen[i, torch.tensor(s.prompt + s.out.token_ids, dtype=torch.long).clamp(0, V - 1)] = 1
            P.repetition_penalty_(logits, seen.to(self.device), torch.tensor(pens, dtype=torch.float32).to(self.device))
        t, k, p, ctr = self._sampling_tensors(seqs)
        toks, lps = P.sample(logits, t, k, p, seed=self.seed, counters=ctr, logprobs_mode=self.logprobs_mode)
        # the one host sync of a step: finish detection needs the ids
        self._record(seqs, toks.cpu().tolist(), lps.cpu().tolist())

    def _prefill(self, all_seqs) -> None:
        seqs = [s for s in all_seqs if getattr(s, "leader", None) is None]     # followers reuse their leader's prefill
        full = [s.prompt + s.out.token_ids for s in seqs]
        for s, f in zip(seqs, full):
            if s.chunk_end <= s.cached:                # sequences admitted before these fields existed, or re-admitted
                s.cached, s.chunk_end = 0, len(f)
        past = [s.cached for s in seqs]
        toks = [torch.tensor(f[s.cached:s.chunk_end], dtype=torch.int32) for s, f in zip(seqs, full)]
        batch = PackedBatch.from_sequences(toks, self.device)
        lens = [int(t.numel()) for t in toks]
        if any(past):
            batch.position_ids = batch.position_ids + torch.cat(
                [torch.full((n,), p, dtype=torch.int32) for n, p in zip(lens, past)]).to(self.device)
            batch.max_seqlen = max(p + n for p, n in zip(past, lens))
        tok_seq = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(lens)]).to(self.device)
        ends = torch.tensor(lens).cumsum(0) - 1
        complete = [s.chunk_end >= len(f) for s, f in zip(seqs, full)]
        last = ends[torch.tensor(complete)].to(self.device) if any(complete) else ends[:1].to(self.device)
        bt = self._block_table(seqs)
        if any(s.mm is not None for s in seqs):
            # vision inputs in packed order, and three rotary rows per token (text-only sequences repeat their positions;
            # tokens generated before a preemption continue after the prompt's largest rotary position)
            rows, pix, grids = [], [], []
            for s, n in zip(seqs, lens):
                if s.mm is None:
                    rows.append(torch.arange(n)[None].expand(3, n))
                    continue
                extra = torch.arange(n - len(s.prompt))[None].expand(3, -1) + len(s.prompt) + s.rope_delta
                rows.append(torch.cat([s.mrope, extra], dim=1))
                for pk, gk in (("pixel_values", "image_grid_thw"), ("pixel_values_videos", "video_grid_thw")):
                    if s.mm.get(pk) is not None and len(s.mm[pk]):
                        pix.append(torch.as_tensor(s.mm[pk]))
                        grids.append(torch.as_tensor(s.mm[gk]).reshape(-1, 3))
            batch.multimodal = {"pixel_values": torch.cat(pix).to(self.device) if pix else None,
                                "image_grid_thw": torch.cat(grids) if grids else None,
                                "mrope_positions": torch.cat(rows, dim=1).to(self.device)}
        if self.capture_routing:
            self.model.last_routing = None
        if any(past):
            logits = self.model.prefill(batch, self.cache, tok_seq, batch.position_ids, bt, last, past_lens=past)
        else:
            logits = self.model.prefill(batch, self.cache, tok_seq, batch.position_ids, bt, last)
        if self.capture_routing:
            rt = self._take_routing()
            if rt is not None:
                rt_h, off = rt.cpu().numpy(), 0
                for s, n in zip(seqs, lens):
                    # a re-prefill after preemption covers prompt + output so far; later chunks of a long prompt follow on
                    s.route_chunks = (s.route_chunks if s.cached > 0 else []) + [rt_h[off:off + n]]
                    off += n
        self.stats["prefill_tokens"] += sum(lens)
        pending = []
        for s, f, done in zip(seqs, full, complete):
            if done:
                s.length = len(f)
                self._register_prefix(f, s.pages, len(f))
            else:
                s.cached = s.chunk_end
                pending.append(s)
        if pending:                                   # chunked prompts continue in the next step; nothing is sampled for them
            self.prefilling.extend(pending)
            all_seqs = [s for s in all_seqs if s not in pending]
            seqs = [s for s in seqs if s not in pending]
            if not all_seqs:
                return
        if len(seqs) != len(all_seqs):
            row = {id(s): i for i, s in enumerate(seqs)}
            src, dst, rows = [], [], []
            for s in all_seqs:
                lead = s.leader if s.leader is not None else s
                rows.append(row[id(lead)])
                if s.leader is not None:
                    s.length = lead.length
                    if self.capture_routing and getattr(lead, "route_chunks", None):
                        s.route_chunks = [np.concatenate(lead.route_chunks, axis=0)]     # same prompt, same routing
                    full_pages = len(s.prompt) // PAGE
                    if len(s.prompt) % PAGE:          # the partly filled last prompt page is private: copy it
                        src.append(lead.pages[full_pages])
                        dst.append(s.pages[full_pages])
                    s.leader = None
            self.cache.copy_pages(src, dst)
            self.stats["shared_prompt_seqs"] = self.stats.get("shared_prompt_seqs", 0) + len(all_seqs) - len(seqs)
            logits = logits[torch.tensor(rows, dtype=torch.long, device=logits.device)]
        self._sample_and_record(all_seqs, logits)
        self.running.extend(s for s in all_seqs if not s.done)

    # ------------------------------------------------------------------ CUDA-graph decode
    def set_max_model_len(self, n: int) -> None:
        """Upper bound on prompt + response length; fixes the block-table width of the decode graphs."""
        self.max_pages_per_seq = (n + PAGE - 1) // PAGE + 1
        self._graphs.clear()

    def _capture(self, bucket: int, cascade: bool = False) -> dict:
        from ..ops import paged as P
        dev = self.device
        g = dict(tokens=torch.zeros(bucket, dtype=torch.int32, device=dev),
                 pos=torch.zeros(bucket, dtype=torch.int32, device=dev),
                 lens=torch.zeros(bucket, dtype=torch.int32, device=dev),
                 bt=torch.full((bucket, self.max_pages_per_seq), -1, dtype=torch.int32, device=dev),
                 temp=torch.ones(bucket, dtype=torch.float32, device=dev),
                 top_k=torch.zeros(bucket, dtype=torch.int32, device=dev),
                 top_p=torch.ones(bucket, dtype=torch.float32, device=dev),
                 ctr=torch.zeros(bucket, dtype=torch.int32, device=dev))
        shared = None
        if cascade:      # prefix-sharing description: one suffix item per row, up to bucket // 2 group items
            ng = max(1, bucket // 2)
            zi = lambda n: torch.zeros(n, dtype=torch.int32, device=dev)      # noqa: E731
            g.update(seq_page0=zi(bucket), seq_keys=zi(bucket), grp_first=zi(ng), grp_size=zi(ng), grp_keys=zi(ng))
            shared = dict(seq_first=torch.arange(bucket, dtype=torch.int32, device=dev), seq_one=torch.ones(bucket, dtype=torch.int32, device=dev),
                          seq_page0=g["seq_page0"], seq_keys=g["seq_keys"], grp_first=g["grp_first"], grp_size=g["grp_size"],
                          grp_zero=zi(ng), grp_keys=g["grp_keys"], max_shared_pages=self.max_pages_per_seq)

        def run():
            if self.capture_routing:
                self.model.last_routing = None
            logits = self.model.decode(g["tokens"], g["pos"], self.cache, g["bt"], g["lens"], shared=shared)
            if self.capture_routing:
                g["routing"] = self._take_routing()      # a graph output: same memory on every replay
            return P.sample(logits, g["temp"], g["top_k"], g["top_p"], seed=self.seed, counters=g["ctr"],
                            logprobs_mode=self.logprobs_mode)

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):        # warm-up: sizes every cached workspace before capture
                run()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        from ..ops import _common as C
        graph = torch.cuda.CUDAGraph()
        n0 = C.LAUNCH_COUNT
        with torch.cuda.graph(graph):
            g["out_tokens"], g["out_lps"] = run()
        g["launches"] = C.LAUNCH_COUNT - n0      # kernels each replay launches
        g["graph"] = graph
        keys = ("tokens", "pos", "lens", "bt", "temp", "top_k", "top_p", "ctr") + \
            (("seq_page0", "seq_keys", "grp_first", "grp_size", "grp_keys") if cascade else ())
        g["host"] = {k: torch.empty(g[k].shape, dtype=g[k].dtype, pin_memory=True) for k in keys}
        return g

    def _share_groups(self, seqs) -> list[tuple[int, int, int]]:
        """(first row, members, shared pages) of every run of >= 2 consecutive sequences that share prompt
        pages, cut into items of at most 32 / (query heads per kv head) members."""
        gmax = max(1, 32 // max(1, self.cfg.num_attention_heads // self.cfg.num_key_value_heads))
        out, i, n = [], 0, len(seqs)
        while i < n:
            s = seqs[i]
            j = i + 1
            if s.shared_pages > 0:
                while j < n and seqs[j].share_key == s.share_key and seqs[j].shared_pages == s.shared_pages:
                    j += 1
            if j - i >= 2:
                for a in range(i, j, gmax):
                    if min(j, a + gmax) - a >= 2:
                        out.append((a, min(j, a + gmax) - a, s.shared_pages))
            i = j
        return out

    def _decode_graph(self, seqs) -> tuple[list, list]:
        t_host0 = time.perf_counter()
        B = len(seqs)
        bucket = next((b for b in self.graph_buckets if b >= B), None)
        if bucket is None:
            bucket = (B + 63) // 64 * 64
        # below this batch size the extra prefix / merge launches cost more than the shared pages save
        groups = self._share_groups(seqs) if (self.share_prompts and self.cascade_attention and B >= self.cascade_min_batch) else []
        cascade = bool(groups)
        g = self._graphs.get((bucket, cascade))
        if g is None:
            g = self._graphs[(bucket, cascade)] = self._capture(bucket, cascade)
        h = g["host"]
        h["tokens"].zero_(); h["pos"].zero_(); h["lens"].zero_(); h["bt"].fill_(-1)
        h["temp"].fill_(1.0); h["top_k"].zero_(); h["top_p"].fill_(1.0); h["ctr"].zero_()
        if cascade:
            for k in ("seq_page0", "seq_keys", "grp_first", "grp_size", "grp_keys"):
                h[k].zero_()
            p0, ky = h["seq_page0"].numpy(), h["seq_keys"].numpy()
            for i, s in enumerate(seqs):
                ky[i] = s.length + 1
            gf, gs, gk = h["grp_first"].numpy(), h["grp_size"].numpy(), h["grp_keys"].numpy()
            for n, (a, m, sh) in enumerate(groups):
                gf[n], gs[n], gk[n] = a, m, sh * PAGE
                p0[a:a + m] = sh
                ky[a:a + m] -= sh * PAGE
        tok, pos, lens, bt = h["tokens"].numpy(), h["pos"].numpy(), h["lens"].numpy(), h["bt"].numpy()
        temp, tk, tp, ctr = h["temp"].numpy(), h["top_k"].numpy(), h["top_p"].numpy(), h["ctr"].numpy()
        for i, s in enumerate(seqs):
            tok[i], pos[i], lens[i] = s.last_token, s.length, s.length + 1
            bt[i, : len(s.pages)] = s.pages
            temp[i], tk[i], tp[i] = s.params.temperature, max(0, s.params.top_k), s.params.top_p
            ctr[i] = len(s.out.token_ids) + 7919 * (s.rid + 1)
        for k in h:
            g[k].copy_(h[k], non_blocking=True)
        g["graph"].replay()
        from ..ops import _common as C
        C.LAUNCH_COUNT += g["launches"]
        # the device is idle while the host fills the step's inputs (the previous step ended with a sync): that time is
        # what overlapping the scheduler with the device would win back
        self.stats["decode_host_prep_s"] = self.stats.get("decode_host_prep_s", 0.0) + (time.perf_counter() - t_host0)
        if self.capture_routing and g.get("routing") is not None:
            rt_h = g["routing"][:B].cpu().numpy()
            for i, s in enumerate(seqs):
                s.route_chunks.append(rt_h[i:i + 1].copy())
        return g["out_tokens"][:B].cpu().tolist(), g["out_lps"][:B].cpu().tolist()

    def enable_routing_capture(self, on: bool = True) -> None:
        if on and getattr(self.cfg, "num_experts", 0) <= 0:
            raise ValueError("routed-experts capture needs a sparse (mixture-of-experts) model")
        self.capture_routing = bool(on)
        self.model.capture_routing = bool(on)
        self._graphs.clear()                     # decode graphs are captured with or without the routing output

    def _take_routing(self) -> torch.Tensor | None:
        """The expert ids of the model call that just ran: int16 [tokens, moe layers, top-k] (still on the device)."""
        rt = getattr(self.model, "last_routing", None)
        self.model.last_routing = None
        if not rt:
            return None
        return torch.stack([r.to(torch.int16) for r in rt], dim=1)

    def _routermap(self, s) -> "np.ndarray | None":
        chunks = getattr(s, "route_chunks", None)
        if not chunks:
            return None
        rm = np.concatenate(chunks, axis=0)
        n = len(s.prompt) + len(s.out.token_ids)
        out = np.full((n,) + rm.shape[1:], -1, dtype=np.int16)
        out[: min(n, rm.shape[0])] = rm[:n]
        return out

    def _record(self, seqs, toks_h, lps_h) -> None:
        eos = self.cfg.eos_token_id
        for s, tok, lp in zip(seqs, toks_h, lps_h):
            s.out.token_ids.append(tok)
            s.out.logprobs.append(lp)
            s.last_token = tok
            sp = s.params
            if not sp.ignore_eos and (tok == eos or tok in sp.stop_token_ids):
                self._finish(s, "stop", tok)
            elif len(s.out.token_ids) >= sp.max_tokens:
                self._finish(s, "length")

    # ------------------------------------------------------------------ speculative decoding (n-gram drafts)
    def _ngram_draft(self, hist: list, budget: int) -> list:
        """Tokens that followed the most recent earlier occurrence of the history's suffix (longest suffix first)."""
        n = len(hist)
        for m in range(min(self.speculative_ngram_match, n - 1), 0, -1):
            tail = hist[n - m:]
            for start in range(n - m - 1, -1, -1):
                if hist[start:start + m] == tail:
                    return hist[start + m:start + m + budget]
        return []

    def _speculate(self, seqs) -> set:
        """Verify n-gram drafts of the sequences that have one; returns the ids of the sequences handled here.
        Position i of a verified run is sampled with the parameters and the random counter plain decoding would use for
        that token, so an accepted draft token IS the token plain decoding would have produced; the first sampled token
        that differs from its draft replaces it and ends the run. Every verified sequence gains at least one token."""
        from ..ops import paged as P
        work = []
        for s in seqs:
            if s.params.repetition_penalty != 1.0 or s.rope_delta:
                continue
            budget = min(self.speculative_ngram, s.params.max_tokens - len(s.out.token_ids) - 1)
            if budget <= 0:
                continue
            d = self._ngram_draft(s.prompt + s.out.token_ids, budget)
            if not d:
                continue
            need = (s.length + 1 + len(d) + PAGE - 1) // PAGE - len(s.pages)
            if need > 0:
                if self.cache.num_free() - len(self.running) < need:
                    continue                      # no room for the draft's keys: this sequence decodes normally
                s.pages.extend(self.cache.alloc(need))
            work.append((s, d))
        if not work:
            return set()
        toks = [torch.tensor([s.last_token] + d, dtype=torch.int32) for s, d in work]
        batch = PackedBatch.from_sequences(toks, self.device)
        lens = [int(t.numel()) for t in toks]
        past = [s.length for s, _ in work]
        batch.position_ids = batch.position_ids + torch.cat([torch.full((n,), p, dtype=torch.int32) for n, p in zip(lens, past)]).to(self.device)
        batch.max_seqlen = max(p + n for p, n in zip(past, lens))
        tok_seq = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(lens)]).to(self.device)
        rows = torch.arange(sum(lens), device=self.device)
        logits = self.model.prefill(batch, self.cache, tok_seq, batch.position_ids, self._block_table([s for s, _ in work]), rows,
                                    past_lens=past)
        rep = [s for (s, _), n in zip(work, lens) for _ in range(n)]
        t, k, p, _ = self._sampling_tensors(rep)
        ctr = torch.tensor([len(s.out.token_ids) + i + 7919 * (s.rid + 1) for (s, _), n in zip(work, lens) for i in range(n)],
                           dtype=torch.int32).to(self.device)
        out_t, out_lp = P.sample(logits, t, k, p, seed=self.seed, counters=ctr, logprobs_mode=self.logprobs_mode)
        out_t, out_lp = out_t.cpu().tolist(), out_lp.cpu().tolist()
        off = 0
        for (s, d), n in zip(work, lens):
            accepted = 0
            for i in range(n):
                tok = out_t[off + i]
                self._record([s], [tok], [out_lp[off + i]])
                s.length += 1
                if s.done or i >= len(d) or tok != d[i]:
                    break
                accepted += 1
            off += n
            self.stats["spec_draft_tokens"] = self.stats.get("spec_draft_tokens", 0) + len(d)
            self.stats["spec_accepted_tokens"] = self.stats.get("spec_accepted_tokens", 0) + accepted
            m = s.out.spec_decode_metrics
            if m is None:
                from .params import SpecDecodeMetrics
                m = s.out.spec_decode_metrics = SpecDecodeMetrics()
            m.num_draft_tokens += len(d)
            m.num_accepted_tokens += accepted
            m.num_completions += 1
            self.stats["decode_tokens"] += accepted + 1
        self.stats["spec_verify_steps"] = self.stats.get("spec_verify_steps", 0) + 1
        return {id(s) for s, _ in work}

    def _decode(self) -> None:
        everyone = self.running
        if self.speculative_ngram > 0 and self._cached_ok and not self.capture_routing:
            handled = self._speculate(everyone)
            if handled:
                rest = [s for s in everyone if id(s) not in handled]
                self.running = rest                   # the plain path below sees only the sequences without a draft
                if rest:
                    self._decode_plain()
                self.running = [s for s in everyone if not s.done and (id(s) in handled or s in self.running)]
                return
        self._decode_plain()

    def _decode_plain(self) -> None:
        seqs = self.running
        # make room for the token about to be written
        for s in seqs:
            if s.length + 1 > len(s.pages) * PAGE:
                if self.cache.num_free() == 0:
                    self._preempt_one()
                    return
                s.pages.extend(self.cache.alloc(1))
        if (self.use_cuda_graph and all(s.params.repetition_penalty == 1.0 for s in seqs)
                and max(len(s.pages) for s in seqs) <= self.max_pages_per_seq):
            toks_h, lps_h = self._decode_graph(seqs)
            for s in seqs:
                s.length += 1
            self.stats["decode_tokens"] += len(seqs)
            self.stats["decode_steps"] += 1
            self._record(seqs, toks_h, lps_h)
            self.running = [s for s in seqs if not s.done]
            return
        tokens = torch.tensor([s.last_token for s in seqs], dtype=torch.int32).to(self.device)
        pos = torch.tensor([s.length for s in seqs], dtype=torch.int32).to(self.device)
        bt = self._block_table(seqs)
        if self.capture_routing:
            self.model.last_routing = None
        if any(s.rope_delta for s in seqs):
            delta = torch.tensor([s.rope_delta for s in seqs], dtype=torch.int32).to(self.device)
            logits = self.model.decode(tokens, pos, self.cache, bt, pos + 1, rope_positions=pos + delta)
        else:
            logits = self.model.decode(tokens, pos, self.cache, bt, pos + 1)
        if self.capture_routing:
            rt = self._take_routing()
            if rt is not None:
                rt_h = rt.cpu().numpy()
                for i, s in enumerate(seqs):
                    s.route_chunks.append(rt_h[i:i + 1].copy())
        for s in seqs:
            s.length += 1
        self.stats["decode_tokens"] += len(seqs)
        self.stats["decode_steps"] += 1
        self._sample_and_record(seqs, logits)
        self.running = [s for s in seqs if not s.done]

    def _preempt_one(self) -> None:
        """Out of pages: push the youngest running sequence back to the queue (recompute later)."""
        s = self.running.pop()
        self.cache.release(s.pages)
        s.pages, s.length = [], 0
        s.share_key, s.shared_pages = -1, 0
        self.waiting.appendleft(s)
        self.stats["preempted"] += 1

    @torch.no_grad()
    def step(self) -> None:
        """One scheduler iteration: admit + prefill new sequences if possible, else decode."""
        assert self.cache is not None, "engine is asleep; call wake_up() first"
        self.step_count += 1
        if self.paused and self.pause_strategy == "hold":
            return
        begin = getattr(self.model, "begin_step", None)
        if begin is not None:
            begin()                      # a sharded model lines its group's streams up before the step's collectives
        if not (self.paused and self.pause_strategy in ("drain", "reset")):
            new = self._admit()
            if new:
                self._prefill(new)
                return
        if self.running:
            self._decode()
        elif (self.waiting or self.prefilling) and not self.paused:
            raise MemoryError("a waiting request does not fit the KV pool even when it is empty")
