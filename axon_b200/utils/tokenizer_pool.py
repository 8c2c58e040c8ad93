"""Process pool of tokenizers for asynchronous, high-concurrency tokenisation
(reference: axon/utils/tokenizer_pool.py:200-566).

Every worker process builds its own tokenizer once (from ``tokenizer_path`` through
``hf_tokenizer``, so a directory without tokenizer files yields the byte tokenizer). The async methods
hand work to the pool without blocking the event loop; batch calls are split across workers. The
``*_sync`` variants serve callers outside an event loop. ``encode_with_strs`` also returns the
surface string of every token, which the prefix tree stores for text-level prefix matching.
"""
from __future__ import annotations

import asyncio
import multiprocessing as mp
import os
from concurrent.futures import ProcessPoolExecutor

_worker_tok = None


def _init_worker(path: str, kwargs: dict) -> None:
    global _worker_tok
    from .tokenizer import hf_tokenizer
    _worker_tok = hf_tokenizer(path, **kwargs)


def _encode(text: str, add_special_tokens: bool = False):
    return _worker_tok.encode(text, add_special_tokens=add_special_tokens) if _accepts_special(_worker_tok) else _worker_tok.encode(text)


def _accepts_special(tok) -> bool:
    import inspect
    try:
        return "add_special_tokens" in inspect.signature(tok.encode).parameters
    except (TypeError, ValueError):
        return False


def _encode_with_strs(text: str, add_special_tokens: bool = False):
    if hasattr(_worker_tok, "encode_with_strs"):
        return _worker_tok.encode_with_strs(text)
    ids = _encode(text, add_special_tokens)
    return ids, [_worker_tok.decode([i]) for i in ids]


def _decode(ids, skip_special_tokens: bool = False):
    try:
        return _worker_tok.decode(list(ids), skip_special_tokens=skip_special_tokens)
    except TypeError:
        return _worker_tok.decode(list(ids))


def _batch(fn_name: str, items: list, arg):
    fn = {"encode": _encode, "encode_with_strs": _encode_with_strs, "decode": _decode}[fn_name]
    return [fn(x, arg) for x in items]


class TokenizerPool:
    def __init__(self, tokenizer, tokenizer_path: str | None = None, num_workers: int | None = None,
                 tokenizer_kwargs: dict | None = None):
        self.tokenizer = tokenizer
        self._path = tokenizer_path or getattr(tokenizer, "name_or_path", None)
        if self._path is None:
            raise ValueError("tokenizer_path is required (the tokenizer has no name_or_path)")
        self._kwargs = dict(tokenizer_kwargs or {})
        self._n = num_workers or min(8, os.cpu_count() or 4)
        self._exec: ProcessPoolExecutor | None = None
        self._started = False

    # attributes of the in-process tokenizer (no IPC)
    num_workers = property(lambda self: self._n)
    eos_token_id = property(lambda self: self.tokenizer.eos_token_id)
    pad_token_id = property(lambda self: self.tokenizer.pad_token_id)
    bos_token_id = property(lambda self: getattr(self.tokenizer, "bos_token_id", None))
    vocab_size = property(lambda self: self.tokenizer.vocab_size)

    def _ensure(self) -> ProcessPoolExecutor:
        if self._exec is None:
            self._exec = ProcessPoolExecutor(max_workers=self._n, mp_context=mp.get_context("spawn"),
                                             initializer=_init_worker, initargs=(self._path, self._kwargs))
        return self._exec

    async def start(self) -> None:
        if self._started:
            return
        loop = asyncio.get_running_loop()
        ex = self._ensure()
        await asyncio.gather(*(loop.run_in_executor(ex, _encode, "warmup", False) for _ in range(self._n)))
        self._started = True

    def start_sync(self) -> None:
        if not self._started:
            list(self._ensure().map(_encode, ["warmup"] * self._n))
            self._started = True

    async def shutdown(self, wait: bool = True) -> None:
        self.shutdown_sync(wait)

    def shutdown_sync(self, wait: bool = True) -> None:
        if self._exec is not None:
            self._exec.shutdown(wait=wait, cancel_futures=not wait)
            self._exec = None
        self._started = False

    # ---- async API
    async def _run(self, fn, *args):
        return await asyncio.get_running_loop().run_in_executor(self._ensure(), fn, *args)

    async def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        return await self._run(_encode, text, add_special_tokens)

    async def encode_with_strs(self, text: str, add_special_tokens: bool = False):
        return await self._run(_encode_with_strs, text, add_special_tokens)

    async def decode(self, ids, skip_special_tokens: bool = False) -> str:
        return await self._run(_decode, list(ids), skip_special_tokens)

    def _chunks(self, items: list):
        n = max(1, min(self._n, len(items)))
        size = -(-len(items) // n)
        return [items[i:i + size] for i in range(0, len(items), size)]

    async def _batch(self, name: str, items: list, arg):
        if not items:
            return []
        parts = await asyncio.gather(*(self._run(_batch, name, chunk, arg) for chunk in self._chunks(list(items))))
        return [x for part in parts for x in part]

    async def batch_encode(self, texts: list[str], add_special_tokens: bool = False):
        return await self._batch("encode", texts, add_special_tokens)

    async def batch_encode_with_strs(self, texts: list[str], add_special_tokens: bool = False):
        return await self._batch("encode_with_strs", texts, add_special_tokens)

    async def batch_decode(self, id_lists, skip_special_tokens: bool = False):
        return await self._batch("decode", [list(x) for x in id_lists], skip_special_tokens)

    # ---- sync API
    def encode_sync(self, text: str, add_special_tokens: bool = False) -> list[int]:
        return self._ensure().submit(_encode, text, add_special_tokens).result()

    def encode_with_strs_sync(self, text: str, add_special_tokens: bool = False):
        return self._ensure().submit(_encode_with_strs, text, add_special_tokens).result()

    def decode_sync(self, ids, skip_special_tokens: bool = False) -> str:
        return self._ensure().submit(_decode, list(ids), skip_special_tokens).result()

    def batch_encode_sync(self, texts: list[str], add_special_tokens: bool = False):
        futs = [self._ensure().submit(_batch, "encode", c, add_special_tokens) for c in self._chunks(list(texts))] if texts else []
        return [x for f in futs for x in f.result()]

    def batch_decode_sync(self, id_lists, skip_special_tokens: bool = False):
        items = [list(x) for x in id_lists]
        futs = [self._ensure().submit(_batch, "decode", c, skip_special_tokens) for c in self._chunks(items)] if items else []
        return [x for f in futs for x in f.result()]

    def __del__(self):
        try:
            self.shutdown_sync(wait=False)
        except Exception:
            pass
