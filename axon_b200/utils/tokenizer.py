"""Tokenizer access. ``hf_tokenizer(path)`` loads a HuggingFace tokenizer when its files exist
(reference: axon/utils/tokenizer.py:39); ``ByteTokenizer`` is a dependency-free UTF-8 byte tokenizer
with ChatML-style special tokens, used by synthetic runs and tests. Both expose the small interface
the engine needs: ``encode``, ``decode``, ``encode_with_strs`` (ids plus the exact text of every
token), ``eos_token_id`` and ``pad_token_id``."""
from __future__ import annotations

import os
import re


class ByteTokenizer:
    SPECIALS = ["<|pad|>", "<|endoftext|>", "<|im_start|>", "<|im_end|>", "<|begin_of_text|>", "<|eot_id|>",
                "<|start_header_id|>", "<|end_header_id|>", "<think>", "</think>", "<tool_call>", "</tool_call>",
                "<tool_response>", "</tool_response>", "<|image_pad|>", "<|vision_start|>", "<|vision_end|>"]

    def __init__(self, vocab_size: int = 512, eos_token: str = "<|im_end|>"):
        self.special_to_id = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self.id_to_special = {v: k for k, v in self.special_to_id.items()}
        self.vocab_size = max(vocab_size, 256 + len(self.SPECIALS))
        self.eos_token, self.pad_token = eos_token, "<|pad|>"
        self.eos_token_id = self.special_to_id[eos_token]
        self.pad_token_id = self.special_to_id["<|pad|>"]
        self.bos_token_id = None
        self._split = re.compile("(" + "|".join(re.escape(s) for s in sorted(self.SPECIALS, key=len, reverse=True)) + ")")
        self.name_or_path = "byte-tokenizer"

    def __len__(self):
        return self.vocab_size

    def encode_with_strs(self, text: str):
        ids, strs = [], []
        for part in self._split.split(text):
            if not part:
                continue
            if part in self.special_to_id:
                ids.append(self.special_to_id[part])
                strs.append(part)
                continue
            for ch in part:                       # one token per byte; the token string of a multi-byte
                b = ch.encode("utf-8")            # character rides on its first byte
                ids.extend(b)
                strs.extend([ch] + [""] * (len(b) - 1))
        return ids, strs

    def encode(self, text: str, add_special_tokens: bool = False):
        return self.encode_with_strs(text)[0]

    def __call__(self, text, add_special_tokens: bool = False, **kw):
        if isinstance(text, str):
            return {"input_ids": self.encode(text)}
        return {"input_ids": [self.encode(t) for t in text]}

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        out, buf = [], bytearray()
        for i in ids:
            i = int(i)
            if i < 256:
                buf.append(i)
                continue
            if buf:
                out.append(buf.decode("utf-8", errors="replace"))
                buf = bytearray()
            if i in self.id_to_special and not skip_special_tokens:
                out.append(self.id_to_special[i])
        if buf:
            out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)

    def convert_ids_to_tokens(self, ids):
        return [self.id_to_special.get(int(i), bytes([int(i)]).decode("latin-1") if int(i) < 256 else f"<{i}>") for i in ids]

    def token_strs(self, ids) -> list[str]:
        """Per-token text whose concatenation equals ``decode(ids)`` for complete UTF-8 sequences."""
        strs, pend, pend_n = [], bytearray(), 0
        for i in ids:
            i = int(i)
            if i >= 256:
                strs.append(self.id_to_special.get(i, ""))
                continue
            pend.append(i)
            pend_n += 1
            try:
                ch = pend.decode("utf-8")
                strs.extend([ch] + [""] * (pend_n - 1))
                pend, pend_n = bytearray(), 0
            except UnicodeDecodeError:
                if pend_n >= 4:
                    strs.extend(["�"] + [""] * (pend_n - 1))
                    pend, pend_n = bytearray(), 0
        strs.extend([""] * pend_n)
        return strs


class HFTokenizerAdapter:
    """Adds ``encode_with_strs`` / ``token_strs`` to a HuggingFace fast tokenizer (offset-based)."""

    def __init__(self, tok):
        self.tok = tok
        self.eos_token_id, self.pad_token_id = tok.eos_token_id, tok.pad_token_id if tok.pad_token_id is not None else tok.eos_token_id
        self.bos_token_id = tok.bos_token_id
        self.eos_token, self.pad_token = tok.eos_token, tok.pad_token
        self.vocab_size = len(tok)
        self.name_or_path = getattr(tok, "name_or_path", "")

    def __len__(self):
        return self.vocab_size

    def __getattr__(self, name):
        return getattr(self.tok, name)

    def encode(self, text, add_special_tokens=False):
        return self.tok.encode(text, add_special_tokens=add_special_tokens)

    def decode(self, ids, skip_special_tokens=False):
        return self.tok.decode(ids, skip_special_tokens=skip_special_tokens)

    def encode_with_strs(self, text):
        enc = self.tok(text, add_special_tokens=False, return_offsets_mapping=True)
        ids, offs = enc["input_ids"], enc["offset_mapping"]
        strs, last = [], 0
        for s, e in offs:
            s = max(s, last)          # byte-fallback pieces can overlap; each character is emitted once
            strs.append(text[s:e] if e > s else "")
            last = max(last, e)
        return ids, strs

    def token_strs(self, ids):
        out, prev = [], ""
        for i in range(len(ids)):
            cur = self.tok.decode(ids[: i + 1], skip_special_tokens=False)
            if cur.endswith("�"):
                out.append("")
                continue
            out.append(cur[len(prev):])
            prev = cur
        return out


def hf_tokenizer(name_or_path: str, correct_pad_token: bool = True, **kwargs):
    """A HuggingFace tokenizer if ``name_or_path`` has tokenizer files, else the byte tokenizer."""
    has_files = os.path.isdir(name_or_path) and any(
        os.path.exists(os.path.join(name_or_path, f)) for f in ("tokenizer.json", "tokenizer.model", "vocab.json"))
    if not has_files:
        return ByteTokenizer()
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(name_or_path, **kwargs)
    if correct_pad_token and tok.pad_token_id is None:
        tok.pad_token = tok.eos_token
    return HFTokenizerAdapter(tok)
