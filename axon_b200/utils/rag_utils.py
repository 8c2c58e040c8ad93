"""Embedding retrieval over a fixed list of documents (reference: ``RAG``, axon/utils/rag_utils.py:20-69).

``RAG(docs).top_k(query, k)`` returns the k most similar documents by cosine similarity as
``[{"score", "text", "idx"}]``. The encoder is a SentenceTransformer when that package and the model are
available; otherwise (air-gapped boxes) a deterministic hashed character-n-gram embedding, which keeps the
tool usable for lexical retrieval without any download.
"""
from __future__ import annotations

import hashlib

import torch

__all__ = ["RAG", "HashedNgramEncoder"]


class HashedNgramEncoder:
    """L2-normalised bag of hashed character n-grams (n = 3..5) plus word unigrams."""

    def __init__(self, dim: int = 4096):
        self.dim = dim

    def _features(self, text: str):
        t = " ".join(text.lower().split())
        for w in t.split(" "):
            yield "w:" + w
        for n in (3, 4, 5):
            for i in range(max(0, len(t) - n + 1)):
                yield t[i:i + n]

    def encode(self, texts, convert_to_tensor: bool = True):
        single = isinstance(texts, str)
        items = [texts] if single else list(texts)
        out = torch.zeros(len(items), self.dim)
        for r, text in enumerate(items):
            for f in self._features(text):
                h = int.from_bytes(hashlib.blake2b(f.encode(), digest_size=8).digest(), "little")
                out[r, h % self.dim] += 1.0 if (h >> 63) == 0 else -1.0
        out = torch.nn.functional.normalize(out, dim=-1)
        return out[0] if single else out


class RAG:
    def __init__(self, docs: list[str], model: str = "sentence-transformers/all-MiniLM-L6-v2", encoder=None):
        self.docs = list(docs)
        if encoder is None:
            try:
                from sentence_transformers import SentenceTransformer
                encoder = SentenceTransformer(model)
            except Exception:  # noqa: BLE001 - package or model files unavailable
                encoder = HashedNgramEncoder()
        self.model = encoder
        self.embeddings = torch.as_tensor(self.model.encode(self.docs, convert_to_tensor=True)).float()

    def top_k(self, query: str, k: int = 1) -> list[dict]:
        q = torch.as_tensor(self.model.encode(query, convert_to_tensor=True)).float().reshape(1, -1)
        e = self.embeddings.to(q.device)
        scores = torch.nn.functional.cosine_similarity(q, e, dim=-1)
        top = torch.topk(scores, k=min(k, len(self.docs)))
        return [{"score": s, "text": self.docs[int(i)], "idx": int(i)} for s, i in zip(top.values, top.indices)]
