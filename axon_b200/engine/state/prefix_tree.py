"""Token prefix tree that records multi-turn rollouts.

Every generate call of a session inserts its full token path (prompt + response); turns that share
history share nodes, so each token is stored — and later trained — once. A node keeps the token id,
the exact text the token stands for, the SET of masks it was seen with (0 = context, 1 = generated),
the smallest step index that touched it, its sampling log-prob and an optional MoE routing record.

Merge rules on re-insertion (reference: axon/engine/state/prefix_tree.py:100-167): masks are united,
the minimum step index wins, a missing token string is back-filled, multimodal data is only replaced
by non-null data, and a routing record is only replaced when the stored one is empty or all -1 while
the new one is valid. ``longest_text_prefix`` matches rendered text against the stored token strings
(longest-child-first) so that re-tokenising a conversation never changes recorded history; expanded
multimodal placeholder runs are skipped as a unit (``prefix_tree.py:288-376``).
"""
from __future__ import annotations

import itertools

import torch

_uid = itertools.count(1)


def _has_entries(rm) -> bool:
    if rm is None:
        return False
    if isinstance(rm, torch.Tensor):
        return rm.numel() > 0
    return hasattr(rm, "__len__") and len(rm) > 0


def _is_all_neg1(rm) -> bool:
    """True when a routing record holds only -1 (the 'no routing known' padding)."""
    try:
        if isinstance(rm, torch.Tensor):
            return rm.numel() > 0 and bool((rm == -1).all())
        if hasattr(rm, "tolist"):
            rm = rm.tolist()
        if isinstance(rm, (list, tuple)):
            return len(rm) > 0 and all(_is_all_neg1(x) if isinstance(x, (list, tuple)) else x == -1 for x in rm)
        return rm == -1
    except (TypeError, AttributeError):
        return False


class PrefixTreeNode:
    __slots__ = ("uid", "token_id", "token_str", "masks", "logprob", "moe_routermap", "step_idx", "children",
                 "multi_modal_data", "mm_expansion_count", "mm_content_hash")

    def __init__(self, token_id, token_str, mask, logprob, moe_routermap=None, step_idx=-1, multi_modal_data=None):
        self.uid = next(_uid)
        self.token_id = token_id
        self.token_str = token_str
        self.masks = {mask}
        self.logprob = logprob
        self.moe_routermap = moe_routermap if moe_routermap is not None else []
        self.step_idx = step_idx
        self.children: dict[int, PrefixTreeNode] = {}
        self.multi_modal_data = multi_modal_data
        self.mm_expansion_count = 0     # > 0 on the first token of an expanded image/video placeholder run
        self.mm_content_hash = ""

    def __hash__(self):
        return self.uid

    def get_child(self, token_id):
        return self.children.get(token_id)

    def is_leaf(self) -> bool:
        return not self.children

    def _merge(self, token_str, mask, moe_routermap, step_idx, multi_modal_data) -> None:
        self.masks.add(mask)
        if step_idx != -1:
            self.step_idx = step_idx if self.step_idx == -1 else min(self.step_idx, step_idx)
        if token_str and not self.token_str:
            self.token_str = token_str
        if multi_modal_data is not None:
            self.multi_modal_data = multi_modal_data
        if _has_entries(moe_routermap):
            if not _has_entries(self.moe_routermap) or (_is_all_neg1(self.moe_routermap) and not _is_all_neg1(moe_routermap)):
                self.moe_routermap = moe_routermap

    def add_child(self, token_id, token_str, mask, logprob, moe_routermap=None, step_idx=-1, multi_modal_data=None):
        node = self.children.get(token_id)
        if node is None:
            node = self.children[token_id] = PrefixTreeNode(token_id, token_str, mask, logprob, moe_routermap,
                                                            step_idx, multi_modal_data)
        else:
            node._merge(token_str, mask, moe_routermap, step_idx, multi_modal_data)
        return node


class PrefixTree:
    def __init__(self):
        self.clear()

    def clear(self) -> None:
        self.root = PrefixTreeNode(token_id=-1, token_str="", mask=-1, logprob=0.0)

    def insert(self, token_ids, token_strs, masks, logprobs, moe_routermaps=None, step_idx=-1,
               multi_modal_data=None, mm_expansions=None) -> PrefixTreeNode:
        """Insert one path; returns its last node. ``moe_routermaps`` may be a tensor
        ``[len, layers, top_k]`` or a per-token list. ``mm_expansions``: (position, count, hash) triples
        marking where an expanded multimodal placeholder run starts."""
        n = len(token_ids)
        if isinstance(moe_routermaps, torch.Tensor):
            assert len(moe_routermaps) == n, f"moe_routermaps length {len(moe_routermaps)} != {n} tokens"
            rms = list(moe_routermaps)
        else:
            rms = list(moe_routermaps) if moe_routermaps else [None] * n
        assert len(token_strs) == len(masks) == len(logprobs) == len(rms) == n, "All inputs must be same length"
        marks = {pos: (cnt, h) for pos, cnt, h in (mm_expansions or [])}
        node = self.root
        for i in range(n):
            node = node.add_child(token_ids[i], token_strs[i], masks[i], logprobs[i], rms[i], step_idx,
                                  multi_modal_data if i == n - 1 else None)
            if i in marks:
                node.mm_expansion_count, node.mm_content_hash = marks[i]
        return node

    def size(self) -> int:
        count, stack = -1, [self.root]
        while stack:
            node = stack.pop()
            count += 1
            stack.extend(node.children.values())
        return count

    def longest_prefix(self, token_ids) -> list[int]:
        out, node = [], self.root
        for t in token_ids:
            node = node.get_child(t)
            if node is None:
                break
            out.append(node.token_id)
        return out

    def longest_text_prefix(self, text: str, mm_regions=None):
        """Returns (token_ids, token_strs, chars_matched, recovered_mm). ``mm_regions`` are
        (text_start, text_end, modality, content_hash, data) tuples for placeholders inside ``text``."""
        mm_at = {s: (e, mod, h, data) for s, e, mod, h, data in (mm_regions or [])}
        node, pos = self.root, 0
        ids, strs, recovered = [], [], []
        while pos < len(text) and node.children:
            run = None
            if pos in mm_at:
                run = next((c for c in node.children.values() if c.mm_expansion_count > 0), None)
            if run is not None:
                end, modality, chash, data = mm_at[pos]
                if run.mm_content_hash and chash != run.mm_content_hash:
                    break                       # different image/video: the suffix is re-tokenised
                cur = run
                ids.append(cur.token_id)
                strs.append(cur.token_str)
                for _ in range(1, run.mm_expansion_count):
                    nxt = cur.get_child(cur.token_id)
                    if nxt is None:
                        break
                    cur = nxt
                    ids.append(cur.token_id)
                    strs.append(cur.token_str)
                pos, node = end, cur
                recovered.append((modality, data))
                continue
            best = None
            for c in node.children.values():
                s = c.token_str
                if s and (best is None or len(s) > len(best.token_str)) and text.startswith(s, pos):
                    best = c
            if best is None:
                break
            ids.append(best.token_id)
            strs.append(best.token_str)
            pos += len(best.token_str)
            node = best
        return ids, strs, pos, recovered

    def __repr__(self) -> str:
        def fmt(n):
            if n.token_id == -1:
                return "ROOT"
            return (f"(id={n.token_id}, str={n.token_str!r}, logprob={n.logprob:.4f}, "
                    f"masks={{{','.join(map(str, sorted(n.masks)))}}}, step_idx={n.step_idx})")
        lines = ["PrefixTree:", fmt(self.root)]
        stack = [(self.root, "")]
        while stack:
            node, indent = stack.pop()
            kids = list(node.children.values())
            while len(kids) == 1:               # straight runs print vertically
                lines += [indent + "  ↓", indent + fmt(kids[0])]
                node, kids = kids[0], list(kids[0].children.values())
            for i, c in reversed(list(enumerate(kids))):
                last = i == len(kids) - 1
                stack.append((c, indent + ("      " if last else "  │   ")))
            for i, c in enumerate(kids):
                lines.append(indent + ("  └─→ " if i == len(kids) - 1 else "  ├─→ ") + fmt(c))
        return "\n".join(lines)
