"""Per-program rollout state: steps, the token prefix tree, rewards, and the extraction of training
rows from the tree.

Training extraction (reference: axon/engine/state/program_state.py:358-471) is an iterative DFS that
yields ONE ``Step`` per leaf. When a node has several children, the first child's path keeps the
masks accumulated so far and every other child's path gets its shared prefix masked to 0, so a token
on a shared prefix is trained in exactly one leaf. A node's mask is the max of the masks it was seen
with; a step's ``order_idx`` is the largest step index on its path.
"""
from __future__ import annotations

import asyncio
import math
import threading
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Mapping

import torch

from .prefix_tree import PrefixTree, _has_entries


class StopPartialProgram(Exception):
    """Raised inside a program to stop at a partial-rollout boundary (resumed next step)."""


class StopProgram(Exception):
    """Raised inside a program to signal that it has terminated."""


@dataclass
class MultiModalData:
    image: list | None = None
    video: list | None = None
    processor_kwargs: Mapping[str, Any] = field(default_factory=dict)


class ModelStopReason:
    LENGTH = "length"
    STOP = "stop"


@dataclass
class ModelOutput:
    response: str
    token_ids: list
    logprobs: list
    stop_reason: str
    moe_routermap: Any = field(default_factory=list)   # [n_tokens, n_moe_layers, top_k] or []
    token_strs: list = field(default_factory=list)
    spec_decode_metrics: object | None = None

    @classmethod
    def from_token_strs(cls, *, token_ids, token_strs, logprobs, stop_reason, moe_routermap, spec_decode_metrics=None):
        """The response text is the exact concatenation of the sampler's per-token strings."""
        return cls("".join(token_strs), token_ids, logprobs, stop_reason, moe_routermap, token_strs, spec_decode_metrics)


class TerminationReason(Enum):
    PROMPT_TRUNCATION = "PROMPT_TRUNCATION"
    MAX_STEPS = "MAX_STEPS"
    PROGRAM_TIMEOUT = "PROGRAM_TIMEOUT"
    TRUNCATION = "TRUNCATION"
    ENV_DONE = "ENV_DONE"
    ENV_TIMEOUT = "ENV_TIMEOUT"
    INTERNAL_ERROR = "INTERNAL_ERROR"
    BAD_PROGRAM = "BAD_PROGRAM"


@dataclass
class ProgramMetrics:
    steps: int = 0
    reward_time: float | None = None
    env_time: float = 0.0
    llm_time: float = 0.0
    total_time: float = 0.0
    spec_draft_tokens: int = 0
    spec_accepted_tokens: int = 0
    spec_verify_count: int = 0


@dataclass
class Step:
    uid: str
    session_id: str
    chat_completions: list = field(default_factory=list)
    reward: float = 0
    order_idx: int = -1
    sample_params: dict = field(default_factory=dict)
    text: str = ""
    tokens: list = field(default_factory=list)
    token_len: int = 0
    masks: list = field(default_factory=list)
    logprobs: list = field(default_factory=list)
    moe_routermap: Any = field(default_factory=list)
    multi_modal_data: MultiModalData | None = None
    # partial-rollout scratch: a response generated over several driver steps
    partial_rollout_max_tokens: int = 0
    partial_tokens: list = field(default_factory=list)
    partial_text: str = ""
    partial_logprobs: list = field(default_factory=list)
    partial_moe_routermap: Any = field(default_factory=list)
    partial_token_strs: list = field(default_factory=list)
    response_token_strs: list = field(default_factory=list)

    def check_empty_partial(self) -> bool:
        return not self.partial_tokens and not self.partial_text and not self.partial_logprobs

    def mask_out_response(self) -> None:
        assert self.check_empty_partial(), "Partial response should be empty when masking out existing responses"
        self.masks = [0] * len(self.tokens)
        self.logprobs = [0] * len(self.tokens)

    def set_response(self, text, tokens, masks, logprobs, moe_routermap) -> None:
        """Append a committed response chunk. A routing record shorter than the token stream (prefix-cache
        hit) keeps the already-stored head, padding missing rows with -1; a longer one is truncated."""
        assert len(tokens) == len(masks) == len(logprobs), \
            f"All inputs require same length: {len(tokens)}, {len(masks)}, {len(logprobs)}"
        self.text += text
        self.tokens.extend(tokens)
        self.token_len += len(tokens)
        self.masks.extend(masks)
        self.logprobs.extend(logprobs)
        if not _has_entries(moe_routermap):
            self.moe_routermap = moe_routermap
            return
        want, have = len(self.tokens), len(moe_routermap)
        if have == want:
            self.moe_routermap = moe_routermap
        elif have > want:
            self.moe_routermap = moe_routermap[:want]
        else:
            missing = want - have
            old = self.moe_routermap if _has_entries(self.moe_routermap) else None
            if isinstance(moe_routermap, torch.Tensor):
                head = old[:missing] if isinstance(old, torch.Tensor) else moe_routermap.new_empty((0, *moe_routermap.shape[1:]))
                if len(head) < missing:
                    pad = torch.full((missing - len(head), *moe_routermap.shape[1:]), -1, dtype=moe_routermap.dtype,
                                     device=moe_routermap.device)
                    head = torch.cat([head, pad], 0)
                self.moe_routermap = torch.cat([head, moe_routermap], 0)
            else:
                head = list(old[:missing]) if old is not None else []
                if len(head) < missing:
                    template = moe_routermap[0]
                    neg = [[-1] * len(r) for r in template] if template and isinstance(template[0], (list, tuple)) \
                        else [-1] * len(template)
                    head = head + [neg] * (missing - len(head))
                self.moe_routermap = head + list(moe_routermap)

    def reset_partial_state(self) -> None:
        self.partial_tokens, self.partial_logprobs, self.partial_moe_routermap = [], [], []
        self.partial_token_strs, self.partial_text = [], ""

    def reset(self) -> None:
        self.token_len, self.tokens, self.masks, self.text, self.logprobs, self.moe_routermap = 0, [], [], "", [], []
        self.partial_rollout_max_tokens = 0
        self.reset_partial_state()
        self.multi_modal_data = None

    def is_empty(self) -> bool:
        return not any(m > 0 for m in self.masks)


@dataclass
class ProgramState:
    group_id: str = ""
    uid: str = ""
    session_id: str = ""
    metrics: ProgramMetrics = field(default_factory=ProgramMetrics)
    num_steps: int = 0
    global_steps: int = -1
    done: bool = False
    reward: float = 0
    termination_reason: TerminationReason | str | None = None
    sample_params: dict = field(default_factory=dict)
    session_lock: asyncio.Lock | None = None
    last_llm_call_time: float = field(default_factory=time.monotonic)
    enable_partial_rollout: bool = False
    partial_rollout_futures: list = field(default_factory=list)
    steps: list = field(default_factory=list)
    prefix_tree: PrefixTree = field(default_factory=PrefixTree)
    training_steps: list = field(default_factory=list)
    step_rewards: dict = field(default_factory=dict)      # order_idx -> reward, overrides ``reward`` per step
    metadata: dict = field(default_factory=dict)

    def reset(self) -> None:
        self.metrics = ProgramMetrics()
        self.num_steps, self.global_steps, self.termination_reason = 0, -1, None
        self.done, self.reward, self.steps = False, 0, []
        self.prefix_tree = PrefixTree()
        self.session_lock = None
        self.last_llm_call_time = time.monotonic()
        self.partial_rollout_futures, self.step_rewards, self.metadata = [], {}, {}

    def record_env_time(self) -> None:
        dt = time.monotonic() - self.last_llm_call_time
        self.metrics.env_time += dt
        self.metrics.total_time += dt

    def record_llm_call_finish_time(self) -> None:
        self.last_llm_call_time = time.monotonic()

    def get_steps_from_prefix_tree(self) -> list[Step]:
        """One Step per leaf: the tokens on the path from the root. Runs of nodes with a single child extend the
        frame's lists in place (a session is mostly one long chain); lists are copied at branch points only, where
        every sibling but the first zeroes the masks of the shared prefix (it is trained once)."""
        out: list[Step] = []
        # frame: node, ids, strs, logprobs, masks, routermaps, max step idx, multimodal data
        stack = [(self.prefix_tree.root, [], [], [], [], [], -1, None)]
        while stack:
            node, ids, strs, lps, masks, rms, top, mm = stack.pop()
            while len(node.children) == 1:
                (child,) = node.children.values()
                ids.append(child.token_id)
                strs.append(child.token_str)
                lps.append(child.logprob)
                masks.append(max(child.masks))
                rms.append(child.moe_routermap if _has_entries(child.moe_routermap) else None)
                if child.step_idx > top:
                    top = child.step_idx
                if child.multi_modal_data:
                    mm = child.multi_modal_data
                node = child
            if node.is_leaf():
                if ids:
                    out.append(self._leaf_step(ids, strs, lps, masks, rms, top, mm))
                continue
            for k, child in enumerate(node.children.values()):
                rm = child.moe_routermap if _has_entries(child.moe_routermap) else None
                prefix_masks = masks if k == 0 else [0] * len(masks)     # siblings do not re-train the shared prefix
                stack.append((child, ids + [child.token_id], strs + [child.token_str], lps + [child.logprob],
                              prefix_masks + [max(child.masks)], rms + [rm], max(top, child.step_idx),
                              child.multi_modal_data if child.multi_modal_data else mm))
        return out

    def _leaf_step(self, ids, strs, lps, masks, rms, top, mm) -> Step:
        st = Step(uid=self.uid, session_id=self.session_id)
        st.order_idx, st.tokens, st.text, st.token_len = top, ids, "".join(strs), len(ids)
        st.masks, st.logprobs, st.multi_modal_data = masks, lps, mm
        known = [r for r in rms if r is not None]
        if known:
            if isinstance(known[0], torch.Tensor):
                st.moe_routermap = torch.stack([r if r is not None else torch.full_like(known[0], -1) for r in rms])
            else:
                st.moe_routermap = known if len(known) != len(rms) else rms
        return st

    def get_training_steps(self) -> list[Step]:
        """Non-empty steps for training. With per-step rewards the raw steps are used one-to-one."""
        if self.training_steps:
            return self.training_steps
        if self.step_rewards and self.steps:
            return [s for s in self.steps if not s.is_empty()]
        return [s for s in self.get_steps_from_prefix_tree() if not s.is_empty()]

    def is_trainable(self, strict: bool = False) -> bool:
        if not self.done:
            return False
        r = self.reward
        if math.isnan(r) or math.isinf(r) or r >= 1e9 or r <= -1e9:
            return False
        if strict and self.termination_reason not in (TerminationReason.ENV_DONE,):
            return False
        return len(self.get_training_steps()) > 0


class ProgramManager:
    """Thread-safe ``group_id -> {uid -> ProgramState}`` buffer with group-complete popping."""

    def __init__(self):
        self.programs: dict[str, dict[str, ProgramState]] = {}
        self._lock = threading.Lock()

    def add_programs(self, programs) -> None:
        with self._lock:
            for p in programs:
                self.programs.setdefault(p.group_id, {})[p.uid] = p

    def pop_programs(self, completed: bool = False) -> list[ProgramState]:
        """completed=True: pop every program of groups whose programs are ALL done;
        completed=False: pop all programs that are not done."""
        out = []
        with self._lock:
            for gid in list(self.programs):
                grp = self.programs[gid]
                if completed:
                    take = list(grp) if all(p.done for p in grp.values()) else []
                else:
                    take = [u for u, p in grp.items() if not p.done]
                out.extend(grp.pop(u) for u in take)
                if not grp:
                    del self.programs[gid]
        return out

    def _count(self, pred) -> int:
        with self._lock:
            return sum(1 for g in self.programs.values() for p in g.values() if pred(p))

    def get_num_programs(self) -> int:
        return self._count(lambda p: True)

    def get_num_completed_programs(self) -> int:
        return self._count(lambda p: p.done)

    def get_num_incomplete_programs(self) -> int:
        return self._count(lambda p: not p.done)

    def get_completed_programs_statistics(self) -> dict:
        with self._lock:
            done = [p for g in self.programs.values() for p in g.values() if p.done]
            groups_done = sum(1 for g in self.programs.values() if g and all(p.done for p in g.values()))
        rewards = [p.reward for p in done]
        return {"num_completed": len(done), "num_completed_groups": groups_done,
                "mean_reward": sum(rewards) / len(rewards) if rewards else 0.0}
