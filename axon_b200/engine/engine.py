"""Agent execution engine: sessions, prefix-tree recording and budgeted generation.

Programs talk to the engine through three calls — ``init_session``, ``generate(messages)``,
``end_session(reward)`` — either in-process or over HTTP. For every ``generate`` the engine renders
the conversation, re-uses the longest recorded TEXT prefix of the session's prefix tree verbatim (so
re-tokenisation never rewrites history), tokenises only the remainder, samples a continuation under
the sequence-length budget, and inserts prompt + response tokens with masks, log-probs and MoE
routing into the tree. Finished programs are handed to the driver as training steps.

Same behaviour as the reference engine (axon/engine/engine.py:480-1221): termination reasons
(prompt truncation, truncation at ``max_seq_length``, max steps), optional left/right prompt
truncation, per-step token cap, partial rollout (a response may be generated over several driver
iterations of ``max_seq_length_per_iter`` tokens each), routing-record recovery from the tree when
the sampler returned fewer rows than tokens, and -1 padding for the last token's routing row.
"""
from __future__ import annotations

import asyncio
import copy
import threading
import time
import uuid
from typing import Any

import torch

from .chat_template.parser import ChatTemplateParser, TokenizeContext
from .state.prefix_tree import _has_entries
from .state.program_state import (ModelOutput, ModelStopReason, ProgramManager, ProgramState, Step, StopPartialProgram,
                                  StopProgram, TerminationReason)

MM_PART_TYPES = ("image", "image_url", "video", "video_url")


def pad_moe_routermap(rm, n_tokens: int):
    """Pad (with -1 rows) or cut a ``[n, layers, k]`` routing record to ``n_tokens`` rows."""
    if not _has_entries(rm):
        return rm
    if isinstance(rm, torch.Tensor):
        if len(rm) < n_tokens:
            pad = torch.full((n_tokens - len(rm), *rm.shape[1:]), -1, dtype=rm.dtype, device=rm.device)
            return torch.cat([rm, pad], 0)
        return rm[:n_tokens]
    rm = list(rm)
    if len(rm) < n_tokens:
        t = rm[0]
        neg = [[-1] * len(r) for r in t] if t and isinstance(t[0], (list, tuple)) else [-1] * len(t)
        rm = rm + [neg] * (n_tokens - len(rm))
    return rm[:n_tokens]


class Engine:
    def __init__(self, sampling_client=None, tokenizer=None, processor=None, chat_parser: ChatTemplateParser | None = None,
                 max_seq_length: int = 8192, max_prompt_length: int = 1024, max_steps: int = 64,
                 max_tokens_per_step: int | None = None, prompt_truncation: str | None = None,
                 enable_partial_rollout: bool = False, partial_rollout_n_iters: int = 1, moe_replay: bool = False,
                 disable_thinking: bool = False, tool_parser=None, default_sample_params: dict | None = None):
        self.sampling_client = sampling_client
        self.tokenizer, self.processor = tokenizer, processor
        self.chat_parser = chat_parser or ChatTemplateParser.get_parser(tokenizer, processor, disable_thinking, tool_parser)
        self.max_seq_length, self.max_prompt_length = max_seq_length, max_prompt_length
        self.max_steps, self.max_tokens_per_step = max_steps, max_tokens_per_step
        self.prompt_truncation = prompt_truncation
        self.enable_partial_rollout = enable_partial_rollout
        self.max_seq_length_per_iter = max(1, max_seq_length // max(1, partial_rollout_n_iters))
        self.moe_replay = moe_replay
        self.default_sample_params = dict(default_sample_params or {})
        self.global_steps = 0
        self.validation_mode = False
        self.session_state_map: dict[str, ProgramState] = {}
        self.program_manager, self.val_program_manager = ProgramManager(), ProgramManager()
        self._session_state_lock: asyncio.Lock | None = None
        self._loop = asyncio.new_event_loop()
        self._thread = threading.Thread(target=self._run_loop, daemon=True, name="engine-loop")
        self._thread.start()
        self.metrics = {"generate_calls": 0, "prefix_hits": 0, "prefix_tokens_reused": 0, "tokens_tokenized": 0}

    # ------------------------------------------------------------------ loop plumbing
    def _run_loop(self) -> None:
        asyncio.set_event_loop(self._loop)
        self._session_state_lock = asyncio.Lock()
        self._loop.run_forever()

    def run_in_engine_loop(self, coro, timeout: float | None = None):
        """Run a coroutine on the engine's loop from any thread and wait for its result."""
        return asyncio.run_coroutine_threadsafe(coro, self._loop).result(timeout)

    async def run_in_engine_loop_async(self, coro):
        """Await a coroutine that must run on the engine's loop from another event loop."""
        if asyncio.get_running_loop() is self._loop:
            return await coro
        return await asyncio.wrap_future(asyncio.run_coroutine_threadsafe(coro, self._loop))

    def set_global_steps(self, step: int) -> None:
        self.global_steps = step

    def set_validation_mode(self, on: bool) -> None:
        self.validation_mode = on

    async def _lock(self) -> asyncio.Lock:
        while self._session_state_lock is None:
            await asyncio.sleep(0)
        return self._session_state_lock

    # ------------------------------------------------------------------ session API
    async def init_session(self, group_id: str | None = None, sample_params: dict | None = None) -> str:
        sid = str(uuid.uuid4())
        st = ProgramState(session_id=sid, uid=sid)
        st.group_id = group_id if group_id is not None else str(uuid.uuid4())
        st.sample_params = dict(sample_params) if sample_params else {}
        st.global_steps = self.global_steps
        st.session_lock = asyncio.Lock()
        st.enable_partial_rollout = self.enable_partial_rollout and not self.validation_mode
        st.record_llm_call_finish_time()
        async with await self._lock():
            self.session_state_map[sid] = st
        (self.val_program_manager if self.validation_mode else self.program_manager).add_programs([st])
        return sid

    async def generate(self, messages: list[dict], session_id: str, sample_params: dict | None = None, images=None,
                       videos=None, processor_kwargs: dict | None = None, tools_json: list | None = None,
                       parser_kwargs: dict | None = None):
        """Returns (assistant text, stop_program, step index)."""
        async with await self._lock():
            assert session_id in self.session_state_map, f"session_id is not found: {session_id}"
            state = self.session_state_map[session_id]
        state.record_env_time()
        try:
            self.check_state_before_generation(state)
        except StopProgram:
            return "", True, -1
        self.metrics["generate_calls"] += 1
        async with state.session_lock:
            step = Step(uid=str(uuid.uuid4()), session_id=session_id, chat_completions=copy.deepcopy(messages))
            pk = dict(parser_kwargs or {})
            if tools_json:
                pk["tools"] = tools_json
            input_key = self.chat_parser.parse(messages, add_generation_prompt=True, **pk)
            has_mm = bool(images or videos) or any(
                isinstance(m.get("content"), list) and any(isinstance(p, dict) and p.get("type") in MM_PART_TYPES
                                                           for p in m["content"]) for m in messages)
            ctx = TokenizeContext(messages, images or [], videos or [], processor_kwargs or {}) \
                if (self.processor is not None and has_mm) else None
            mm_regions = self.chat_parser.get_mm_regions(input_key, messages) if has_mm else []
            p_ids, p_strs, p_pos, recovered = state.prefix_tree.longest_text_prefix(input_key, mm_regions or None)
            mm = None
            if p_ids:
                self.metrics["prefix_hits"] += 1
                self.metrics["prefix_tokens_reused"] += len(p_ids)
                rest = input_key[p_pos:]
                if rest:
                    new_regions = [r for r in mm_regions if r[0] >= p_pos]
                    sub_ctx = None
                    if new_regions and ctx is not None:
                        sub_ctx = TokenizeContext(None, [r[4] for r in new_regions if r[2] == "image"],
                                                  [r[4] for r in new_regions if r[2] == "video"], ctx.processor_kwargs)
                    out = await self.chat_parser.tokenize(rest, ctx=sub_ctx)
                    s_ids, s_strs, mm = out.token_ids, out.token_strs, out.multi_modal_data
                else:
                    s_ids, s_strs = [], []
                tokens, prompt_strs = p_ids + s_ids, p_strs + s_strs
                self.metrics["tokens_tokenized"] += len(s_ids)
                if recovered and mm is None:
                    from .state.program_state import MultiModalData
                    mm = MultiModalData(image=[d for m_, d in recovered if m_ == "image"] or None,
                                        video=[d for m_, d in recovered if m_ == "video"] or None)
            else:
                out = await self.chat_parser.tokenize(input_key, ctx=ctx)
                tokens, prompt_strs, mm = out.token_ids, out.token_strs, out.multi_modal_data
                self.metrics["tokens_tokenized"] += len(tokens)
            mm_copy = copy.deepcopy(mm) if mm else None
            step.set_response(text=input_key, tokens=tokens, masks=[0] * len(tokens), logprobs=[0.0] * len(tokens),
                              moe_routermap=[])
            if mm:
                step.multi_modal_data = mm
            step.sample_params = copy.deepcopy(sample_params) if sample_params else copy.deepcopy(state.sample_params)

        text, stop_program, stop_partial = await self.generate_llm_response_with_checks(step)
        while stop_partial and not stop_program:
            fut = asyncio.get_running_loop().create_future()
            async with state.session_lock:
                state.partial_rollout_futures.append(fut)
            await fut                                   # resumed by resume_partial_rollout_programs()
            text, stop_program, stop_partial = await self.generate_llm_response_with_checks(step)

        async with state.session_lock:
            step.order_idx = len(state.steps)
            state.steps.append(step)
            state.num_steps += 1
            rms = step.moe_routermap
            if self.moe_replay and _has_entries(rms) and len(rms) != len(step.tokens):
                rms = step.moe_routermap = pad_moe_routermap(rms, len(step.tokens))
            strs = (prompt_strs + list(step.response_token_strs))[: len(step.tokens)]
            strs += [""] * (len(step.tokens) - len(strs))
            state.prefix_tree.insert(token_ids=step.tokens, token_strs=strs, masks=step.masks, logprobs=step.logprobs,
                                     moe_routermaps=rms if _has_entries(rms) else None, step_idx=step.order_idx,
                                     multi_modal_data=mm_copy,
                                     mm_expansions=self._detect_mm_expansions(step.tokens, mm_regions) if mm_regions else None)
            state.record_llm_call_finish_time()
            state.metrics.steps += 1
        return text, stop_program, step.order_idx

    def _detect_mm_expansions(self, tokens, mm_regions):
        """(position, run length, content hash) of each expanded pad-token run, in region order."""
        pad_ids = {self.tokenizer.encode(p)[0] for p in ("<|image_pad|>", "<|video_pad|>")
                   if hasattr(self.tokenizer, "encode") and len(self.tokenizer.encode(p)) == 1}
        runs, i = [], 0
        while i < len(tokens):
            if tokens[i] in pad_ids:
                j = i
                while j < len(tokens) and tokens[j] == tokens[i]:
                    j += 1
                runs.append((i, j - i))
                i = j
            else:
                i += 1
        return [(pos, cnt, region[3]) for (pos, cnt), region in zip(runs, mm_regions)]

    async def end_session(self, session_id: str, reward: float, step_rewards: dict | None = None):
        """Mark a session complete. A second call, or a call on a program the engine already finished
        (prompt truncation), is a no-op. A reward beyond +-1e9 flags the program as bad."""
        async with await self._lock():
            state = self.session_state_map.get(session_id)
            if state is None:
                return {"status": "unknown_session"}
            if state.done:
                return {"status": "already_done"}
            state.record_env_time()
            state.done, state.reward = True, reward
            if step_rewards:
                state.step_rewards = {int(k): float(v) for k, v in step_rewards.items()}
            if reward >= 1e9 or reward <= -1e9:
                state.termination_reason = TerminationReason.BAD_PROGRAM
            elif not state.termination_reason:
                state.termination_reason = TerminationReason.ENV_DONE
            for fut in state.partial_rollout_futures:
                if not fut.done():
                    fut.cancel()
            state.partial_rollout_futures = []
        return {"status": "ok"}

    async def get_engine_metrics(self) -> dict:
        mgr = self.val_program_manager if self.validation_mode else self.program_manager
        return {"engine/pending_programs": mgr.get_num_incomplete_programs(),
                "engine/completed_programs": mgr.get_num_completed_programs(),
                **{f"engine/{k}": v for k, v in mgr.get_completed_programs_statistics().items()},
                **{f"engine/{k}": v for k, v in self.metrics.items()}}

    # ------------------------------------------------------------------ driver-side collection
    async def get_finished_programs(self, validation: bool = False) -> list[ProgramState]:
        """Programs of groups in which EVERY program is done; their sessions are forgotten."""
        mgr = self.val_program_manager if validation else self.program_manager
        done = mgr.pop_programs(completed=True)
        async with await self._lock():
            for p in done:
                self.session_state_map.pop(p.session_id, None)
        return [postprocess_program_state(p) for p in done]

    async def resume_partial_rollout_programs(self) -> int:
        """Wake every session parked at a partial-rollout boundary (called once per driver step)."""
        n = 0
        async with await self._lock():
            states = list(self.session_state_map.values())
        for st in states:
            async with st.session_lock:
                futs, st.partial_rollout_futures = st.partial_rollout_futures, []
            for f in futs:
                if not f.done():
                    f.set_result(True)
                    n += 1
        return n

    async def all_programs_safe_to_collect(self) -> bool:
        """True when no session is mid-generation: each is done or parked at a partial boundary."""
        async with await self._lock():
            return all(st.done or st.partial_rollout_futures for st in self.session_state_map.values())

    async def get_session_diagnostics(self) -> str:
        async with await self._lock():
            vals = list(self.session_state_map.values())
        done = sum(s.done for s in vals)
        partial = sum((not s.done) and bool(s.partial_rollout_futures) for s in vals)
        return f"sessions={len(vals)} done={done} partial={partial} running={len(vals) - done - partial}"

    def get_metrics(self) -> dict:
        return dict(self.metrics)

    async def shutdown(self) -> None:
        self._loop.call_soon_threadsafe(self._loop.stop)

    # ------------------------------------------------------------------ generation with checks
    async def generate_llm_response_with_checks(self, step: Step):
        state = self.session_state_map[step.session_id]
        text, stop_program, stop_partial = "", False, False
        try:
            self.check_state_before_generation(state)
            self.check_prompt_truncation_termination(step)
            self.check_truncation_termination(step, last_assistant_response=False)
            text = await self.generate_llm_response(step)
            self.check_truncation_termination(step, last_assistant_response=True)
        except StopProgram:
            stop_program = True
        except StopPartialProgram:
            step.partial_rollout_max_tokens += self.max_seq_length_per_iter
            stop_partial = True
        return text, stop_program, stop_partial

    async def generate_llm_response(self, step: Step) -> str:
        state = self.session_state_map[step.session_id]
        if not state.enable_partial_rollout:
            limit = self.max_seq_length
            if self.max_tokens_per_step is not None:
                limit = min(limit, len(step.tokens) + self.max_tokens_per_step)
        else:
            limit = step.partial_rollout_max_tokens + self.max_seq_length_per_iter
        budget = limit - len(step.tokens) - len(step.partial_tokens)
        if budget <= 0 and state.enable_partial_rollout:
            raise StopPartialProgram(f"Program {state.uid} preempted due to partial sampler limit.")
        assert budget > 0, f"Max tokens must be positive, got {budget}"
        step.sample_params["max_tokens"] = budget
        t0 = time.time()
        out = await self._get_model_response(prompt_ids=step.tokens + step.partial_tokens, application_id=state.uid,
                                             multi_modal_data=step.multi_modal_data, **step.sample_params)
        step.partial_text += out.response
        step.partial_tokens.extend(out.token_ids)
        step.partial_logprobs.extend(out.logprobs)
        step.partial_token_strs.extend(out.token_strs)
        step.partial_moe_routermap = self._complete_routermap(state, step, out.moe_routermap)
        dt = time.time() - t0
        state.metrics.llm_time += dt
        state.metrics.total_time += dt
        if out.spec_decode_metrics is not None:
            state.metrics.spec_draft_tokens += out.spec_decode_metrics.num_draft_tokens
            state.metrics.spec_accepted_tokens += out.spec_decode_metrics.num_accepted_tokens
            state.metrics.spec_verify_count += out.spec_decode_metrics.num_completions
        if (state.enable_partial_rollout and out.stop_reason == ModelStopReason.LENGTH
                and step.token_len + len(step.partial_tokens) < self.max_seq_length):
            raise StopPartialProgram(f"Program {state.uid} preempted due to partial sampler limit.")
        content = self.chat_parser.assistant_message_content(step.partial_text)
        step.set_response(text=step.partial_text, tokens=step.partial_tokens, masks=[1] * len(step.partial_tokens),
                          logprobs=step.partial_logprobs, moe_routermap=step.partial_moe_routermap)
        step.chat_completions.append({"role": "assistant", "content": content})
        step.response_token_strs.extend(step.partial_token_strs)
        step.reset_partial_state()
        return content

    def _complete_routermap(self, state: ProgramState, step: Step, rm):
        """The sampler reports routing only for tokens it computed. When that is shorter than prompt +
        response (prefix-cache hit), take the head from the session's prefix tree if it has it all."""
        if not self.moe_replay or not _has_entries(rm):
            return rm
        want = len(step.tokens) + len(step.partial_logprobs)
        if len(rm) >= want:
            return rm
        missing = want - len(rm)
        head, node = [], state.prefix_tree.root
        for tok in (step.tokens + step.partial_tokens)[:missing]:
            node = node.get_child(tok) if node is not None else None
            if node is None or not _has_entries(node.moe_routermap):
                break
            head.append(node.moe_routermap)
        if len(head) != missing or not head:
            return rm
        if isinstance(rm, torch.Tensor):
            return torch.cat([torch.stack([torch.as_tensor(h) for h in head]).to(rm.dtype), rm], 0)
        return head + list(rm)

    async def _get_model_response(self, prompt_ids, application_id: str, multi_modal_data=None, **sample_params) -> ModelOutput:
        """One completion from the sampling client. The routing record of the LAST generated token is
        unknown to the sampler (it was never fed through the model), so a -1 row is appended."""
        params = {**self.default_sample_params, **sample_params}
        params.pop("n", None)
        res = await self.sampling_client.sample(prompt_ids, params, session_id=application_id,
                                                image_data=multi_modal_data)
        ids, lps = res["token_ids"][0], res["logprobs"][0]
        strs = res["token_strs"][0] or ([self.tokenizer.decode([t]) for t in ids] if self.tokenizer is not None else [""] * len(ids))
        rm = res["moe_routermap"][0] if res.get("moe_routermap") else None
        if rm is not None and _has_entries(rm):
            rm = torch.as_tensor(rm)
            rm = pad_moe_routermap(rm, len(prompt_ids) + len(ids)) if len(rm) == len(prompt_ids) + len(ids) - 1 else rm
        else:
            rm = []
        fin = res["finish_reasons"][0]
        spec = (res.get("spec_decode_metrics") or [None])[0]
        if spec:
            from ..sampler.params import SpecDecodeMetrics
            spec = SpecDecodeMetrics(**{k: int(v) for k, v in spec.items()})
        return ModelOutput.from_token_strs(token_ids=ids, token_strs=strs, logprobs=lps,
                                           stop_reason=ModelStopReason.LENGTH if fin == "length" else ModelStopReason.STOP,
                                           moe_routermap=rm, spec_decode_metrics=spec or None)

    # ------------------------------------------------------------------ termination checks
    def check_prompt_truncation_termination(self, step: Step) -> None:
        state = self.session_state_map[step.session_id]
        if state.num_steps != 0 or step.token_len <= self.max_prompt_length:
            return
        if self.prompt_truncation in ("left", "right"):
            cut = step.token_len - self.max_prompt_length
            sl = slice(cut, None) if self.prompt_truncation == "left" else slice(0, self.max_prompt_length)
            step.tokens, step.masks, step.logprobs = step.tokens[sl], step.masks[sl], step.logprobs[sl]
            step.token_len = len(step.tokens)
            return
        state.termination_reason, state.reward, state.done = TerminationReason.PROMPT_TRUNCATION, 0, True
        raise StopProgram(f"Program {state.uid} terminated due to prompt truncation "
                          f"({step.token_len} > {self.max_prompt_length}).")

    def check_truncation_termination(self, step: Step, last_assistant_response: bool = False) -> None:
        state = self.session_state_map[step.session_id]
        if step.token_len < self.max_seq_length:
            return
        over = step.token_len - self.max_seq_length
        if over > 0:
            step.tokens, step.masks, step.logprobs = step.tokens[:-over], step.masks[:-over], step.logprobs[:-over]
        if self.moe_replay and _has_entries(step.moe_routermap):
            step.moe_routermap = step.moe_routermap[: len(step.tokens)]
        if last_assistant_response:
            state.reward = 0.0
        step.token_len = self.max_seq_length
        state.termination_reason = TerminationReason.TRUNCATION
        raise StopProgram(f"Program {state.uid} terminated due to truncation.")

    def check_state_before_generation(self, state: ProgramState) -> None:
        if state.done:
            if not state.termination_reason:
                state.termination_reason = TerminationReason.ENV_DONE
            raise StopProgram(f"Program {state.uid} terminated previously already.")
        if state.num_steps >= self.max_steps:
            state.termination_reason = TerminationReason.MAX_STEPS
            raise StopProgram(f"Program {state.uid} terminated due to max steps.")


def postprocess_program_state(state: ProgramState) -> ProgramState:
    """Freeze the training view of a finished program (one step per prefix-tree leaf) and drop the
    engine-only fields that must not travel to the trainer."""
    state.training_steps = state.get_training_steps()
    state.session_lock = None
    state.partial_rollout_futures = []
    return state
