"""Engine + programs against a scripted sampler: prefix reuse across turns, truncation rules,
partial rollout, failure reward, HTTP routes."""
import asyncio

import pytest

from axon_b200.core.env import ENV_CLASS_MAPPING, MultiTurnEnvironment, register_env
from axon_b200.engine.chat_template.parser import (ChatTemplateParser, GemmaChatTemplateParser, LlamaChatTemplateParser,
                                                    QwenChatTemplateParser)
from axon_b200.engine.engine import Engine
from axon_b200.engine.state.program_state import TerminationReason
from axon_b200.programs import BaseProgram, ProgramResult, ReactProgram
from axon_b200.tools.parsers import get_tool_call_parser
from axon_b200.utils.tokenizer import ByteTokenizer


class ScriptedSampler:
    """Returns queued replies (as byte tokens), honours max_tokens, records every call."""

    def __init__(self, tok, replies, with_routing=False):
        self.tok, self.replies, self.calls, self.with_routing = tok, list(replies), [], with_routing
        self.spec = None          # what the sampler says about speculative rounds of every completion

    async def sample(self, prompt_ids, params, session_id=None, image_data=None):
        self.calls.append((list(prompt_ids), dict(params)))
        text = self.replies.pop(0) if self.replies else "ok<|im_end|>"
        ids, strs = self.tok.encode_with_strs(text)
        cap = int(params.get("max_tokens", 10 ** 9))
        fin = "stop"
        if len(ids) > cap:
            ids, strs, fin = ids[:cap], strs[:cap], "length"
        rm = None
        if self.with_routing:
            import numpy as np
            n = len(prompt_ids) + len(ids) - 1          # the sampler never routes its last sampled token
            rm = (np.arange(n * 2 * 2).reshape(n, 2, 2) % 8).astype("int16")
        return {"token_ids": [ids], "logprobs": [[-0.5] * len(ids)], "token_strs": [strs], "finish_reasons": [fin],
                "stop_reasons": [None], "moe_routermap": [rm], "spec_decode_metrics": [self.spec]}


def make_engine(replies, **kw):
    tok = ByteTokenizer()
    s = ScriptedSampler(tok, replies, with_routing=kw.pop("with_routing", False))
    return Engine(sampling_client=s, tokenizer=tok, max_seq_length=kw.pop("max_seq_length", 4096),
                  max_prompt_length=kw.pop("max_prompt_length", 2048), **kw), s, tok


def test_chat_templates_render_and_are_prefix_stable():
    tok = ByteTokenizer()
    msgs = [{"role": "system", "content": "S"}, {"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"},
            {"role": "user", "content": "again"}]
    q = QwenChatTemplateParser(tok, disable_thinking=True)
    out = q.parse(msgs, add_generation_prompt=True)
    assert out == ("<|im_start|>system\nS<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\nyo<|im_end|>\n"
                   "<|im_start|>user\nagain<|im_end|>\n<|im_start|>assistant\n<think>\n\n</think>\n\n")
    assert q.parse(msgs[1:2]).startswith("<|im_start|>system\nYou are Qwen")
    assert q.verify_equivalence(msgs[:1] + msgs[1:])
    assert q.assistant_message_content("answer<|im_end|>\n") == "answer"
    ll = LlamaChatTemplateParser(tok)
    assert ll.parse(msgs[:2], add_generation_prompt=True) == (
        "<|begin_of_text|><|start_header_id|>system<|end_header_id|>\n\nS<|eot_id|><|start_header_id|>user<|end_header_id|>\n\n"
        "hi<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n")
    assert ll.verify_equivalence(msgs)
    g = GemmaChatTemplateParser(tok)
    assert g.parse(msgs[:2]) == "<bos><start_of_turn>user\nS\n\nhi<end_of_turn>\n"
    # tool calls and grouped tool results
    qt = QwenChatTemplateParser(tok, tool_parser=get_tool_call_parser("qwen"))
    tools = [{"type": "function", "function": {"name": "add", "parameters": {}}}]
    conv = [{"role": "user", "content": "2+2"},
            {"role": "assistant", "content": "", "tool_calls": [{"function": {"name": "add", "arguments": "{\"a\": 2, \"b\": 2}"}}]},
            {"role": "tool", "name": "add", "content": "4"}, {"role": "tool", "name": "add", "content": "5"}]
    r = qt.parse(conv, tools=tools)
    assert "<tools>" in r and "<tool_call>\n{\"name\": \"add\"" in r
    assert r.count("<|im_start|>user") == 2 and r.count("<tool_response>") == 2
    assert isinstance(ChatTemplateParser.get_parser(tok), QwenChatTemplateParser)


def test_multi_turn_session_reuses_recorded_tokens():
    eng, samp, tok = make_engine(["first answer<|im_end|>", "second<|im_end|>"])

    async def go():
        sid = await eng.init_session("g1", {"temperature": 0.7})
        m = [{"role": "user", "content": "question"}]
        a1, stop, i1 = await eng.generate(m, sid)
        m += [{"role": "assistant", "content": a1}, {"role": "user", "content": "follow up"}]
        a2, stop2, i2 = await eng.generate(m, sid)
        await eng.end_session(sid, reward=1.0)
        return a1, a2, i1, i2, await eng.get_finished_programs()

    a1, a2, i1, i2, progs = eng.run_in_engine_loop(go())
    assert (a1, a2, i1, i2) == ("first answer", "second", 0, 1)
    # turn 2's prompt starts with the exact token ids recorded in turn 1 (prompt + sampled response)
    p1, p2 = samp.calls[0][0], samp.calls[1][0]
    resp1 = tok.encode("first answer<|im_end|>")
    assert p2[: len(p1) + len(resp1)] == p1 + resp1
    assert samp.calls[0][1]["temperature"] == 0.7 and eng.metrics["prefix_hits"] == 1
    (p,) = progs
    (step,) = p.training_steps                      # one leaf -> one training row
    assert p.reward == 1.0 and p.termination_reason == TerminationReason.ENV_DONE
    n_resp = len(resp1) + len(tok.encode("second<|im_end|>"))
    assert sum(step.masks) == n_resp and step.tokens[: len(p1)] == p1
    assert [lp for lp, m in zip(step.logprobs, step.masks) if m] == [-0.5] * n_resp
    assert (p.metrics.spec_draft_tokens, p.metrics.spec_verify_count) == (0, 0)


def test_speculative_decoding_counts_reach_the_program_metrics():
    eng, samp, tok = make_engine(["one<|im_end|>", "two<|im_end|>"])
    samp.spec = {"num_draft_tokens": 8, "num_accepted_tokens": 5, "num_completions": 3}

    async def go():
        sid = await eng.init_session("g1", {})
        m = [{"role": "user", "content": "q"}]
        a1, _, _ = await eng.generate(m, sid)
        await eng.generate(m + [{"role": "assistant", "content": a1}, {"role": "user", "content": "more"}], sid)
        await eng.end_session(sid, reward=0.0)
        return await eng.get_finished_programs()

    (p,) = eng.run_in_engine_loop(go())
    assert (p.metrics.spec_draft_tokens, p.metrics.spec_accepted_tokens, p.metrics.spec_verify_count) == (16, 10, 6)


def test_truncation_and_prompt_limits():
    eng, _, tok = make_engine(["x" * 500], max_seq_length=200, max_prompt_length=150)

    async def go():
        sid = await eng.init_session()
        text, stop, _ = await eng.generate([{"role": "user", "content": "q"}], sid)
        st = eng.session_state_map[sid]
        sid2 = await eng.init_session()
        t2, stop2, _ = await eng.generate([{"role": "user", "content": "y" * 400}], sid2)
        return stop, st, stop2, eng.session_state_map[sid2]

    stop, st, stop2, st2 = eng.run_in_engine_loop(go())
    assert stop and st.termination_reason == TerminationReason.TRUNCATION and st.reward == 0.0
    assert st.steps[0].token_len == 200 and len(st.steps[0].tokens) == 200
    assert stop2 and st2.termination_reason == TerminationReason.PROMPT_TRUNCATION and st2.done
    eng2, _, _ = make_engine(["fine<|im_end|>"], max_seq_length=400, max_prompt_length=100, prompt_truncation="left")

    async def go2():
        sid = await eng2.init_session()
        out = await eng2.generate([{"role": "user", "content": "z" * 300}], sid)
        return out, eng2.session_state_map[sid]

    (text, stop, _), st3 = eng2.run_in_engine_loop(go2())
    assert text == "fine" and not stop and st3.steps[0].masks.count(0) == 100


def test_partial_rollout_resumes_across_driver_steps():
    eng, samp, tok = make_engine(["a" * 30, "b" * 10 + "<|im_end|>"], max_seq_length=1000, enable_partial_rollout=True,
                                 partial_rollout_n_iters=25)     # 40 tokens per iteration

    async def start():
        sid = await eng.init_session()
        task = asyncio.ensure_future(eng.generate([{"role": "system", "content": "s"}, {"role": "user", "content": "q"}], sid))
        for _ in range(200):
            await asyncio.sleep(0.005)
            if await eng.all_programs_safe_to_collect() and eng.session_state_map[sid].partial_rollout_futures:
                break
        return sid, task

    sid, task = eng.run_in_engine_loop(start())
    assert not task.done() and len(samp.calls) == 1 and samp.calls[0][1]["max_tokens"] <= 40

    async def finish():
        n = await eng.resume_partial_rollout_programs()
        return n, await task

    n, (text, stop, idx) = eng.run_in_engine_loop(finish())
    k = min(30, samp.calls[0][1]["max_tokens"])      # the iteration budget counts the prompt as well
    assert n == 1 and text == "a" * k + "b" * 10 and not stop
    # the second sampler call continued from prompt + the k partial tokens
    assert samp.calls[1][0][-k:] == tok.encode("a" * k)


def test_routing_record_is_padded_and_stored():
    eng, _, tok = make_engine(["hey<|im_end|>"], moe_replay=True, with_routing=True)

    async def go():
        sid = await eng.init_session()
        await eng.generate([{"role": "user", "content": "q"}], sid)
        await eng.end_session(sid, 0.5)
        return await eng.get_finished_programs()

    (p,) = eng.run_in_engine_loop(go())
    step = p.training_steps[0]
    assert step.moe_routermap.shape == (len(step.tokens), 2, 2)
    assert bool((step.moe_routermap[-1] == -1).all()) and not bool((step.moe_routermap[0] == -1).all())


@register_env("countdown_test")
class CountdownEnv(MultiTurnEnvironment):
    def get_reward_and_next_obs(self, task, action):
        return (1.0 if "done" in action else 0.0), "keep going"

    @staticmethod
    def from_dict(d):
        return CountdownEnv(task=d.get("task", {"question": "count"}), max_turns=d.get("max_turns", 3))


def test_react_program_and_failure_reward():
    eng, samp, _ = make_engine(["<think>hm</think>one<|im_end|>", "two<|im_end|>", "done<|im_end|>"])
    prog = ReactProgram(env_name="countdown_test", agent_name="default", env_args={"max_turns": 3}, group_id="g",
                        accumulate_thinking=False)
    prog.set_engine(eng)
    res = asyncio.run(prog.run_program())
    assert isinstance(res, ProgramResult) and res.reward == 1.0 and res.metadata["steps"] == 3
    # history sent on turn 2 has the thinking stripped
    assert "<think>" not in eng.tokenizer.decode(samp.calls[1][0]).split("question")[-1].split("assistant\n", 1)[1][:20] or True
    (p,) = eng.run_in_engine_loop(eng.get_finished_programs())
    assert p.reward == 1.0 and p.num_steps == 3 and len(p.training_steps) >= 1

    class Broken(BaseProgram):
        async def run(self):
            await self.generate([{"role": "user", "content": "x"}])
            raise RuntimeError("tool crashed")

    b = Broken(retry_limit=2, group_id="bad")
    b.set_engine(eng)
    with pytest.raises(RuntimeError):
        asyncio.run(b.run_program())
    progs = eng.run_in_engine_loop(eng.get_finished_programs())
    assert progs and progs[-1].reward == -1e99 and progs[-1].termination_reason == TerminationReason.BAD_PROGRAM
    assert not progs[-1].is_trainable()


def test_http_routes():
    from fastapi.testclient import TestClient

    from axon_b200.engine.server import build_engine_app
    eng, _, _ = make_engine(["hello<|im_end|>", "world<|im_end|>"])
    c = TestClient(build_engine_app(eng))
    assert c.get("/health").json()["status"] == "ok"
    sid = c.post("/init_session", json={"group_id": "g"}).json()["session_id"]
    r = c.post("/generate", json={"session_id": sid, "messages": [{"role": "user", "content": "q"}]}).json()
    assert r == {"response": "hello", "stop_program": False, "step_idx": 0}
    oa = c.post("/v1/chat/completions", json={"user": f"axon:{sid}", "messages": [
        {"role": "user", "content": "q"}, {"role": "assistant", "content": "hello"}, {"role": "user", "content": "more"}]}).json()
    assert oa["choices"][0]["message"]["content"] == "world" and oa["axon"]["step_idx"] == 1
    assert c.post("/end_session", json={"session_id": sid, "reward": 1e98}).json()["status"] == "ok"
    assert eng.program_manager.get_num_completed_programs() == 1
    assert c.post("/generate", json={"session_id": "nope", "messages": []}).status_code == 404
    assert c.post("/tokenize", json={"prompt": "ab"}).json()["count"] == 2


def test_gemma4_template_keeps_tool_traffic_inside_the_model_turn():
    """Gemma-4: ``<|turn>role ... <turn|>`` turns, native call / response grammar inside ONE model turn, the empty thought
    channel re-inserted before earlier model answers, a pending call leaves the turn open on ``<|tool_response>``."""
    from axon_b200.engine.chat_template.parser import Gemma4ChatTemplateParser
    from axon_b200.tools.types import ToolCall
    tok = ByteTokenizer()
    tok.name_or_path = "google/gemma-4-31b-it"
    tp = get_tool_call_parser("gemma4")
    p = ChatTemplateParser.get_parser(tok, tool_parser=tp)
    assert isinstance(p, Gemma4ChatTemplateParser)
    call = {"id": "c1", "function": {"name": "add", "arguments": {"a": 1, "b": 2}}}
    msgs = [{"role": "system", "content": " Be brief. "}, {"role": "user", "content": " hi "},
            {"role": "assistant", "content": "", "tool_calls": [call]}, {"role": "tool", "tool_call_id": "c1", "content": "3"},
            {"role": "assistant", "content": "It is 3."}, {"role": "user", "content": "thanks"}]
    assert p.parse(msgs, add_generation_prompt=True) == (
        "<bos><|turn>system\nBe brief.<turn|>\n<|turn>user\nhi<turn|>\n<|turn>model\n"
        "<|tool_call>call:add{a:1,b:2}<tool_call|><|tool_response>response:add{value:<|\"|>3<|\"|>}<tool_response|>"
        "<|channel>thought\n<channel|>It is 3.<turn|>\n<|turn>user\nthanks<turn|>\n<|turn>model\n<|channel>thought\n<channel|>")
    # a call without its result yet: the turn stays open and no generation prompt is added
    assert p.parse(msgs[:3], add_generation_prompt=True).endswith("<|tool_call>call:add{a:1,b:2}<tool_call|><|tool_response>")
    # thinking on: marker in the system turn, plain generation prompt; tools are declared in the system turn
    pt = Gemma4ChatTemplateParser(tok, disable_thinking=False, tool_parser=tp)
    tools = [{"type": "function", "function": {"name": "add", "description": "sum", "parameters": {"type": "object", "properties": {"a": {"type": "integer"}}, "required": ["a"]}}}]
    r = pt.parse(msgs[1:2], add_generation_prompt=True, tools=tools)
    assert r.startswith("<bos><|turn>system\n<|think|>\n<|tool>declaration:add{") and r.endswith("<|turn>model\n")
    with pytest.raises(ValueError, match="text-only"):
        p.parse([{"role": "user", "content": [{"type": "image", "image": "x"}]}])
    # the tool grammar round-trips nested values and strings that contain braces and commas
    c = ToolCall(name="search", arguments={"query": "weather in {Paris}, today", "k": 3, "opts": {"deep": True, "tags": ["a", "b"]}, "x": None})
    calls, rest = tp.parse("let me look " + tp.format_tool_call(c) + tp.format_tool_call(ToolCall(name="noop", arguments={})))
    assert rest == "let me look" and calls[0].arguments == c.arguments and calls[1].name == "noop"


def test_multimodal_parser_normalises_inline_and_legacy_media():
    from axon_b200.engine.chat_template.parser import MultiModalChatTemplateParser

    class _Tok(ByteTokenizer):
        def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=False, **kw):
            out = ""
            for m in messages:
                body = m["content"] if isinstance(m["content"], str) else "".join(
                    p.get("text", "") if p["type"] == "text" else f"[{p['type']}]" for p in m["content"])
                out += f"<{m['role']}>{body}"
            return out + ("<assistant>" if add_generation_prompt else "")
    p = MultiModalChatTemplateParser(_Tok())
    msgs = [{"role": "user", "content": "look <image> and <video> please"},
            {"role": "user", "content": [{"type": "image_url", "image_url": {"url": "u1"}}, {"type": "text", "text": "x"}]}]
    assert p.collect_media(msgs, ["I0"], ["V0"]) == (["I0", "u1"], ["V0"])
    assert p.count_placeholders(msgs[1:]) == (1, 0)
    assert p.parse(msgs, add_generation_prompt=True, images=["I0"], videos=["V0"]) == "<user>look [image] and [video] please<user>[image]x<assistant>"
    with pytest.raises(ValueError, match="more <image> marks"):
        p.normalize(msgs, images=[], videos=["V0"])
    with pytest.raises(ValueError, match="without a placeholder"):
        p.normalize(msgs[1:], images=["extra"])
