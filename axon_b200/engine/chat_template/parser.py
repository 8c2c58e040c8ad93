"""Chat-template parsers: render message lists to the exact prompt string of a model family and
tokenise rendered text. Rendering is done here (not through ``tokenizer.apply_chat_template``) so
that rendering message-by-message equals rendering the whole list — the property the prefix tree's
text matching depends on (``verify_equivalence``).

Families and factory follow the reference (axon/engine/chat_template/parser.py:69-1800): Qwen
(ChatML, optional ``<think>`` suppression, tool calls/results), DeepSeek-R1-distilled Qwen, Llama-3,
Gemma, OpenAI Harmony (gpt-oss), Moonlight/Kimi, GLM-4, and a multimodal Qwen-VL variant that
reports placeholder regions for images/videos.
"""
from __future__ import annotations

import re

import hashlib
import json
from dataclasses import dataclass, field
from typing import Any


@dataclass
class TokenizeContext:
    messages: list | None = None
    images: list = field(default_factory=list)
    videos: list = field(default_factory=list)
    processor_kwargs: dict = field(default_factory=dict)


@dataclass
class TokenizeOutput:
    token_ids: list
    token_strs: list = field(default_factory=list)
    multi_modal_data: Any = None


def _text_of(content) -> str:
    """Message content as text; list-style content keeps text parts and marks media parts."""
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    out = []
    for part in content:
        if isinstance(part, str):
            out.append(part)
        elif isinstance(part, dict):
            t = part.get("type")
            if t == "text":
                out.append(part.get("text", ""))
            elif t in ("image", "image_url"):
                out.append("<|vision_start|><|image_pad|><|vision_end|>")
            elif t in ("video", "video_url"):
                out.append("<|vision_start|><|video_pad|><|vision_end|>")
    return "".join(out)


class ChatTemplateParser:
    """Base parser. ``tokenizer`` needs ``encode_with_strs`` (or ``encode``), ``decode`` and ``eos_token``."""

    system_token = user_token = assistant_token = tool_token = eot_token = ""
    generation_prompt = ""
    default_system = ""
    separator = ""

    def __init__(self, tokenizer, tool_parser=None, tokenizer_pool=None):
        self.tokenizer = tokenizer
        self.tokenizer_pool = tokenizer_pool
        self.tool_parser = tool_parser

    # ------------------------------------------------------------------ rendering
    def parse_system(self, m) -> str:
        return self.system_token + _text_of(m["content"]) + self.eot_token

    def parse_user(self, m) -> str:
        return self.user_token + _text_of(m["content"]) + self.eot_token

    def parse_assistant(self, m) -> str:
        text = _text_of(m.get("content", ""))
        out = self.assistant_token + text
        calls = m.get("tool_calls") or []
        if calls:
            assert self.tool_parser, f"a tool parser is required to render tool calls: {m}"
            from ...tools.types import ToolCall
            out += ("\n" if text else "") + self.tool_parser.format_tool_calls([ToolCall.from_raw_tool_call(c) for c in calls])
        return out + self.eot_token

    def parse_tool(self, m, i, messages) -> str:
        body = _text_of(m.get("content", ""))
        if self.tool_parser:
            body = self.tool_parser.format_tool_result(content=body, name=m.get("name", ""))
        return self.tool_token + body + self.eot_token

    def _prefix(self, messages, tools) -> tuple[str, list]:
        """Text emitted before the first message (default system prompt / tool definitions)."""
        if tools:
            assert self.tool_parser, "a tool parser is required when tools are given"
            sys_text = _text_of(messages[0]["content"]) + "\n\n" if messages and messages[0]["role"] == "system" \
                else (self.default_system + "\n\n" if self.default_system else "")
            rest = messages[1:] if messages and messages[0]["role"] == "system" else messages
            return self.system_token + sys_text + self.tool_parser.get_tool_system_prompt(tools) + self.eot_token, rest
        if messages and messages[0]["role"] not in ("system", "skip") and self.default_system:
            return self.system_token + self.default_system + self.eot_token, messages
        return "", messages

    def parse(self, messages, add_generation_prompt: bool = False, tools=None, **kwargs) -> str:
        if not messages:
            return ""
        out, messages = self._prefix(list(messages), tools)
        for i, m in enumerate(messages):
            role = m["role"]
            if out:
                out += self.separator
            if role == "system":
                out += self.parse_system(m)
            elif role == "user":
                out += self.parse_user(m)
            elif role == "assistant":
                out += self.parse_assistant(m)
            elif role == "tool":
                out += self.parse_tool(m, i, messages)
            elif role == "skip":                # pre-rendered text inserted verbatim
                out += m["content"]
            else:
                raise NotImplementedError(f"Unsupported message role: {role}")
        if add_generation_prompt and messages and messages[-1]["role"] != "skip":
            out += self.separator + self.generation_prompt
        return out

    # ------------------------------------------------------------------ tokenisation
    async def tokenize(self, input_text: str, ctx: TokenizeContext | None = None) -> TokenizeOutput:
        if self.tokenizer_pool is not None:
            ids, strs = await self.tokenizer_pool.encode_with_strs(input_text, add_special_tokens=False)
        elif hasattr(self.tokenizer, "encode_with_strs"):
            ids, strs = self.tokenizer.encode_with_strs(input_text)
        else:
            ids = self.tokenizer.encode(input_text, add_special_tokens=False)
            strs = [self.tokenizer.decode([i]) for i in ids]
        return TokenizeOutput(token_ids=list(ids), token_strs=list(strs))

    def _assistant_message_stop_texts(self) -> tuple:
        stops = []
        eos = getattr(self.tokenizer, "eos_token", None)
        if isinstance(eos, str) and eos:
            stops.append(eos)
        eid = getattr(self.tokenizer, "eos_token_id", None)
        for t in ([eid] if isinstance(eid, int) else list(eid or [])):
            try:
                s = self.tokenizer.decode([t], skip_special_tokens=False)
            except Exception:  # noqa: BLE001
                continue
            if s:
                stops.append(s)
        if self.eot_token.strip():
            stops.append(self.eot_token.strip())
        return tuple(dict.fromkeys(stops))

    def assistant_message_content(self, response: str) -> str:
        """The sampled text as it should appear in chat history: trailing end-of-turn tokens removed
        (the recorded token stream itself is never altered)."""
        stops = sorted(set(self._assistant_message_stop_texts()), key=len, reverse=True)
        text = response
        while stops:
            stripped = text.rstrip()
            hit = next((s for s in stops if stripped.endswith(s)), None)
            if hit is None:
                break
            text = stripped[: -len(hit)].rstrip()
        return text

    def get_mm_regions(self, input_key: str, messages) -> list:
        return []

    def verify_equivalence(self, messages, verbose: bool = True) -> bool:
        """Rendering must be prefix-stable: the rendering of the first k messages is a prefix of the
        rendering of the first k+1 (what the prefix tree's text matching relies on)."""
        prev = ""
        for k in range(1, len(messages) + 1):
            cur = self.parse(messages[:k])
            if not cur.startswith(prev):
                if verbose:
                    raise AssertionError(f"Parser failed equivalence check at message {k}.\nprevious:\n{prev}\n\ncurrent:\n{cur}")
                return False
            prev = cur
        return True

    # ------------------------------------------------------------------ factory
    @classmethod
    def get_parser(cls, tokenizer, processor=None, disable_thinking: bool = False, tool_parser=None,
                   tokenizer_pool=None) -> "ChatTemplateParser":
        name = (getattr(tokenizer, "name_or_path", "") or "").lower()
        kw = dict(tool_parser=tool_parser, tokenizer_pool=tokenizer_pool)
        if "deepseek" in name and ("distill" in name or "r1" in name):
            return DeepseekQwenChatTemplateParser(tokenizer, **kw)
        if "gpt-oss" in name or "harmony" in name:
            return OpenAIHarmonyChatTemplateParser(tokenizer, **kw)
        if "qwen" in name and ("vl" in name) and processor is not None:
            return QwenVLChatTemplateParser(tokenizer, processor=processor, disable_thinking=disable_thinking, **kw)
        if "qwen" in name or "byte-tokenizer" in name or "r2e" in name or "deepswe" in name:
            return QwenChatTemplateParser(tokenizer, disable_thinking=disable_thinking, **kw)
        if "llama" in name:
            return LlamaChatTemplateParser(tokenizer, **kw)
        if "gemma-4" in name or "gemma4" in name:
            return Gemma4ChatTemplateParser(tokenizer, disable_thinking=disable_thinking or True, **kw)
        if "gemma" in name:
            return GemmaChatTemplateParser(tokenizer, **kw)
        if "moonlight" in name or "kimi" in name:
            return MoonlightChatTemplateParser(tokenizer, **kw)
        if "glm" in name:
            return GlmChatTemplateParser(tokenizer, **kw)
        return HFChatTemplateParser(tokenizer, **kw)


class HFChatTemplateParser(ChatTemplateParser):
    """Fallback: defer to the tokenizer's own jinja chat template."""

    def parse(self, messages, add_generation_prompt=False, tools=None, **kwargs) -> str:
        return self.tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt,
                                                  **({"tools": tools} if tools else {}))


class QwenChatTemplateParser(ChatTemplateParser):
    system_token = "<|im_start|>system\n"
    user_token = "<|im_start|>user\n"
    assistant_token = "<|im_start|>assistant\n"
    eot_token = "<|im_end|>"
    separator = "\n"
    default_system = "You are Qwen, created by Alibaba Cloud. You are a helpful assistant."

    def __init__(self, tokenizer, disable_thinking: bool = True, is_qwen3_next: bool = False, **kw):
        super().__init__(tokenizer, **kw)
        self.disable_thinking, self.is_qwen3_next = disable_thinking, is_qwen3_next
        self.generation_prompt = self.assistant_token + ("<think>\n\n</think>\n\n" if disable_thinking and not is_qwen3_next else "")

    def parse_tool(self, m, i, messages) -> str:
        """Consecutive tool results share one ``user`` turn."""
        assert self.tool_parser, f"a tool parser is required to render tool results: {m}"
        first = i == 0 or messages[i - 1]["role"] != "tool"
        last = i == len(messages) - 1 or messages[i + 1]["role"] != "tool"
        out = self.user_token.rstrip("\n") if first else ""
        out += "\n" + self.tool_parser.format_tool_result(content=_text_of(m.get("content", "")), name=m.get("name", ""))
        return out + (self.eot_token if last else "")

    def parse(self, messages, add_generation_prompt=False, tools=None, **kwargs) -> str:
        # grouped tool turns must not be separated by the "\n" join inside a group
        out = super().parse(messages, add_generation_prompt, tools, **kwargs)
        return out.replace("</tool_response>\n\n<tool_response>", "</tool_response>\n<tool_response>")


class DeepseekQwenChatTemplateParser(ChatTemplateParser):
    """DeepSeek-R1 distilled models: ``<｜User｜>`` / ``<｜Assistant｜>`` markers, generation opens ``<think>``."""
    bos = "<｜begin▁of▁sentence｜>"
    system_token = ""
    user_token = "<｜User｜>"
    assistant_token = "<｜Assistant｜>"
    eot_token = "<｜end▁of▁sentence｜>"

    def __init__(self, tokenizer, **kw):
        super().__init__(tokenizer, **kw)
        self.generation_prompt = self.assistant_token + "<think>\n"

    def parse_system(self, m) -> str:
        return _text_of(m["content"])

    def parse_user(self, m) -> str:
        return self.user_token + _text_of(m["content"])

    def parse(self, messages, add_generation_prompt=False, tools=None, **kwargs) -> str:
        body = super().parse(messages, add_generation_prompt, tools, **kwargs)
        return body if not messages or body.startswith(self.bos) or messages[0]["role"] == "skip" else self.bos + body


class LlamaChatTemplateParser(ChatTemplateParser):
    bos = "<|begin_of_text|>"
    system_token = "<|start_header_id|>system<|end_header_id|>\n\n"
    user_token = "<|start_header_id|>user<|end_header_id|>\n\n"
    assistant_token = "<|start_header_id|>assistant<|end_header_id|>\n\n"
    tool_token = "<|start_header_id|>ipython<|end_header_id|>\n\n"
    eot_token = "<|eot_id|>"

    def __init__(self, tokenizer, **kw):
        super().__init__(tokenizer, **kw)
        self.generation_prompt = self.assistant_token

    def parse(self, messages, add_generation_prompt=False, tools=None, **kwargs) -> str:
        body = super().parse(messages, add_generation_prompt, tools, **kwargs)
        return self.bos + body if messages and messages[0]["role"] != "skip" else body


class GemmaChatTemplateParser(ChatTemplateParser):
    """Gemma has no system role: a system message is folded into the first user turn."""
    bos = "<bos>"
    user_token = "<start_of_turn>user\n"
    assistant_token = "<start_of_turn>model\n"
    eot_token = "<end_of_turn>\n"

    def __init__(self, tokenizer, **kw):
        super().__init__(tokenizer, **kw)
        self.generation_prompt = self.assistant_token

    def parse(self, messages, add_generation_prompt=False, tools=None, **kwargs) -> str:
        msgs = list(messages)
        if msgs and msgs[0]["role"] == "system" and len(msgs) > 1 and msgs[1]["role"] == "user":
            merged = dict(msgs[1])
            merged["content"] = _text_of(msgs[0]["content"]) + "\n\n" + _text_of(msgs[1]["content"])
            msgs = [merged] + msgs[2:]
        body = super().parse(msgs, add_generation_prompt, tools, **kwargs)
        return self.bos + body if msgs and msgs[0]["role"] != "skip" else body

    def parse_system(self, m) -> str:
        return self.user_token + _text_of(m["content"]) + self.eot_token

    def parse_tool(self, m, i, messages) -> str:
        return self.user_token + _text_of(m.get("content", "")) + self.eot_token


class Gemma4ChatTemplateParser(ChatTemplateParser):
    """Gemma-4 (reference: axon/engine/chat_template/parser.py:543-808, the chat template shipped with
    google/gemma-4-*-it). Turns are ``<|turn>role\ncontent<turn|>\n`` with roles system / user / model. Tool calls
    and their results live INSIDE the model turn (``<|tool_call>...<tool_call|><|tool_response>...<tool_response|>``):
    ``tool`` messages are consumed by the assistant message before them, and an assistant message that follows
    tool results continues the open model turn instead of starting a new one. Thinking: with thinking off (the
    default for RL) the generation prompt carries an empty thought channel, which is re-inserted before the content
    of every earlier model turn so that rendered histories stay prefix-cumulative with the token tree; with thinking
    on, the system turn starts with ``<|think|>``. Text only: media parts are refused."""
    bos = "<bos>"
    start_turn, end_turn = "<|turn>", "<turn|>"
    THINK = "<|think|>"
    EMPTY_THOUGHT = "<|channel>thought\n<channel|>"
    _MEDIA = ("image", "input_image", "image_url", "audio", "input_audio", "audio_url", "video", "input_video", "video_url")

    def __init__(self, tokenizer, disable_thinking: bool = True, **kw):
        super().__init__(tokenizer, **kw)
        self.bos = getattr(tokenizer, "bos_token", None) or self.bos
        self.disable_thinking = disable_thinking
        self.generation_prompt = f"{self.start_turn}model\n" + (self.EMPTY_THOUGHT if disable_thinking else "")

    def _assistant_message_stop_texts(self) -> tuple:
        return (self.end_turn, *super()._assistant_message_stop_texts())

    def _text(self, content, strip: bool) -> str:
        if isinstance(content, str):
            return content.strip() if strip else content
        out = []
        for part in content or []:
            if not isinstance(part, dict):
                continue
            if part.get("type") in ("text", "input_text"):
                t = part.get("text") or ""
                out.append(t.strip() if strip else t)
            elif part.get("type") in self._MEDIA:
                raise ValueError("Gemma4ChatTemplateParser is text-only; use a multimodal parser for media content")
        return "".join(out)

    def parse(self, messages, add_generation_prompt: bool = False, tools=None, **kwargs) -> str:
        from ...tools.types import ToolCall
        msgs = list(messages)
        out = self.bos
        thinking = not self.disable_thinking
        has_system = bool(msgs) and msgs[0].get("role") in ("system", "developer")
        if thinking or tools or has_system:
            out += f"{self.start_turn}system\n"
            if thinking:
                out += self.THINK + "\n"
            if has_system:
                c = msgs[0].get("content", "")
                out += c.strip() if isinstance(c, str) else "".join((p.get("text") or "").strip() + " " for p in c
                                                                    if isinstance(p, dict) and p.get("type") in ("text", "input_text"))
                msgs = msgs[1:]
            if tools:
                assert self.tool_parser, "a tool parser is required when tools are given"
                out += self.tool_parser.get_tool_system_prompt(tools)
            out += f"{self.end_turn}\n"
        last_user = max((i for i, m in enumerate(msgs) if m.get("role") == "user"), default=-1)
        prev_role, tail = None, None               # tail: what the last rendered message ended with (call / response / None)
        for i, m in enumerate(msgs):
            role = m.get("role")
            if role == "tool":                     # rendered by the assistant message in front of it
                continue
            if role == "skip":
                out += m["content"]
                continue
            tail = None
            mapped = "model" if role == "assistant" else role
            if not (mapped == "model" and prev_role == "assistant"):      # a model message after tool results continues its turn
                out += f"{self.start_turn}{mapped}\n"
            calls = m.get("tool_calls")
            thought = m.get("reasoning") or m.get("reasoning_content")
            if thought and i > last_user and calls:
                out += f"<|channel>thought\n{thought}\n<channel|>"
            answered = False
            if calls:
                assert self.tool_parser, f"a tool parser is required to render tool calls: {m}"
                objs = [ToolCall.from_raw_tool_call(c) for c in calls]
                out += self.tool_parser.format_tool_calls(objs)
                tail = "call"
                for follow in msgs[i + 1:]:
                    if follow.get("role") != "tool":
                        break
                    name = follow.get("name", "unknown")
                    for c in objs:
                        if follow.get("tool_call_id") and c.id == follow["tool_call_id"]:
                            name = c.name
                    body = follow.get("content", "")
                    out += self.tool_parser.format_tool_result(content=self._text(body, False) if not isinstance(body, dict) else body, name=name)
                    answered, tail = True, "response"
            for r in m.get("tool_responses") or []:
                assert self.tool_parser
                out += self.tool_parser.format_tool_result(content=r.get("response"), name=r.get("name", "unknown"))
                answered, tail = True, "response"
            text = self._text(m.get("content", ""), strip=mapped != "model")
            if text:
                out += (self.EMPTY_THOUGHT if mapped == "model" and self.disable_thinking else "") + text
            if tail == "call" and not answered:
                out += "<|tool_response>"          # the call waits for its result: the turn stays open on the opener
            elif answered and not text.strip():
                pass                               # turn left open: the next assistant message continues it
            else:
                out += f"{self.end_turn}\n"
            prev_role = role
        if add_generation_prompt and tail not in ("call", "response") and not (msgs and msgs[-1].get("role") == "skip"):
            out += self.generation_prompt
        return out


class OpenAIHarmonyChatTemplateParser(ChatTemplateParser):
    """gpt-oss Harmony format: ``<|start|>role<|message|>...<|end|>``; assistant turns carry a channel."""
    eot_token = "<|end|>"

    def __init__(self, tokenizer, reasoning_effort: str = "medium", **kw):
        super().__init__(tokenizer, **kw)
        self.reasoning_effort = reasoning_effort
        self.generation_prompt = "<|start|>assistant"

    def parse_system(self, m) -> str:
        return "<|start|>developer<|message|># Instructions\n\n" + _text_of(m["content"]) + "<|end|>"

    def parse_user(self, m) -> str:
        return "<|start|>user<|message|>" + _text_of(m["content"]) + "<|end|>"

    def parse_assistant(self, m) -> str:
        out = ""
        if m.get("reasoning_content"):
            out += "<|start|>assistant<|channel|>analysis<|message|>" + m["reasoning_content"] + "<|end|>"
        for c in m.get("tool_calls") or []:
            fn = c.get("function", c)
            args = fn.get("arguments", "{}")
            args = args if isinstance(args, str) else json.dumps(args)
            out += f"<|start|>assistant to=functions.{fn.get('name')}<|channel|>commentary json<|message|>{args}<|call|>"
        text = _text_of(m.get("content", ""))
        if text or not out:
            out += "<|start|>assistant<|channel|>final<|message|>" + text + "<|end|>"
        return out

    def parse_tool(self, m, i, messages) -> str:
        return f"<|start|>functions.{m.get('name', 'tool')} to=assistant<|channel|>commentary<|message|>" + \
            _text_of(m.get("content", "")) + "<|end|>"

    def _prefix(self, messages, tools):
        head = ("<|start|>system<|message|>You are ChatGPT, a large language model trained by OpenAI.\n"
                f"Reasoning: {self.reasoning_effort}\n\n# Valid channels: analysis, commentary, final.<|end|>")
        if messages and messages[0]["role"] == "skip":
            return "", messages
        return head, messages

    def _assistant_message_stop_texts(self) -> tuple:
        return ("<|return|>", "<|end|>", "<|call|>", *super()._assistant_message_stop_texts())

    def assistant_message_content(self, response: str) -> str:
        text = super().assistant_message_content(response)
        marker = "<|channel|>final<|message|>"
        return text.split(marker)[-1] if marker in text else text


class MoonlightChatTemplateParser(ChatTemplateParser):
    system_token = "<|im_system|>system<|im_middle|>"
    user_token = "<|im_user|>user<|im_middle|>"
    assistant_token = "<|im_assistant|>assistant<|im_middle|>"
    tool_token = "<|im_system|>tool<|im_middle|>"
    eot_token = "<|im_end|>"

    def __init__(self, tokenizer, **kw):
        super().__init__(tokenizer, **kw)
        self.generation_prompt = self.assistant_token


class GlmChatTemplateParser(ChatTemplateParser):
    bos = "[gMASK]<sop>"
    system_token = "<|system|>\n"
    user_token = "<|user|>\n"
    assistant_token = "<|assistant|>\n"
    tool_token = "<|observation|>\n"
    eot_token = ""

    def __init__(self, tokenizer, **kw):
        super().__init__(tokenizer, **kw)
        self.generation_prompt = "<|assistant|>\n"

    def parse(self, messages, add_generation_prompt=False, tools=None, **kwargs) -> str:
        body = super().parse(messages, add_generation_prompt, tools, **kwargs)
        return self.bos + body if messages and messages[0]["role"] != "skip" else body

    def _assistant_message_stop_texts(self) -> tuple:
        return ("<|user|>", "<|observation|>", "<|endoftext|>", *super()._assistant_message_stop_texts())


class MultiModalChatTemplateParser(ChatTemplateParser):
    """Base of the vision-language parsers (reference: axon/engine/chat_template/parser.py:1301-1700). Callers pass
    ``messages`` only. Media travel inline as content parts - ``{"type": "image", "image": x}``, ``{"type": "image_url",
    "image_url": x | {"url": x}}`` and the same for ``video`` - or, in the legacy form, as ``<image>`` / ``<video>`` marks
    in the text with the payloads in ``images=`` / ``videos=`` (consumed in order). ``normalize`` brings both to the
    canonical part list, ``collect_media`` returns the payloads in placeholder order, ``parse`` renders through the
    processor's (else the tokenizer's) chat template."""
    LEGACY_MARKS = {"image": "<image>", "video": "<video>"}

    def __init__(self, tokenizer, processor=None, **kw):
        super().__init__(tokenizer, **kw)
        self.processor = processor

    @staticmethod
    def _unwrap(x):
        return x.get("url", x) if isinstance(x, dict) else x

    def normalize(self, messages, images=None, videos=None, allow_legacy_placeholders: bool = True) -> list:
        pools = {"image": list(images or []), "video": list(videos or [])}
        out = []
        for m in messages:
            c = m.get("content")
            parts = []
            if isinstance(c, str):
                if allow_legacy_placeholders and any(mark in c for mark in self.LEGACY_MARKS.values()):
                    rx = re.compile("(" + "|".join(re.escape(v) for v in self.LEGACY_MARKS.values()) + ")")
                    for piece in rx.split(c):
                        mod = next((k for k, v in self.LEGACY_MARKS.items() if v == piece), None)
                        if mod is None:
                            if piece:
                                parts.append({"type": "text", "text": piece})
                        else:
                            if not pools[mod]:
                                raise ValueError(f"more {self.LEGACY_MARKS[mod]} marks than {mod}s passed")
                            parts.append({"type": mod, mod: pools[mod].pop(0)})
                else:
                    out.append(dict(m))
                    continue
            else:
                for part in c or []:
                    if not isinstance(part, dict):
                        parts.append({"type": "text", "text": str(part)})
                        continue
                    t = part.get("type", "text")
                    if t in ("text", "input_text"):
                        parts.append({"type": "text", "text": part.get("text") or ""})
                    elif "image" in t:
                        parts.append({"type": "image", "image": self._unwrap(part.get("image", part.get("image_url", part.get(t))))})
                    elif "video" in t:
                        parts.append({"type": "video", "video": self._unwrap(part.get("video", part.get("video_url", part.get(t))))})
                    else:
                        parts.append(dict(part))
            out.append({**m, "content": parts})
        left = {k: len(v) for k, v in pools.items() if v}
        if left:
            raise ValueError(f"payloads without a placeholder: {left}")
        return out

    def count_placeholders(self, messages) -> tuple[int, int]:
        n = {"image": 0, "video": 0}
        for m in self.normalize(messages, allow_legacy_placeholders=False):
            for part in m["content"] if isinstance(m.get("content"), list) else []:
                if part.get("type") in n:
                    n[part["type"]] += 1
        return n["image"], n["video"]

    def collect_media(self, messages, images=None, videos=None) -> tuple[list, list]:
        got = {"image": [], "video": []}
        for m in self.normalize(messages, images, videos):
            for part in m["content"] if isinstance(m.get("content"), list) else []:
                if part.get("type") in got:
                    got[part["type"]].append(part[part["type"]])
        return got["image"], got["video"]

    def parse(self, messages, add_generation_prompt: bool = False, tools=None, **kwargs) -> str:
        norm = self.normalize(messages, kwargs.pop("images", None), kwargs.pop("videos", None),
                              kwargs.pop("allow_legacy_placeholders", True))
        owner = self.processor if hasattr(self.processor, "apply_chat_template") else self.tokenizer
        if not hasattr(owner, "apply_chat_template"):
            raise NotImplementedError(f"{type(self).__name__} needs a processor or tokenizer with a chat template")
        if tools:
            kwargs["tools"] = tools
        return owner.apply_chat_template(norm, tokenize=False, add_generation_prompt=add_generation_prompt, **kwargs)


class QwenVLChatTemplateParser(QwenChatTemplateParser):
    """Qwen-VL: images / videos render as ``<|vision_start|><|image_pad|><|vision_end|>``; the processor
    later expands each pad into N tokens. ``get_mm_regions`` reports where the placeholders sit in the
    rendered text and a content hash per item so the prefix tree can detect changed media."""
    default_system = "You are a helpful assistant."
    PLACEHOLDERS = {"image": "<|vision_start|><|image_pad|><|vision_end|>",
                    "video": "<|vision_start|><|video_pad|><|vision_end|>"}

    def __init__(self, tokenizer, processor=None, **kw):
        super().__init__(tokenizer, **kw)
        self.processor = processor

    @staticmethod
    def _content_hash(item) -> str:
        try:
            raw = item.tobytes() if hasattr(item, "tobytes") else repr(item).encode()
        except Exception:  # noqa: BLE001
            raw = repr(item).encode()
        return hashlib.sha1(raw).hexdigest()[:16]

    def get_mm_regions(self, input_key: str, messages) -> list:
        items = []
        for m in messages:
            c = m.get("content")
            if isinstance(c, list):
                for part in c:
                    if isinstance(part, dict) and part.get("type") in ("image", "image_url", "video", "video_url"):
                        mod = "image" if "image" in part["type"] else "video"
                        items.append((mod, part.get(mod) or part.get(part["type"]) or part))
        regions, pos = [], 0
        for mod, data in items:
            ph = self.PLACEHOLDERS[mod]
            start = input_key.find(ph, pos)
            if start < 0:
                break
            regions.append((start, start + len(ph), mod, self._content_hash(data), data))
            pos = start + len(ph)
        return regions

    async def tokenize(self, input_text: str, ctx: TokenizeContext | None = None) -> TokenizeOutput:
        out = await super().tokenize(input_text, ctx)
        if ctx is None or not (ctx.images or ctx.videos) or self.processor is None:
            return out
        from ..state.program_state import MultiModalData
        enc = self.processor(text=[input_text], images=ctx.images or None, videos=ctx.videos or None,
                             return_tensors="pt", **ctx.processor_kwargs)
        ids = enc["input_ids"][0].tolist()
        strs = [self.tokenizer.decode([i]) for i in ids]
        return TokenizeOutput(ids, strs, MultiModalData(image=ctx.images or None, video=ctx.videos or None,
                                                        processor_kwargs=ctx.processor_kwargs))
