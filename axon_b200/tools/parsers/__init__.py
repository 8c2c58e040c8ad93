"""Model-specific tool-call parsers: extract ``ToolCall``s from sampled text, and format calls,
results and the tool section of the system prompt the way each model family expects
(reference: axon/tools/parsers/base_parser.py:44-154 and the qwen / r1 / json / xml / glm /
openai_harmony / gemma4 parsers)."""
from __future__ import annotations

import json
import re
from abc import ABC, abstractmethod
from typing import Any

from ..types import ToolCall, ToolResult

_PARSERS: dict[str, type] = {}


class ToolCallParser(ABC):
    @abstractmethod
    def parse(self, response: str) -> tuple[list[ToolCall], str]:
        """Returns (tool calls found, remaining text with the call markup removed)."""

    @abstractmethod
    def format_tool_call(self, tool_call: ToolCall) -> str: ...

    def format_tool_calls(self, tool_calls: list[ToolCall]) -> str:
        return "\n".join(self.format_tool_call(c) for c in tool_calls)

    def format_tool_result(self, content: Any, name: str = "") -> str:
        return str(content)

    def format_tool_results(self, results: list[ToolResult]) -> str:
        return "\n".join(self.format_tool_result(r.content, r.name) for r in results)

    def get_tool_system_prompt(self, tools_json: list[dict]) -> str:
        return "# Tools\n\n" + "\n".join(json.dumps(t, ensure_ascii=False) for t in tools_json)


def register_parser(name: str):
    def deco(cls):
        if not (isinstance(cls, type) and issubclass(cls, ToolCallParser)):
            raise TypeError(f"{cls} is not a ToolCallParser")
        _PARSERS[name] = cls
        return cls
    return deco


def get_tool_call_parser(name: str, **kwargs) -> ToolCallParser:
    if name not in _PARSERS:
        raise ValueError(f"unknown tool-call parser '{name}'. Available: {sorted(_PARSERS)}")
    return _PARSERS[name](**kwargs)


def _loads_lenient(raw: str):
    """json.loads with the usual model slips repaired: trailing commas, single quotes, unbalanced braces."""
    raw = raw.strip()
    for cand in (raw, re.sub(r",\s*([}\]])", r"\1", raw), raw.replace("'", '"'),
                 raw + "}" * max(0, raw.count("{") - raw.count("}"))):
        try:
            return json.loads(cand)
        except json.JSONDecodeError:
            continue
    return None


def _call_from_obj(obj) -> ToolCall | None:
    if not isinstance(obj, dict) or "name" not in obj:
        return None
    args = obj.get("arguments", obj.get("parameters", {}))
    if isinstance(args, str):
        args = _loads_lenient(args) or {"_raw": args}
    return ToolCall(name=str(obj["name"]), arguments=args or {})


@register_parser("qwen")
@register_parser("hermes")
class QwenToolCallParser(ToolCallParser):
    """``<tool_call>{"name": ..., "arguments": {...}}</tool_call>``; results in ``<tool_response>``."""
    _RX = re.compile(r"<tool_call>\s*(.*?)\s*(?:</tool_call>|$)", re.S)

    def parse(self, response: str):
        calls = [c for c in (_call_from_obj(_loads_lenient(m)) for m in self._RX.findall(response)) if c]
        return calls, self._RX.sub("", response).strip()

    def format_tool_call(self, tool_call: ToolCall) -> str:
        return "<tool_call>\n" + json.dumps(tool_call.to_dict(), ensure_ascii=False) + "\n</tool_call>"

    def format_tool_result(self, content: Any, name: str = "") -> str:
        return f"<tool_response>\n{content}\n</tool_response>"

    def get_tool_system_prompt(self, tools_json):
        body = "\n".join(json.dumps(t, ensure_ascii=False) for t in tools_json)
        return ("# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
                "You are provided with function signatures within <tools></tools> XML tags:\n<tools>\n" + body +
                "\n</tools>\n\nFor each function call, return a json object with function name and arguments within "
                "<tool_call></tool_call> XML tags:\n<tool_call>\n{\"name\": <function-name>, \"arguments\": "
                "<args-json-object>}\n</tool_call>")


@register_parser("r1")
class R1ToolCallParser(ToolCallParser):
    """DeepSeek-R1 markup: ``<｜tool▁call▁begin｜>function<｜tool▁sep｜>NAME\\n```json\\n{...}\\n```<｜tool▁call▁end｜>``."""
    B, S, E = "<｜tool▁call▁begin｜>", "<｜tool▁sep｜>", "<｜tool▁call▁end｜>"
    _RX = re.compile(r"<｜tool▁call▁begin｜>(?:function)?<｜tool▁sep｜>(.*?)\n```json\n(.*?)\n```<｜tool▁call▁end｜>", re.S)

    def parse(self, response: str):
        calls = []
        for name, raw in self._RX.findall(response):
            calls.append(ToolCall(name=name.strip(), arguments=_loads_lenient(raw) or {}))
        text = self._RX.sub("", response).replace("<｜tool▁calls▁begin｜>", "").replace("<｜tool▁calls▁end｜>", "")
        return calls, text.strip()

    def format_tool_call(self, c: ToolCall) -> str:
        return f"{self.B}function{self.S}{c.name}\n```json\n{json.dumps(c.arguments, ensure_ascii=False)}\n```{self.E}"

    def format_tool_calls(self, calls):
        return "<｜tool▁calls▁begin｜>" + "\n".join(self.format_tool_call(c) for c in calls) + "<｜tool▁calls▁end｜>"

    def format_tool_result(self, content, name=""):
        return f"<｜tool▁output▁begin｜>{content}<｜tool▁output▁end｜>"


@register_parser("json")
class JsonToolCallParser(ToolCallParser):
    """A bare JSON object (or list of objects, or fenced ```json block) with ``name`` / ``arguments``."""
    _FENCE = re.compile(r"```(?:json)?\s*(.*?)```", re.S)

    def parse(self, response: str):
        blobs = self._FENCE.findall(response) or [response]
        calls, rest = [], response
        for b in blobs:
            start = min([i for i in (b.find("{"), b.find("[")) if i >= 0], default=-1)
            if start < 0:
                continue
            obj = _loads_lenient(b[start:])
            for o in (obj if isinstance(obj, list) else [obj]):
                c = _call_from_obj(o)
                if c:
                    calls.append(c)
        if calls:
            rest = self._FENCE.sub("", response).strip() if self._FENCE.search(response) else ""
        return calls, rest

    def format_tool_call(self, c: ToolCall) -> str:
        return json.dumps(c.to_dict(), ensure_ascii=False)


@register_parser("xml")
class XmlToolCallParser(ToolCallParser):
    """``<function=NAME><parameter=KEY>VALUE</parameter>...</function>`` (Qwen3-Coder style)."""
    _FN = re.compile(r"<function=([^>]+)>(.*?)</function>", re.S)
    _PARAM = re.compile(r"<parameter=([^>]+)>(.*?)</parameter>", re.S)

    def parse(self, response: str):
        calls = []
        for name, body in self._FN.findall(response):
            args = {}
            for k, v in self._PARAM.findall(body):
                v = v.strip("\n")
                parsed = _loads_lenient(v) if v[:1] in "[{0123456789-tfn\"" else None
                args[k.strip()] = parsed if parsed is not None else v
            calls.append(ToolCall(name=name.strip(), arguments=args))
        text = re.sub(r"<tool_call>\s*</tool_call>", "", self._FN.sub("", response))
        return calls, text.replace("<tool_call>", "").replace("</tool_call>", "").strip()

    def format_tool_call(self, c: ToolCall) -> str:
        params = "\n".join(f"<parameter={k}>\n{v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)}\n</parameter>"
                           for k, v in c.arguments.items())
        return f"<tool_call>\n<function={c.name}>\n{params}\n</function>\n</tool_call>"

    def format_tool_result(self, content, name=""):
        return f"<tool_response>\n{content}\n</tool_response>"


@register_parser("glm")
class GlmToolCallParser(ToolCallParser):
    """GLM-4: ``<tool_call>NAME\\n<arg_key>K</arg_key>\\n<arg_value>V</arg_value>...</tool_call>``."""
    _RX = re.compile(r"<tool_call>\s*([^\n<]+)\s*(.*?)</tool_call>", re.S)
    _KV = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)

    def parse(self, response: str):
        calls = []
        for name, body in self._RX.findall(response):
            args = {}
            for k, v in self._KV.findall(body):
                parsed = _loads_lenient(v) if v.strip()[:1] in "[{0123456789-tfn\"" else None
                args[k.strip()] = parsed if parsed is not None else v
            calls.append(ToolCall(name=name.strip(), arguments=args))
        return calls, self._RX.sub("", response).strip()

    def format_tool_call(self, c: ToolCall) -> str:
        kv = "\n".join(f"<arg_key>{k}</arg_key>\n<arg_value>{v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)}</arg_value>"
                       for k, v in c.arguments.items())
        return f"<tool_call>{c.name}\n{kv}\n</tool_call>"

    def format_tool_result(self, content, name=""):
        return f"<tool_response>\n{content}\n</tool_response>"


@register_parser("openai_harmony")
class HarmonyToolCallParser(ToolCallParser):
    """gpt-oss: ``<|start|>assistant to=functions.NAME<|channel|>commentary json<|message|>{...}<|call|>``."""
    _RX = re.compile(r"to=functions\.([\w\-.]+).*?<\|message\|>(.*?)(?:<\|call\|>|<\|end\|>|$)", re.S)

    def parse(self, response: str):
        calls = [ToolCall(name=n, arguments=_loads_lenient(raw) or {}) for n, raw in self._RX.findall(response)]
        final = response.split("<|channel|>final<|message|>")[-1] if "<|channel|>final<|message|>" in response else \
            self._RX.sub("", response)
        for tok in ("<|end|>", "<|return|>", "<|call|>", "<|start|>assistant"):
            final = final.replace(tok, "")
        return calls, final.strip()

    def format_tool_call(self, c: ToolCall) -> str:
        return (f"<|start|>assistant to=functions.{c.name}<|channel|>commentary json<|message|>"
                f"{json.dumps(c.arguments, ensure_ascii=False)}<|call|>")

    def format_tool_calls(self, calls):
        return "".join(self.format_tool_call(c) for c in calls)


@register_parser("gemma")
class GemmaToolCodeParser(ToolCallParser):
    """Gemma 2 / 3: fenced ``tool_code`` blocks holding ``name(arg=value, ...)`` Python-style calls."""
    _RX = re.compile(r"```tool_code\s*(.*?)\s*```", re.S)
    _CALL = re.compile(r"([\w.]+)\((.*)\)\s*$", re.S)

    def parse(self, response: str):
        import ast
        calls = []
        for body in self._RX.findall(response):
            m = self._CALL.match(body.strip())
            if not m:
                continue
            args = {}
            try:
                node = ast.parse(f"f({m.group(2)})", mode="eval").body
                for kw in node.keywords:
                    args[kw.arg] = ast.literal_eval(kw.value)
            except (SyntaxError, ValueError):
                args = {"_raw": m.group(2)}
            calls.append(ToolCall(name=m.group(1), arguments=args))
        return calls, self._RX.sub("", response).strip()

    def format_tool_call(self, c: ToolCall) -> str:
        return "```tool_code\n" + c.name + "(" + ", ".join(f"{k}={v!r}" for k, v in c.arguments.items()) + ")\n```"

    def format_tool_result(self, content, name=""):
        return f"```tool_output\n{content}\n```"


_G4_Q = '<|"|>'


class _Gemma4Values:
    """Gemma-4's compact value grammar: ``{key:value,...}``, ``[v,...]``, strings between ``<|"|>`` marks, ``true`` /
    ``false`` / ``null``, numbers; a bare word that is none of those is a string."""

    def __init__(self, text: str):
        self.t, self.i = text, 0

    def _ws(self):
        while self.i < len(self.t) and self.t[self.i].isspace():
            self.i += 1

    def value(self):
        self._ws()
        t = self.t
        if t.startswith(_G4_Q, self.i):
            end = t.find(_G4_Q, self.i + len(_G4_Q))
            end = len(t) if end < 0 else end
            out = t[self.i + len(_G4_Q):end]
            self.i = min(len(t), end + len(_G4_Q))
            return out
        if self.i < len(t) and t[self.i] == "{":
            self.i += 1
            return self.members("}")
        if self.i < len(t) and t[self.i] == "[":
            self.i += 1
            out = []
            while True:
                self._ws()
                if self.i >= len(t) or t[self.i] == "]":
                    self.i += 1
                    return out
                out.append(self.value())
                self._ws()
                if self.i < len(t) and t[self.i] == ",":
                    self.i += 1
        j = self.i
        while j < len(t) and t[j] not in ",}]":
            j += 1
        word = t[self.i:j].strip()
        self.i = j
        if word in ("true", "false"):
            return word == "true"
        if word == "null":
            return None
        try:
            return float(word) if any(c in word for c in ".eE") else int(word)
        except ValueError:
            return word

    def members(self, close: str | None) -> dict:
        out = {}
        t = self.t
        while True:
            self._ws()
            if self.i >= len(t) or (close and t[self.i] == close):
                self.i += 1
                return out
            if t.startswith(_G4_Q, self.i):
                key = self.value()
            else:
                j = t.find(":", self.i)
                if j < 0:
                    self.i = len(t)
                    return out
                key = t[self.i:j].strip()
                self.i = j
            self._ws()
            if self.i < len(t) and t[self.i] == ":":
                self.i += 1
            out[key] = self.value()
            self._ws()
            if self.i < len(t) and t[self.i] == ",":
                self.i += 1


def _g4_render(v, quote_keys: bool = False) -> str:
    if isinstance(v, str):
        return f"{_G4_Q}{v}{_G4_Q}"
    if isinstance(v, bool):
        return "true" if v else "false"
    if v is None:
        return "null"
    if isinstance(v, dict):
        return "{" + ",".join(f"{(_G4_Q + str(k) + _G4_Q) if quote_keys else k}:{_g4_render(v[k], quote_keys)}" for k in sorted(v)) + "}"
    if isinstance(v, (list, tuple)):
        return "[" + ",".join(_g4_render(x, quote_keys) for x in v) + "]"
    return str(v)


def _g4_balanced(text: str, start: int) -> int:
    """Index of the brace that closes the one at ``start`` (string marks respected); -1 if it never closes."""
    depth, i = 0, start
    while i < len(text):
        if text.startswith(_G4_Q, i):
            j = text.find(_G4_Q, i + len(_G4_Q))
            if j < 0:
                return -1
            i = j + len(_G4_Q)
            continue
        if text[i] == "{":
            depth += 1
        elif text[i] == "}":
            depth -= 1
            if depth == 0:
                return i
        i += 1
    return -1


@register_parser("gemma4")
class Gemma4ToolCallParser(ToolCallParser):
    """Gemma-4's native tool grammar (reference: axon/tools/parsers/gemma4_parser.py):
    ``<|tool_call>call:name{arg:<|"|>text<|"|>,n:3}<tool_call|>`` in the model turn, results as
    ``<|tool_response>response:name{value:...}<tool_response|>``, declarations as ``<|tool>declaration:...<tool|>``."""
    CALL_START, CALL_END = "<|tool_call>", "<tool_call|>"
    RESP_START, RESP_END = "<|tool_response>", "<tool_response|>"

    def parse(self, response: str):
        calls, kept, pos = [], [], 0
        while True:
            start = response.find(self.CALL_START, pos)
            if start < 0:
                kept.append(response[pos:])
                break
            head = start + len(self.CALL_START)
            brace = response.find("{", head)
            if not response.startswith("call:", head) or brace < 0:
                kept.append(response[pos:head])
                pos = head
                continue
            close = _g4_balanced(response, brace)
            if close < 0:
                kept.append(response[pos:])
                break
            name = response[head + len("call:"):brace].strip()
            args = _Gemma4Values(response[brace + 1:close]).members(None)
            end = close + 1
            for closer in (self.CALL_END, "<turn|>"):
                if response.startswith(closer, end):
                    end += len(closer)
                    break
            if response.startswith(self.RESP_START, end):          # the template leaves a bare opener after a pending call
                end += len(self.RESP_START)
            kept.append(response[pos:start])
            calls.append(ToolCall(name=name, arguments=args))
            pos = end
        return calls, "".join(kept).strip()

    def format_tool_call(self, c: ToolCall) -> str:
        args = c.arguments if isinstance(c.arguments, dict) else {"raw": c.arguments}
        return f"{self.CALL_START}call:{c.name}{{" + ",".join(f"{k}:{_g4_render(args[k])}" for k in sorted(args)) + f"}}{self.CALL_END}"

    def format_tool_calls(self, calls):
        return "".join(self.format_tool_call(c) for c in calls)

    def format_tool_result(self, content, name=""):
        inner = ",".join(f"{k}:{_g4_render(content[k])}" for k in sorted(content)) if isinstance(content, dict) \
            else f"value:{_g4_render(content)}"
        return f"{self.RESP_START}response:{name or 'unknown'}{{{inner}}}{self.RESP_END}"

    def get_tool_system_prompt(self, tools) -> str:
        out = []
        for tool in tools:
            fn = tool.get("function", tool)
            decl = {"description": fn.get("description", "")}
            params = fn.get("parameters") or {}
            if params:
                props = {k: {kk: (str(vv).upper() if kk == "type" else vv) for kk, vv in v.items()} for k, v in (params.get("properties") or {}).items()}
                decl["parameters"] = {"properties": props, "required": list(params.get("required") or []),
                                      "type": str(params.get("type", "object")).upper()}
            out.append(f"<|tool>declaration:{fn.get('name', '')}{_g4_render(decl)}<tool|>")
        return "".join(out)


