"""Tool-call data types (reference: axon/tools/types.py)."""
from __future__ import annotations

import json
import uuid
from dataclasses import dataclass, field
from typing import Any


@dataclass
class ToolCall:
    name: str
    arguments: dict = field(default_factory=dict)
    id: str = field(default_factory=lambda: "call_" + uuid.uuid4().hex[:24])

    def to_dict(self) -> dict:
        return {"name": self.name, "arguments": self.arguments}

    def to_openai_dict(self) -> dict:
        return {"id": self.id, "type": "function",
                "function": {"name": self.name, "arguments": json.dumps(self.arguments, ensure_ascii=False)}}

    @classmethod
    def from_raw_tool_call(cls, d: Any) -> "ToolCall":
        """Accepts a ToolCall, an OpenAI-style dict ({id, function:{name, arguments}}) or a flat dict."""
        if isinstance(d, ToolCall):
            return d
        if hasattr(d, "function"):          # openai SDK object
            d = {"id": getattr(d, "id", None), "function": {"name": d.function.name, "arguments": d.function.arguments}}
        fn = d.get("function", d)
        args = fn.get("arguments", fn.get("parameters", {}))
        if isinstance(args, str):
            try:
                args = json.loads(args) if args.strip() else {}
            except json.JSONDecodeError:
                args = {"_raw": args}
        kw = {"id": d["id"]} if d.get("id") else {}
        return cls(name=fn.get("name", ""), arguments=args or {}, **kw)


@dataclass
class ToolOutput:
    name: str = ""
    output: Any = None
    error: str | None = None
    metadata: dict = field(default_factory=dict)

    def to_content_string(self) -> str:
        if self.error:
            return f"Error: {self.error}"
        if self.output is None:
            return ""
        if isinstance(self.output, (dict, list)):
            return json.dumps(self.output, ensure_ascii=False)
        return str(self.output)

    def __str__(self) -> str:
        return self.to_content_string()


@dataclass
class ToolResult:
    tool_call_id: str
    name: str
    content: str
    success: bool = True
    metadata: dict = field(default_factory=dict)

    def to_openai_dict(self) -> dict:
        return {"role": "tool", "tool_call_id": self.tool_call_id, "name": self.name, "content": self.content}
