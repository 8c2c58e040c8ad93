"""``Tool``: something an agent can call during a rollout. Wrap a plain function (its schema is
derived from the signature and docstring) or subclass and override ``forward`` / ``async_forward``
(reference: axon/tools/tools.py:121-260). ``MCPTool`` forwards to a Model-Context-Protocol session."""
from __future__ import annotations

import asyncio
import inspect
from typing import Any, Callable

from .types import ToolOutput

_JSON_TYPES = {int: "integer", float: "number", str: "string", bool: "boolean", list: "array", dict: "object"}


def _function_to_schema(func: Callable) -> dict:
    sig = inspect.signature(func)
    doc = inspect.getdoc(func) or ""
    props, required = {}, []
    for name, p in sig.parameters.items():
        if name in ("self", "kwargs", "args"):
            continue
        ann = p.annotation if p.annotation is not inspect.Parameter.empty else str
        origin = getattr(ann, "__origin__", ann)
        props[name] = {"type": _JSON_TYPES.get(origin, "string")}
        if p.default is inspect.Parameter.empty:
            required.append(name)
    return {"type": "function", "function": {"name": func.__name__, "description": doc.split("\n\n")[0],
                                             "parameters": {"type": "object", "properties": props, "required": required}}}


class Tool:
    def __init__(self, name: str | None = None, description: str | None = None, function: Callable | None = None):
        self.function = function
        if function is not None:
            self._json = _function_to_schema(function)
            if name:
                self._json["function"]["name"] = name
            if description:
                self._json["function"]["description"] = description
            self.name = self._json["function"]["name"]
            self.description = self._json["function"]["description"]
        else:
            self._json = None
            self.name = name or self.__class__.__name__
            self.description = description or (inspect.getdoc(self) or "")

    @property
    def json(self) -> dict:
        if self._json is not None:
            return self._json
        return {"type": "function", "function": {"name": self.name, "description": self.description,
                                                 "parameters": {"type": "object", "properties": {}, "required": []}}}

    def forward(self, **kwargs) -> ToolOutput:
        if self.function is None:
            raise NotImplementedError("override forward() or pass function=")
        try:
            res = self.function(**kwargs)
            if inspect.isawaitable(res):
                res = asyncio.run(res)
            return res if isinstance(res, ToolOutput) else ToolOutput(name=self.name, output=res)
        except Exception as e:  # noqa: BLE001
            return ToolOutput(name=self.name, error=f"{type(e).__name__}: {e}")

    async def async_forward(self, **kwargs) -> ToolOutput:
        if self.function is not None and inspect.iscoroutinefunction(self.function):
            try:
                res = await self.function(**kwargs)
                return res if isinstance(res, ToolOutput) else ToolOutput(name=self.name, output=res)
            except Exception as e:  # noqa: BLE001
                return ToolOutput(name=self.name, error=f"{type(e).__name__}: {e}")
        return await asyncio.get_running_loop().run_in_executor(None, lambda: self.forward(**kwargs))

    def __call__(self, **kwargs) -> ToolOutput:
        return self.forward(**kwargs)


class MCPTool(Tool):
    def __init__(self, session, tool_name: str, tool_description: str, tool_schema: dict):
        super().__init__(name=tool_name, description=tool_description)
        self.session, self.schema = session, tool_schema

    @property
    def json(self) -> dict:
        return {"type": "function", "function": {"name": self.name, "description": self.description,
                                                 "parameters": self.schema}}

    async def async_forward(self, **kwargs) -> ToolOutput:
        try:
            res = await self.session.call_tool(self.name, kwargs)
            parts = getattr(res, "content", res)
            text = "\n".join(getattr(p, "text", str(p)) for p in parts) if isinstance(parts, (list, tuple)) else str(parts)
            return ToolOutput(name=self.name, output=text)
        except Exception as e:  # noqa: BLE001
            return ToolOutput(name=self.name, error=f"{type(e).__name__}: {e}")

    def forward(self, **kwargs) -> ToolOutput:
        return asyncio.run(self.async_forward(**kwargs))
