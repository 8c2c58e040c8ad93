"""Tool executors: run parsed tool calls locally or against an HTTP tool server
(reference: axon/tools/executors.py:122-350)."""
from __future__ import annotations

import asyncio
import importlib
import importlib.util
import os
from abc import ABC, abstractmethod
from typing import Any

from .tools import Tool
from .types import ToolCall, ToolOutput, ToolResult


def load_tool_class(path: str) -> type:
    """``pkg.module:ClassName`` or ``/path/file.py:ClassName``."""
    mod_path, _, cls_name = path.rpartition(":")
    if not mod_path:
        raise ValueError(f"expected 'module:ClassName', got '{path}'")
    if mod_path.endswith(".py") or os.path.sep in mod_path:
        spec = importlib.util.spec_from_file_location(os.path.splitext(os.path.basename(mod_path))[0], mod_path)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
    else:
        module = importlib.import_module(mod_path)
    if not hasattr(module, cls_name):
        raise AttributeError(f"Module {mod_path} does not have class '{cls_name}'")
    return getattr(module, cls_name)


def _error_result(call: ToolCall, error: str) -> ToolResult:
    return ToolResult(tool_call_id=call.id, name=call.name, content=f"Error: {error}", success=False)


def _success_result(call: ToolCall, out: ToolOutput) -> ToolResult:
    return ToolResult(tool_call_id=call.id, name=call.name, content=out.to_content_string(), success=out.error is None,
                      metadata=out.metadata)


class ToolExecutor(ABC):
    @abstractmethod
    async def execute(self, tool_call: ToolCall) -> ToolResult: ...

    async def execute_batch(self, tool_calls: list[ToolCall]) -> list[ToolResult]:
        return list(await asyncio.gather(*(self.execute(c) for c in tool_calls)))

    def execute_sync(self, tool_call: ToolCall) -> ToolResult:
        return asyncio.run(self.execute(tool_call))

    def execute_batch_sync(self, tool_calls: list[ToolCall]) -> list[ToolResult]:
        return asyncio.run(self.execute_batch(tool_calls))


class LocalToolExecutor(ToolExecutor):
    """Registry of in-process tools. Values may be Tool instances, Tool classes, plain functions or
    'module:Class' strings."""

    def __init__(self, tools: dict[str, Any] | None = None):
        self._tools: dict[str, Tool] = {}
        for name, t in (tools or {}).items():
            self.register(name, t)

    def register(self, name: str, tool: Any) -> None:
        if isinstance(tool, str):
            tool = load_tool_class(tool)
        if isinstance(tool, type):
            tool = tool()
        if not isinstance(tool, Tool):
            if callable(tool):
                tool = Tool(name=name, function=tool)
            else:
                raise TypeError(f"cannot register {tool!r} as a tool")
        self._tools[name] = tool

    def get(self, name: str) -> Tool | None:
        return self._tools.get(name)

    def __getitem__(self, name: str) -> Tool:
        return self._tools[name]

    def __contains__(self, name: str) -> bool:
        return name in self._tools

    def __len__(self) -> int:
        return len(self._tools)

    def __iter__(self):
        return iter(self._tools)

    def names(self) -> list[str]:
        return list(self._tools)

    @property
    def tools(self) -> dict[str, Tool]:
        return dict(self._tools)

    @property
    def schemas(self) -> list[dict]:
        return [t.json for t in self._tools.values()]

    async def execute(self, tool_call: ToolCall) -> ToolResult:
        tool = self._tools.get(tool_call.name)
        if tool is None:
            return _error_result(tool_call, f"unknown tool '{tool_call.name}'. Available: {self.names()}")
        try:
            out = await tool.async_forward(**tool_call.arguments)
        except TypeError as e:
            return _error_result(tool_call, f"bad arguments: {e}")
        except Exception as e:  # noqa: BLE001
            return _error_result(tool_call, f"{type(e).__name__}: {e}")
        return _success_result(tool_call, out)


class HTTPToolExecutor(ToolExecutor):
    """POSTs ``{name, arguments}`` to ``{base_url}/execute``; expects ``{content, success}``."""

    def __init__(self, http_client, base_url: str):
        self.client, self.base_url = http_client, base_url.rstrip("/")

    async def execute(self, tool_call: ToolCall) -> ToolResult:
        try:
            r = await self.client.post(f"{self.base_url}/execute", json=tool_call.to_dict())
            r.raise_for_status()
            d = r.json()
            return ToolResult(tool_call.id, tool_call.name, str(d.get("content", "")), bool(d.get("success", True)))
        except Exception as e:  # noqa: BLE001
            return _error_result(tool_call, f"{type(e).__name__}: {e}")
