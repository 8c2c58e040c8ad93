from .executors import HTTPToolExecutor, LocalToolExecutor, ToolExecutor, load_tool_class
from .parsers import ToolCallParser, get_tool_call_parser, register_parser
from .tools import MCPTool, Tool
from .types import ToolCall, ToolOutput, ToolResult

__all__ = ["Tool", "MCPTool", "ToolCall", "ToolOutput", "ToolResult", "ToolExecutor", "LocalToolExecutor",
           "HTTPToolExecutor", "load_tool_class", "ToolCallParser", "register_parser", "get_tool_call_parser"]
