from .core import ToolGroup, tool

__all__ = ["ToolGroup", "tool"]
