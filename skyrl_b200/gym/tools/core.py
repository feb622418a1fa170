"""Tool groups: named collections of ``@tool`` methods an environment can expose to the model
(reference: skyrl-gym/skyrl_gym/tools/core.py)."""

from __future__ import annotations

from typing import Any, Callable, Dict, List


def tool(fn: Callable) -> Callable:
    """Mark a ``ToolGroup`` method as callable by the agent."""
    fn._is_tool = True
    return fn


class ToolGroup:
    def __init__(self, name: str):
        self.name = name
        self._tools: Dict[str, Callable] = {}
        for attr in dir(self):
            if attr.startswith("__"):
                continue
            fn = getattr(self, attr)
            if callable(fn) and getattr(fn, "_is_tool", False):
                self._tools[attr] = fn

    def get_name(self) -> str:
        return self.name

    def get_tool(self, name: str) -> Callable | None:
        return self._tools.get(name)

    def get_tool_names(self) -> List[str]:
        return sorted(self._tools)

    def execute_tool(self, name: str, *args, **kwargs) -> Any:
        fn = self._tools.get(name)
        if fn is None:
            raise ValueError(f"tool '{name}' not found in group '{self.name}'")
        return fn(*args, **kwargs)

    def get_tool_to_group_mapping(self) -> Dict[str, str]:
        return {t: self.name for t in self._tools}
