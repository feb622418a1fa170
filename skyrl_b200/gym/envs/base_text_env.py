"""``BaseTextEnv``: text-in / text-out environment with optional tool groups and a turn limit
(reference: skyrl-gym/skyrl_gym/envs/base_text_env.py:9-100)."""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

from ..core import Env, EnvStepOutput
from ..tools.core import ToolGroup

ConversationType = List[Dict[str, Any]]


class BaseTextEnvStepOutput(EnvStepOutput, total=False):
    pass


class BaseTextEnv(Env[ConversationType, str]):
    def __init__(self):
        self.turns = 0
        self.max_turns = 1
        self.tool_groups: List[ToolGroup] = []
        self.tool_to_toolgroup: Dict[str, str] = {}

    def init_tool_groups(self, tool_groups: Optional[List[ToolGroup]] = None) -> None:
        self.tool_groups = list(tool_groups or [])
        self.tool_to_toolgroup = {}
        for g in self.tool_groups:
            for t in g.get_tool_names():
                self.tool_to_toolgroup[t] = g.get_name()

    def _execute_tool(self, tool_group_name: str, tool_name: str, tool_input: Any) -> Any:
        for g in self.tool_groups:
            if g.get_name() == tool_group_name:
                if isinstance(tool_input, (list, tuple)):
                    return g.execute_tool(tool_name, *tool_input)
                if isinstance(tool_input, dict):
                    return g.execute_tool(tool_name, **tool_input)
                return g.execute_tool(tool_name, tool_input)
        raise ValueError(f"tool group '{tool_group_name}' not found")

    def init(self, prompt: ConversationType) -> Tuple[ConversationType, Dict[str, Any]]:
        return prompt, {}

    def step(self, action: str) -> BaseTextEnvStepOutput:
        raise NotImplementedError
