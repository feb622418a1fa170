"""Agent runners on top of the inference client: a ReAct loop with tool calls and an async dispatcher
(the reference ships these as the separate ``skyrl-agent`` package)."""
from .react import AgentResult, AsyncDispatcher, ReActAgent, Tool  # noqa: F401
