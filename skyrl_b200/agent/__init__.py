"""Agent layer: ReAct runner, tools, tasks, dispatchers and the adapter that lets the trainer use agents as its
generator (reference: the peripheral skyrl-agent package)."""

from .dispatchers import DISPATCHER_REGISTRY, register_dispatcher
from .react import AgentResult, AsyncDispatcher, ReActAgent, Tool
from .runner import AgentGenerator, AgentRunner
from .tasks import TASK_REGISTRY, BaseTask, GeneralReactTask, register_task
from .tools import TOOL_REGISTRY, BM25Index, exact_match, make_tool, normalize_answer, register_tool

__all__ = ["AgentResult", "AsyncDispatcher", "ReActAgent", "Tool", "AgentRunner", "AgentGenerator", "BaseTask",
           "GeneralReactTask", "register_task", "TASK_REGISTRY", "register_dispatcher", "DISPATCHER_REGISTRY",
           "register_tool", "TOOL_REGISTRY", "make_tool", "BM25Index", "exact_match", "normalize_answer"]
