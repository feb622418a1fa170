"""A compact ReAct-style agent runner and an async dispatcher for batches of tasks.

Reference (peripheral package): skyrl-agent/skyrl_agent (ReAct / CodeAct runners, tool registry, async dispatchers with
bounded concurrency, trajectories returned with per-token loss masks for training).  This module keeps the parts the
trainer needs: token-in/token-out turns through any ``InferenceEngineInterface``, tool calls parsed from
``<tool>{"name": ..., "arguments": {...}}</tool>`` blocks, observations appended as user turns, a final answer in
``<answer>``, and a trajectory record (prompt ids, response ids, loss mask, log-probs) in the generator's format.
"""

from __future__ import annotations

import asyncio
import json
import re
from dataclasses import dataclass, field
from typing import Any, Awaitable, Callable, Dict, List, Optional
from ..utils.tokenizer import chat_template_ids

_TOOL = re.compile(r"<tool>(.*?)</tool>", re.DOTALL)
_ANSWER = re.compile(r"<answer>(.*?)</answer>", re.DOTALL)


@dataclass
class Tool:
    name: str
    fn: Callable[..., Any]
    description: str = ""

    async def __call__(self, **kwargs) -> str:
        out = self.fn(**kwargs)
        if asyncio.iscoroutine(out):
            out = await out
        return out if isinstance(out, str) else json.dumps(out, default=str)


@dataclass
class AgentResult:
    prompt_ids: List[int]
    response_ids: List[int]
    loss_mask: List[int]
    logprobs: Optional[List[float]]
    answer: Optional[str]
    turns: int
    stop_reason: str
    messages: List[Dict[str, str]] = field(default_factory=list)


class ReActAgent:
    def __init__(self, client, tokenizer, tools: List[Tool], max_turns: int = 8, max_tokens_per_turn: int = 512,
                 system_prompt: Optional[str] = None, sampling_params: Optional[Dict[str, Any]] = None):
        self.client, self.tok = client, tokenizer
        self.tools = {t.name: t for t in tools}
        self.max_turns, self.max_tokens = max_turns, max_tokens_per_turn
        self.sampling_params = dict(sampling_params or {})
        desc = "\n".join(f"- {t.name}: {t.description}" for t in tools)
        self.system_prompt = system_prompt or (
            "Solve the task. To call a tool write <tool>{\"name\": NAME, \"arguments\": {...}}</tool>; the result comes "
            "back as the next message. Finish with <answer>...</answer>.\nTools:\n" + desc)

    async def _observe(self, text: str) -> Optional[str]:
        m = _TOOL.search(text)
        if m is None:
            return None
        try:
            call = json.loads(m.group(1))
            tool = self.tools[call["name"]]
            return await tool(**(call.get("arguments") or {}))
        except KeyError as e:
            return f"Unknown tool or missing field: {e}"
        except Exception as e:  # noqa: BLE001 - the error text is what the model sees
            return f"Tool error: {type(e).__name__}: {e}"

    async def run(self, task: str, session_id: Optional[str] = None) -> AgentResult:
        msgs = [{"role": "system", "content": self.system_prompt}, {"role": "user", "content": task}]
        prompt_ids = chat_template_ids(self.tok, msgs, add_generation_prompt=True)
        ctx = list(prompt_ids)
        resp, mask, lps = [], [], []
        have_lp = True
        answer, stop = None, "max_turns"
        turns = 0
        sp = dict(self.sampling_params, max_generate_length=self.max_tokens)
        for turns in range(1, self.max_turns + 1):
            out = await self.client.generate({"prompt_token_ids": [ctx], "sampling_params": sp, "session_ids": [session_id]})
            ids = list(out["response_ids"][0])
            text = out["responses"][0] if out.get("responses") and out["responses"][0] is not None else self.tok.decode(ids)
            lp = out["response_logprobs"][0] if out.get("response_logprobs") else None
            resp += ids
            mask += [1] * len(ids)
            have_lp = have_lp and lp is not None
            lps += list(lp) if lp is not None else [0.0] * len(ids)
            ctx += ids
            msgs.append({"role": "assistant", "content": text})
            a = _ANSWER.search(text)
            if a is not None:
                answer, stop = a.group(1).strip(), "answer"
                break
            obs = await self._observe(text)
            if obs is None:
                stop = "no_action"
                break
            msgs.append({"role": "user", "content": obs})
            full = chat_template_ids(self.tok, msgs, add_generation_prompt=True)
            obs_ids = full[len(ctx):] if full[: len(ctx)] == ctx else list(self.tok.encode(obs))
            resp += obs_ids
            mask += [0] * len(obs_ids)  # environment tokens carry no loss
            lps += [0.0] * len(obs_ids)
            ctx += obs_ids
        return AgentResult(prompt_ids, resp, mask, lps if have_lp else None, answer, turns, stop, msgs)


class AsyncDispatcher:
    """Runs many agent tasks with bounded concurrency; results keep the input order."""

    def __init__(self, agent: ReActAgent, max_concurrency: int = 64):
        self.agent, self.sem = agent, asyncio.Semaphore(max_concurrency)

    async def _one(self, i: int, task: str):
        async with self.sem:
            return i, await self.agent.run(task, session_id=f"agent-{i}")

    async def run(self, tasks: List[str]) -> List[AgentResult]:
        done = await asyncio.gather(*[self._one(i, t) for i, t in enumerate(tasks)])
        return [r for _, r in sorted(done, key=lambda x: x[0])]
