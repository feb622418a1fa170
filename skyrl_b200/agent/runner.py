"""``AgentRunner``: dataset rows -> agent episodes -> a generator output the trainer can consume.

Reference (peripheral package): skyrl-agent/skyrl_agent/auto.py (``AutoAgentRunner``: builds agent, task and
dispatcher from a config, runs ``num_trajectories`` episodes per instance, post-processes the trajectories into
prompt ids / response ids / loss masks / rewards for the training integration).  ``AgentGenerator`` plugs the runner in
where the trainer expects a ``GeneratorInterface``.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

from ..train.generators.base import GeneratorInput, GeneratorInterface, GeneratorOutput
from .dispatchers import DISPATCHER_REGISTRY
from .react import AgentResult, ReActAgent, Tool
from .tasks import TASK_REGISTRY, BaseTask
from .tools import make_tool


class AgentRunner:
    """``cfg`` keys: ``task`` (registered task name), ``tools`` (list of names or ``{"name": ..., **kwargs}``),
    ``dispatcher`` (``async_batch`` | ``async_pipeline``), ``num_trajectories``, ``max_turns``, ``max_tokens_per_turn``,
    ``max_parallel_agents`` / ``max_eval_parallel_agents``, ``sampling_params``, ``system_prompt``."""

    def __init__(self, cfg: Dict[str, Any], client, tokenizer, extra_tools: Optional[List[Tool]] = None):
        self.cfg = dict(cfg)
        tools = list(extra_tools or [])
        for spec in self.cfg.get("tools", []):
            tools.append(make_tool(spec) if isinstance(spec, str) else make_tool(spec["name"], **{k: v for k, v in spec.items() if k != "name"}))
        self.agent = ReActAgent(client, tokenizer, tools, max_turns=int(self.cfg.get("max_turns", 8)),
                                max_tokens_per_turn=int(self.cfg.get("max_tokens_per_turn", 512)),
                                system_prompt=self.cfg.get("system_prompt"), sampling_params=self.cfg.get("sampling_params"))
        name = self.cfg.get("task", "general_react")
        if name not in TASK_REGISTRY:
            raise KeyError(f"unknown task '{name}'; registered: {sorted(TASK_REGISTRY)}")
        self.task_cls = TASK_REGISTRY[name]
        disp = self.cfg.get("dispatcher", "async_batch")
        if disp not in DISPATCHER_REGISTRY:
            raise KeyError(f"unknown dispatcher '{disp}'; registered: {sorted(DISPATCHER_REGISTRY)}")
        self.dispatch = DISPATCHER_REGISTRY[disp]

    async def run(self, instances: List[Dict[str, Any]]) -> Dict[str, Any]:
        """Runs ``num_trajectories`` episodes per instance.  Returns per-episode lists ordered instance-major (all
        samples of instance 0, then instance 1, ...), the order ``n_samples_per_prompt`` grouping expects."""
        n_traj = int(self.cfg.get("num_trajectories", 1))
        n = len(instances)
        tasks: List[List[BaseTask]] = [[self.task_cls(inst) for _ in range(n_traj)] for inst in instances]
        results: List[List[Optional[AgentResult]]] = [[None] * n_traj for _ in range(n)]
        rewards: List[List[float]] = [[0.0] * n_traj for _ in range(n)]

        async def init(i, t):
            await tasks[i][t].initialize()

        async def run(i, t):
            results[i][t] = await self.agent.run(tasks[i][t].instruction(), session_id=f"inst{i}-traj{t}")

        async def evaluate(i, t):
            try:
                rewards[i][t] = float(await tasks[i][t].evaluate(results[i][t])) if results[i][t] is not None else 0.0
            finally:
                await tasks[i][t].close()

        await self.dispatch(self.cfg, n, n_traj, init, run, evaluate)
        flat = [(results[i][t], rewards[i][t]) for i in range(n) for t in range(n_traj)]
        return {"results": [r for r, _ in flat], "rewards": [w for _, w in flat]}

    @staticmethod
    def to_generator_output(run_out: Dict[str, Any]) -> GeneratorOutput:
        res: List[AgentResult] = run_out["results"]
        have_lp = all(r.logprobs is not None for r in res)
        turns = [r.turns for r in res]
        return {"prompt_token_ids": [r.prompt_ids for r in res], "response_ids": [r.response_ids for r in res],
                "rewards": list(run_out["rewards"]), "loss_masks": [r.loss_mask for r in res],
                "stop_reasons": ["stop" if r.stop_reason == "answer" else "length" for r in res],
                "rollout_logprobs": [r.logprobs for r in res] if have_lp else None,
                "rollout_metrics": {"agent/avg_turns": sum(turns) / max(1, len(turns)),
                                    "agent/answered": sum(r.answer is not None for r in res) / max(1, len(res)),
                                    "agent/avg_reward": sum(run_out["rewards"]) / max(1, len(res))},
                "trajectory_ids": None, "is_last_step": None}  # type: ignore[return-value]


class AgentGenerator(GeneratorInterface):
    """The trainer's generator slot filled by an agent runner: each prompt row's ``env_extras`` is the task instance
    (the question and its gold answer); the trainer has already repeated the prompts ``n_samples_per_prompt`` times,
    so the runner is called with one trajectory per row."""

    def __init__(self, cfg: Dict[str, Any], client, tokenizer, extra_tools: Optional[List[Tool]] = None):
        self.runner = AgentRunner(dict(cfg, num_trajectories=1), client, tokenizer, extra_tools)

    async def generate(self, input_batch: GeneratorInput) -> GeneratorOutput:
        rows = []
        for prompt, extras in zip(input_batch["prompts"], input_batch.get("env_extras") or [{}] * len(input_batch["prompts"])):
            inst = dict(extras or {})
            if "question" not in inst and "prompt" not in inst:
                last = prompt[-1]["content"] if isinstance(prompt, list) and prompt else prompt
                inst["question"] = last if isinstance(last, str) else " ".join(str(t) for t in last)
            rows.append(inst)
        out = self.runner.to_generator_output(await self.runner.run(rows))
        out["trajectory_ids"] = input_batch.get("trajectory_ids")
        return out
