"""Generator for REPL-driven "recursive language model" environments: besides driving the episode, it gives the
environment two callables so that the code the policy writes can query the policy.

* ``lm_callback(prompts) -> answers``: plain generations for ``llm_query`` / ``llm_query_batched`` -- one chat turn per
  prompt through the same inference client (or through ``frozen_client`` when the sub-calls should not come from the
  policy being trained).
* ``subcall_fn(prompt) -> answer``: a *child episode* of the same environment class for ``rlm_query`` /
  ``rlm_query_batched``: own REPL, the prompt as its question and as its context, the parent's turn budget, depth + 1;
  its ``FINAL`` answer is the return value.  Children deeper than ``max_depth`` fall back to a plain generation.  Child
  trajectories are not trained on: they appear in the parent's trajectory only through what the REPL printed.

Environment steps run in the generator's thread pool, so the callables block their worker thread while the coroutine
they scheduled runs on the event loop.  Reference: examples/train/rlm/rlm_generator.py (``RLMGymGenerator``; there the
children's trajectories also join the batch).
"""

from __future__ import annotations

import asyncio
import contextvars
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Dict, List, Optional

from ...inference.base import InferenceEngineInput
from .skyrl_gym_generator import SkyRLGymGenerator


_DEPTH = contextvars.ContextVar("rlm_depth", default=0)


class RLMGenerator(SkyRLGymGenerator):
    RLM_ENV_CLASSES = ("rlm",)

    def __init__(self, *args, max_depth: int = 1, frozen_client=None, subcall_max_tokens: Optional[int] = None, **kwargs):
        super().__init__(*args, **kwargs)
        if self.env_executor is None:
            raise ValueError("RLMGenerator needs environment worker threads (skyrl_gym.max_env_workers > 0): the "
                             "environment's callbacks block while the event loop serves them")
        self.max_depth, self.frozen_client, self.subcall_max_tokens = max_depth, frozen_client, subcall_max_tokens
        self.subcall_stats = {"lm_queries": 0, "child_episodes": 0}
        # a parent's environment step blocks its worker thread until its children are done, so every depth gets its own
        # pool: children can always find a free thread however many parents are waiting
        self._pools: Dict[int, ThreadPoolExecutor] = {0: self.env_executor}

    async def _in_executor(self, fn, *args):
        d = _DEPTH.get()
        if d not in self._pools:
            self._pools[d] = ThreadPoolExecutor(max_workers=self.env_executor._max_workers, thread_name_prefix=f"env-d{d}")
        return await asyncio.get_running_loop().run_in_executor(self._pools[d], fn, *args)

    # ------------------------------------------------------------------ callables handed to the environment
    def _setup_env_extras(self, env_class, extras, session_id, sampling_params):
        if env_class not in self.RLM_ENV_CLASSES:
            return extras
        loop = asyncio.get_running_loop()
        depth = int(extras.get("depth", 0))
        extras = dict(extras)
        extras["lm_callback"] = self._make_lm_callback(loop, sampling_params, session_id)
        extras["subcall_fn"] = self._make_subcall_fn(loop, env_class, extras, sampling_params, depth, session_id)
        return extras

    async def _answer(self, prompts: List[str], sampling_params: Optional[Dict[str, Any]], session_id: str) -> List[str]:
        from ...utils.tokenizer import chat_template_ids

        client = self.frozen_client or self.client
        sp = dict(sampling_params) if sampling_params is not None else self._default_sampling_params()
        if self.subcall_max_tokens:
            sp["max_generate_length"] = self.subcall_max_tokens
        ids = [chat_template_ids(self.tokenizer, [{"role": "user", "content": p}], add_generation_prompt=True,
                                 **self.generator_cfg.chat_template_kwargs) for p in prompts]
        out = await client.generate(InferenceEngineInput(prompt_token_ids=ids, sampling_params=sp,
                                                         session_ids=[f"{session_id}/q{i}" for i in range(len(ids))],
                                                         cache_salt=self._cache_salt()))
        self.subcall_stats["lm_queries"] += len(prompts)
        return [str(r) for r in out["responses"]]

    def _make_lm_callback(self, loop, sampling_params, session_id):
        def callback(prompts: List[str]) -> List[str]:
            return asyncio.run_coroutine_threadsafe(self._answer(list(prompts), sampling_params, session_id), loop).result()

        return callback

    def _make_subcall_fn(self, loop, env_class, parent_extras, sampling_params, depth, session_id):
        async def child(prompt: str) -> str:
            if depth + 1 > self.max_depth:
                return (await self._answer([prompt], sampling_params, session_id))[0]
            self.subcall_stats["child_episodes"] += 1
            _DEPTH.set(depth + 1)  # this coroutine is its own task: the setting stays inside the child episode
            extras = {k: v for k, v in parent_extras.items() if k not in ("lm_callback", "subcall_fn", "context", "extra_info")}
            extras.update({"depth": depth + 1, "context": prompt, "root_prompt": prompt,
                           # a child is judged by nobody: any final answer ends it
                           "reward_spec": {"ground_truth": "", "method": "contains"}})
            sp = dict(sampling_params) if sampling_params is not None else self._default_sampling_params()
            out = await self.agent_loop([{"role": "user", "content": prompt}], env_class, extras,
                                        sp.get("max_generate_length", self.generator_cfg.sampling_params.max_generate_length),
                                        self.generator_cfg.max_input_length, sampling_params)
            last = out[-1] if isinstance(out, list) else out
            final = (last.env_metrics or {}).get("final_answer")
            return str(final) if final is not None else self.tokenizer.decode(last.response_ids, skip_special_tokens=True)

        def subcall_fn(prompt: str, context=None) -> str:
            return asyncio.run_coroutine_threadsafe(child(str(prompt)), loop).result()

        return subcall_fn
