"""Rollout orchestration against Gym-style environments, token-in / token-out.

Behavioural reference: skyrl/train/generators/skyrl_gym_generator.py (``agent_loop`` :280-606,
``generate_batched`` and ``generate`` :811-986, observation tokenisation :646-681, per-token rewards
:608-644).  The bookkeeping is restructured around a ``_Trajectory`` accumulator that owns the token
stream of one episode:

* every model turn appends its generated ids with loss-mask 1 and the engine's log-probabilities;
* every environment observation appends chat-templated ids with loss-mask 0 and log-probability 0;
* each turn's reward is attached to the index of that turn's last generated token;
* on finish the trailing observation is cut, so the response ends on a generated token.

The engine is always given the *token ids accumulated so far* (never re-tokenised text), which keeps
training and sampling on identical token sequences across turns.
"""

from __future__ import annotations

import asyncio
import copy
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple, Union
from uuid import uuid4

from ... import gym as skyrl_gym
from ...inference.base import InferenceEngineInput, InferenceEngineInterface
from .base import GeneratorInput, GeneratorInterface, GeneratorOutput, TrajectoryID
from .utils import get_rollout_metrics
from ...utils.tokenizer import chat_template_ids


@dataclass
class TrajectoryOutput:
    prompt_ids: List[int]
    response_ids: List[int]
    reward: Union[float, List[float]]
    loss_mask: List[int]
    stop_reason: str
    rollout_logprobs: Optional[List[float]]
    env_metrics: Dict[str, Any] = field(default_factory=dict)
    e2e_time: float = 0.0
    time_splits: Dict[str, float] = field(default_factory=dict)
    is_last_step: bool = True
    # experts chosen at rollout time for the tokens of prompt + response, ``[rows <= len, layers, top_k]`` (MoE policies
    # with ``inference_engine.enable_return_routed_experts``); rows past the recorded ones were never routed
    rollout_expert_indices: Optional[Any] = None


class _Trajectory:
    """Token stream of one episode after the initial prompt."""

    def __init__(self, prompt_ids: List[int], track_logprobs: bool):
        self.prompt_ids = list(prompt_ids)
        self.ids: List[int] = []
        self.mask: List[int] = []
        self.logprobs: Optional[List[float]] = [] if track_logprobs else None
        self.turn_rewards: List[Tuple[float, int]] = []  # (reward, index into ids of the turn's last generated token)
        self.last_generated_end = 0  # one past the last generated token

    @property
    def context(self) -> List[int]:
        return self.prompt_ids + self.ids

    def add_model_turn(self, out_ids: List[int], out_logprobs: Optional[List[float]], reward: float,
                       appended_eos: bool = False) -> None:
        n = len(out_ids)
        self.ids.extend(out_ids)
        # an EOS appended by the generator (not sampled) is part of the context but is not trained on
        self.mask.extend([1] * (n - 1) + [0 if appended_eos else 1] if n else [])
        if self.logprobs is not None:
            if out_logprobs is None:
                self.logprobs = None
            else:
                assert len(out_logprobs) == n, f"got {len(out_logprobs)} logprobs for {n} tokens"
                self.logprobs.extend(out_logprobs)
        self.last_generated_end = len(self.ids)
        if n:
            self.turn_rewards.append((float(reward), len(self.ids) - 1))

    def add_observation(self, obs_ids: List[int]) -> None:
        self.ids.extend(obs_ids)
        self.mask.extend([0] * len(obs_ids))
        if self.logprobs is not None:
            self.logprobs.extend([0.0] * len(obs_ids))

    def finalize(self, per_token_reward: bool) -> Tuple[List[int], List[int], Optional[List[float]], Union[float, List[float]]]:
        end = self.last_generated_end
        ids, mask = self.ids[:end], self.mask[:end]
        lps = self.logprobs[:end] if self.logprobs is not None else None
        if per_token_reward:
            rew = [0.0] * end
            for r, idx in self.turn_rewards:
                if idx < end:
                    rew[idx] += r
            return ids, mask, lps, rew
        return ids, mask, lps, float(sum(r for r, _ in self.turn_rewards))


class SkyRLGymGenerator(GeneratorInterface):
    def __init__(self, generator_cfg, skyrl_gym_cfg, inference_engine_client: InferenceEngineInterface, tokenizer,
                 model_name: str = "policy"):
        self.generator_cfg = generator_cfg
        self.skyrl_gym_cfg = skyrl_gym_cfg
        self.client = inference_engine_client
        self.inference_engine_client = inference_engine_client
        self.tokenizer = tokenizer
        self.model_name = model_name
        self.max_turns = generator_cfg.max_turns
        self.batched = generator_cfg.batched
        self.use_conversation_multi_turn = generator_cfg.use_conversation_multi_turn
        n_workers = getattr(skyrl_gym_cfg, "max_env_workers", 32) if skyrl_gym_cfg is not None else 32
        self.env_executor = ThreadPoolExecutor(max_workers=n_workers, thread_name_prefix="env") if n_workers > 0 else None
        self.weight_version_fn = getattr(inference_engine_client, "weight_version", None)
        # a custom chat template (generator.chat_template) switches the multi-turn loop to re-tokenising the whole chat
        # history every turn; the assistant mask then comes from the template's {% generation %} blocks
        from .utils import get_custom_chat_template

        self.custom_chat_template = get_custom_chat_template(getattr(generator_cfg, "chat_template", None))
        if self.batched and self.max_turns > 1:
            raise ValueError("generator.batched=true only supports single-turn rollouts (max_turns=1)")
        # ids of an empty conversation: the prefix that observation tokenisation strips off
        self._base_conv = [{"role": "system", "content": ""}]
        try:
            self._base_ids = chat_template_ids(self.tokenizer, self._base_conv, add_generation_prompt=False)
        except Exception:
            self._base_conv, self._base_ids = [], []
        # What a template writes after the end-of-turn token (ChatML: a newline) belongs in front of the next message:
        # a sampled turn stops at its end-of-turn token, so the observation that follows has to bring those tokens
        # along.  Cutting the base at its last end-of-turn token makes every observation start with them.
        eos = getattr(self.tokenizer, "eos_token_id", None)
        if eos is not None and eos in self._base_ids:
            self._base_ids = self._base_ids[: len(self._base_ids) - self._base_ids[::-1].index(eos)]

    # ------------------------------------------------------------------ helpers
    async def _in_executor(self, fn, *args):
        if self.env_executor is None:
            return fn(*args)
        return await asyncio.get_running_loop().run_in_executor(self.env_executor, fn, *args)

    def _cache_salt(self) -> Optional[str]:
        """Prefix-cache entries must not outlive the weights that produced them."""
        if not getattr(self.generator_cfg, "use_cache_salt", True):
            return None
        v = getattr(self.client, "weight_version", 0)
        return f"{self.model_name}@{v}"

    def _obs_ids(self, observations: List[Dict[str, Any]], done: bool) -> List[int]:
        """Token ids of new observation messages (+ generation prompt unless the episode is over)."""
        if not observations:
            if done or not self.use_conversation_multi_turn:
                return []
            full = chat_template_ids(self.tokenizer, self._base_conv, add_generation_prompt=True)
            return list(full[len(self._base_ids):])
        if not self.use_conversation_multi_turn:
            text = "".join(str(m.get("content", "")) for m in observations)
            return list(self.tokenizer.encode(text, add_special_tokens=False))
        full = chat_template_ids(self.tokenizer, self._base_conv + list(observations), add_generation_prompt=not done,
                                 **self.generator_cfg.chat_template_kwargs)
        return list(full[len(self._base_ids):])

    def _setup_env_extras(self, env_class: str, extras: Dict[str, Any], session_id: str,
                          sampling_params: Optional[Dict[str, Any]]) -> Dict[str, Any]:
        """Hook for subclasses: what the environment's constructor receives (e.g. callables that let the environment
        query the policy itself).  Runs on the event loop, before the environment exists."""
        return extras

    # ------------------------------------------------------------------ one episode
    async def agent_loop(self, prompt, env_class: str, env_extras: Dict[str, Any], max_tokens: int, max_input_length: int,
                         sampling_params: Optional[Dict[str, Any]] = None, trajectory_id: Optional[TrajectoryID] = None,
                         prompt_token_ids: Optional[List[int]] = None) -> Union[TrajectoryOutput, List[TrajectoryOutput]]:
        t0 = time.monotonic()
        splits = {"llm": 0.0, "env": 0.0}
        extras = dict(env_extras or {})
        extras.setdefault("max_turns", self.max_turns)
        env_cfg = getattr(self.skyrl_gym_cfg, env_class, None) if self.skyrl_gym_cfg is not None else None
        session_id = trajectory_id.to_string() if trajectory_id is not None else uuid4().hex
        extras = self._setup_env_extras(env_class, extras, session_id, sampling_params)
        env = skyrl_gym.make(env_class, env_config=env_cfg, extras=extras)
        sp = dict(sampling_params) if sampling_params is not None else self._default_sampling_params()
        sp.setdefault("max_generate_length", max_tokens)
        step_wise = bool(self.generator_cfg.step_wise_trajectories)
        steps: List[TrajectoryOutput] = []
        try:
            chat, _ = await self._in_executor(env.init, prompt)
            if prompt_token_ids is not None:
                ids0 = list(prompt_token_ids)
            else:
                tkw = dict(self.generator_cfg.chat_template_kwargs)
                if self.use_conversation_multi_turn and self.custom_chat_template:
                    tkw["chat_template"] = self.custom_chat_template
                ids0 = chat_template_ids(self.tokenizer, chat, add_generation_prompt=True, **tkw)
            traj = _Trajectory(ids0, track_logprobs=sp.get("logprobs", 1) is not None)
            stop_reason = "stop"
            done = False
            turn = 0
            routes = None
            retokenize = bool(self.use_conversation_multi_turn and self.custom_chat_template)
            if retokenize and step_wise:
                raise ValueError("step_wise_trajectories is not supported with a custom chat template")
            history = [dict(m) for m in chat] if isinstance(chat, list) else []
            n_prompt_msgs = len(history)
            last_obs: List[Dict[str, Any]] = []
            last_reward = 0.0
            eos_text = getattr(self.tokenizer, "eos_token", None)
            while not done:
                if retokenize:
                    ctx = chat_template_ids(self.tokenizer, history, chat_template=self.custom_chat_template,
                                            add_generation_prompt=True, **self.generator_cfg.chat_template_kwargs)
                else:
                    ctx = traj.context
                if len(ctx) > max_input_length:
                    stop_reason = "length"
                    break
                tl = time.monotonic()
                out = await self.client.generate(InferenceEngineInput(prompt_token_ids=[ctx], session_ids=[session_id],
                                                                      sampling_params=sp, cache_salt=self._cache_salt()))
                splits["llm"] += time.monotonic() - tl
                text, out_ids = out["responses"][0], list(out["response_ids"][0])
                stop_reason = out["stop_reasons"][0]
                lps = out.get("response_logprobs")
                lps = list(lps[0]) if lps is not None and lps[0] is not None else None
                # every turn re-submits the whole context, so the latest table covers all earlier turns as well
                turn_routes = (out.get("rollout_expert_indices") or [None])[0]
                if turn_routes is not None and retokenize:
                    raise ValueError("rollout expert indices cannot be kept when a custom chat template re-tokenises the history")
                appended_eos = False
                stops = sp.get("stop")
                if (stops and self.generator_cfg.append_eos_token_after_stop_str_in_multi_turn
                        and self.use_conversation_multi_turn and text.endswith(tuple(stops))
                        and out_ids and out_ids[-1] != self.tokenizer.eos_token_id):
                    out_ids.append(self.tokenizer.eos_token_id)
                    if lps is not None:
                        lps.append(0.0)
                    appended_eos = True
                te = time.monotonic()
                step_out = await self._in_executor(env.step, text)
                splits["env"] += time.monotonic() - te
                done = bool(step_out["done"])
                reward = float(step_out["reward"] or 0.0)
                if step_out.get("postprocessed_action") is not None:
                    text = step_out["postprocessed_action"]
                    out_ids = list(self.tokenizer.encode(text, add_special_tokens=False))
                    lps = None
                    if turn_routes is not None:
                        turn_routes = turn_routes[: len(ctx)]  # the re-tokenised action was not what the model saw
                if retokenize:
                    # the template puts the end-of-turn token back: keep the plain text in the history
                    msg = text[: -len(eos_text)] if eos_text and text.endswith(eos_text) else text
                    last_obs = list(step_out.get("observations") or [])
                    history.append({"role": "assistant", "content": msg})
                    history.extend(last_obs)
                    last_reward = reward
                    turn += 1
                    continue
                obs_ids = self._obs_ids(step_out.get("observations") or [], done)
                if not self.use_conversation_multi_turn and not step_wise and not done:
                    # every turn continues one assistant message: the end-of-sequence token a turn ended on would sit in
                    # the middle of it, so it is dropped.  The last turn keeps its own (with its sampled log-prob); if
                    # it has none, one is appended below.
                    if out_ids and out_ids[-1] == self.tokenizer.eos_token_id:
                        out_ids = out_ids[:-1]
                        lps = lps[: len(out_ids)] if lps is not None else None
                if step_wise:
                    gen_part = len(out_ids)
                    mask = [1] * gen_part + [0] * len(obs_ids)
                    if appended_eos:
                        mask[gen_part - 1] = 0
                    rew = [0.0] * (gen_part + len(obs_ids))
                    if gen_part:
                        rew[gen_part - 1] = reward
                    steps.append(TrajectoryOutput(ctx, out_ids + obs_ids, rew, mask, stop_reason,
                                                  (lps + [0.0] * len(obs_ids)) if lps is not None else None,
                                                  env.get_metrics() if done else {}, is_last_step=False))
                if turn_routes is not None:
                    routes = turn_routes
                traj.add_model_turn(out_ids, lps, reward, appended_eos)
                traj.add_observation(obs_ids)
                turn += 1
                if stop_reason == "length" and not done and len(traj.context) >= max_input_length:
                    break
            env_metrics = env.get_metrics()
            await self._in_executor(env.close)
            if step_wise:
                if steps:
                    steps[-1].is_last_step = True
                    # the last step ends on its generated tokens: drop the trailing observation
                    last = steps[-1]
                    n_gen = max((i + 1 for i, m in enumerate(last.loss_mask) if m), default=len(last.response_ids))
                    last.response_ids, last.loss_mask = last.response_ids[:n_gen], last.loss_mask[:n_gen]
                    last.reward = last.reward[:n_gen]
                    if last.rollout_logprobs is not None:
                        last.rollout_logprobs = last.rollout_logprobs[:n_gen]
                for s in steps:
                    s.e2e_time, s.time_splits = time.monotonic() - t0, splits
                return steps
            if retokenize:
                # response = every message after the prompt except the observations of the last step; the assistant
                # mask comes from the template; one scalar reward (the last step's) and no rollout log-probs, because the
                # tokens trained on are not necessarily the ones that were sampled
                tail = history[n_prompt_msgs : len(history) - len(last_obs)]
                enc = self.tokenizer.apply_chat_template(tail, chat_template=self.custom_chat_template,
                                                         add_generation_prompt=False, return_dict=True,
                                                         return_assistant_tokens_mask=True, tokenize=True,
                                                         **self.generator_cfg.chat_template_kwargs)
                rew_f = 0.0 if (self.generator_cfg.zero_reward_on_non_stop and stop_reason != "stop") else float(last_reward)
                return TrajectoryOutput(ids0, list(enc["input_ids"]), rew_f, [int(x) for x in enc["assistant_masks"]],
                                        stop_reason, None, env_metrics, time.monotonic() - t0, splits)
            per_token = self.max_turns > 1 or len(traj.turn_rewards) > 1
            resp, mask, lps_all, rew = traj.finalize(per_token_reward=per_token)
            if (not self.use_conversation_multi_turn and stop_reason != "length" and resp
                    and resp[-1] != self.tokenizer.eos_token_id):
                resp.append(self.tokenizer.eos_token_id)
                mask.append(1)
                if lps_all is not None:
                    lps_all.append(0.0)
                if isinstance(rew, list) and traj.turn_rewards:
                    # the last turn's reward moves from its last sampled token onto the token that now ends the response
                    r_last, idx = traj.turn_rewards[-1]
                    rew = rew + [0.0]
                    if idx < len(rew) - 1:
                        rew[idx] -= r_last
                        rew[-1] += r_last
            if self.generator_cfg.zero_reward_on_non_stop and stop_reason != "stop":
                rew = [0.0] * len(rew) if isinstance(rew, list) else 0.0
            return TrajectoryOutput(traj.prompt_ids, resp, rew, mask, stop_reason, lps_all, env_metrics,
                                    time.monotonic() - t0, splits, rollout_expert_indices=routes)
        finally:
            await self.client.finish_session(session_id)

    def _default_sampling_params(self) -> Dict[str, Any]:
        sp = self.generator_cfg.sampling_params
        d = sp.to_dict() if hasattr(sp, "to_dict") else dict(sp)
        return d

    # ------------------------------------------------------------------ batched single-turn
    async def generate_batched(self, prompts, env_classes, env_extras, max_tokens: int, max_input_length: int,
                               sampling_params: Optional[Dict[str, Any]], prompt_token_ids=None) -> List[TrajectoryOutput]:
        envs, ids = [], []
        for i, (p, cls, ex) in enumerate(zip(prompts, env_classes, env_extras)):
            env_cfg = getattr(self.skyrl_gym_cfg, cls, None) if self.skyrl_gym_cfg is not None else None
            env = skyrl_gym.make(cls, env_config=env_cfg, extras=dict(ex or {}))
            chat, _ = env.init(p)
            envs.append(env)
            if prompt_token_ids is not None:
                ids.append(list(prompt_token_ids[i]))
            else:
                ids.append(chat_template_ids(self.tokenizer, chat, add_generation_prompt=True,
                                             **self.generator_cfg.chat_template_kwargs))
        sp = dict(sampling_params) if sampling_params is not None else self._default_sampling_params()
        sp.setdefault("max_generate_length", max_tokens)
        per_req = [e.get("sampling_params") for e in (env_extras or [])] if env_extras else None
        t0 = time.monotonic()
        if hasattr(self.client, "generate_sync") and not getattr(self, "_force_async", False):
            if per_req and any(per_req):
                sps = [{**sp, **(o or {})} for o in per_req]
                out = await asyncio.to_thread(self.client.generate_sync, ids, sps, self._cache_salt())
            else:
                out = await asyncio.to_thread(self.client.generate_sync, ids, sp, self._cache_salt())
        else:
            out = await self.client.generate(InferenceEngineInput(prompt_token_ids=ids, sampling_params=sp,
                                                                  cache_salt=self._cache_salt()))
        llm_t = time.monotonic() - t0
        res = []
        lps_all = out.get("response_logprobs")
        routes_all = out.get("rollout_expert_indices")
        for i, env in enumerate(envs):
            step_out = env.step(out["responses"][i])
            resp = list(out["response_ids"][i])
            reward = float(step_out["reward"] or 0.0)
            stop = out["stop_reasons"][i]
            if self.generator_cfg.zero_reward_on_non_stop and stop != "stop":
                reward = 0.0
            res.append(TrajectoryOutput(ids[i], resp, reward, [1] * len(resp), stop,
                                        list(lps_all[i]) if lps_all is not None and lps_all[i] is not None else None,
                                        env.get_metrics(), llm_t, {"llm": llm_t, "env": 0.0},
                                        rollout_expert_indices=routes_all[i] if routes_all is not None else None))
            env.close()
        return res

    # ------------------------------------------------------------------ batch API
    async def generate(self, input_batch: GeneratorInput) -> GeneratorOutput:
        prompts = input_batch["prompts"]
        env_classes = input_batch["env_classes"]
        env_extras = input_batch.get("env_extras") or [{} for _ in prompts]
        traj_ids = input_batch.get("trajectory_ids")
        sampling_params = input_batch.get("sampling_params")
        pre_ids = input_batch.get("prompt_token_ids")
        sp_cfg = self.generator_cfg.sampling_params
        max_tokens = (sampling_params or {}).get("max_generate_length", sp_cfg.max_generate_length)
        max_input_length = self.generator_cfg.max_input_length
        if self.batched:
            outs: List[Any] = await self.generate_batched(prompts, env_classes, env_extras, max_tokens, max_input_length,
                                                          sampling_params, pre_ids)
        else:
            tasks = [self.agent_loop(prompts[i], env_classes[i], env_extras[i], max_tokens, max_input_length,
                                     sampling_params, traj_ids[i] if traj_ids else None,
                                     pre_ids[i] if pre_ids is not None else None) for i in range(len(prompts))]
            outs = await asyncio.gather(*tasks)
        flat: List[TrajectoryOutput] = []
        out_traj_ids: Optional[List[TrajectoryID]] = [] if traj_ids else None
        for i, o in enumerate(outs):
            items = o if isinstance(o, list) else [o]
            flat.extend(items)
            if out_traj_ids is not None:
                out_traj_ids.extend([traj_ids[i]] * len(items))
        responses = [t.response_ids for t in flat]
        rewards = [t.reward for t in flat]
        masks = [t.loss_mask for t in flat]
        stops = [t.stop_reason for t in flat]
        if self.generator_cfg.apply_overlong_filtering:
            # truncated responses (no EOS) contribute no gradient
            eos = self.tokenizer.eos_token_id
            masks = [[0] * len(m) if (not r or r[-1] != eos) else m for m, r in zip(masks, responses)]
        has_lp = all(t.rollout_logprobs is not None for t in flat) and len(flat) > 0
        # one environment class per row (step-wise rollouts have several rows per trajectory)
        flat_classes = [env_classes[i] for i, o in enumerate(outs) for _ in (o if isinstance(o, list) else [o])]
        metrics = get_rollout_metrics(responses, rewards, [t.env_metrics for t in flat], env_classes=flat_classes, loss_masks=masks,
                                      trajectory_completion_times=[t.e2e_time for t in flat],
                                      trajectory_time_splits={"llm": [t.time_splits.get("llm", 0.0) for t in flat],
                                                              "env": [t.time_splits.get("env", 0.0) for t in flat]})
        return GeneratorOutput(
            prompt_token_ids=[t.prompt_ids for t in flat], response_ids=responses, rewards=rewards, loss_masks=masks,
            stop_reasons=stops, rollout_metrics=metrics,
            rollout_logprobs=[t.rollout_logprobs for t in flat] if has_lp else None, trajectory_ids=out_traj_ids,
            trajectory_generation_times=[t.e2e_time for t in flat],
            trajectory_time_splits={"llm": [t.time_splits.get("llm", 0.0) for t in flat],
                                    "env": [t.time_splits.get("env", 0.0) for t in flat]},
            rollout_expert_indices=([t.rollout_expert_indices for t in flat]
                                    if any(t.rollout_expert_indices is not None for t in flat) else None),
            is_last_step=[t.is_last_step for t in flat] if self.generator_cfg.step_wise_trajectories else None,
            env_metrics=[t.env_metrics for t in flat], pixel_values=None, image_grid_thw=None)
