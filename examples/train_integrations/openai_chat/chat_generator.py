"""A generator for agent scaffolds that only speak the OpenAI chat protocol.

The reference's integrations (Verifiers, Harbor, OpenEnv, mini-SWE-agent: examples/train_integrations/*) all have this
shape: a third-party loop drives the policy through ``{endpoint}/v1/chat/completions`` and the adapter turns what came
back into token ids, loss masks and rollout log-probs.  None of those packages is needed here; the loop below is the
SkyRL-Gym environment protocol (``init`` / ``step``), driven through HTTP instead of through the engine client, which
makes it a template for any such adapter:

* the endpoint is ``inference_engine_client.get_endpoint_url()`` -- a server thread in front of the colocated engines,
  or the router of stand-alone servers;
* every response carries ``prompt_token_ids`` and the choice's ``token_ids`` / ``logprobs``, so the trajectory is built
  from the tokens the engine actually saw and sampled (no re-tokenisation of assistant text);
* when a turn's prompt does not extend the previous turn's tokens (a scaffold that rewrites history), the adapter
  falls back to encoding the messages one by one (``get_response_ids_and_loss_mask_from_messages``) and gives up the
  rollout log-probs for that trajectory.
"""

import asyncio
from typing import Any, Dict, List, Optional

import aiohttp

from skyrl_b200 import gym as skyrl_gym
from skyrl_b200.train.generators.base import GeneratorInput, GeneratorInterface, GeneratorOutput
from skyrl_b200.train.generators.utils import get_response_ids_and_loss_mask_from_messages, get_rollout_metrics


class ChatCompletionsGenerator(GeneratorInterface):
    def __init__(self, generator_cfg, skyrl_gym_cfg, inference_engine_client, tokenizer, model_name: str = "policy",
                 max_concurrency: int = 64):
        self.cfg, self.gym_cfg, self.tokenizer, self.model_name = generator_cfg, skyrl_gym_cfg, tokenizer, model_name
        self.client = inference_engine_client
        self.base_url = inference_engine_client.get_endpoint_url().rstrip("/") + "/v1"
        self.max_concurrency = max_concurrency

    async def _chat(self, http: aiohttp.ClientSession, messages: List[Dict[str, Any]], sp: Dict[str, Any], session: str):
        body = {"model": self.model_name, "messages": messages, "logprobs": True,
                "max_tokens": sp.get("max_generate_length", self.cfg.sampling_params.max_generate_length)}
        for k in ("temperature", "top_p", "top_k", "min_p", "stop"):
            if sp.get(k) is not None:
                body[k] = sp[k]
        async with http.post(self.base_url + "/chat/completions", json=body, headers={"X-Session-ID": session}) as r:
            r.raise_for_status()
            return await r.json()

    async def _episode(self, http, sem, prompt, env_class: str, extras: Dict[str, Any], sp: Dict[str, Any], session: str):
        env_cfg = getattr(self.gym_cfg, env_class, None) if self.gym_cfg is not None else None
        extras = dict(extras or {})
        extras.setdefault("max_turns", self.cfg.max_turns)
        env = skyrl_gym.make(env_class, env_config=env_cfg, extras=extras)
        messages, _ = env.init(prompt)
        messages = [dict(m) for m in messages]
        first_prompt: Optional[List[int]] = None
        ids: List[int] = []       # everything after the first prompt
        mask: List[int] = []
        lps: Optional[List[float]] = []
        rewards: List[tuple] = []  # (reward, index of the turn's last sampled token in ids)
        new_messages: List[Dict[str, Any]] = []
        stop, done, consistent = "stop", False, True
        max_len = self.cfg.max_input_length + self.cfg.sampling_params.max_generate_length
        while not done:
            async with sem:
                r = await self._chat(http, messages, sp, session)
            c = r["choices"][0]
            p_ids, t_ids = list(r["prompt_token_ids"]), list(c["token_ids"])
            stop = c["finish_reason"]
            if first_prompt is None:
                first_prompt = p_ids
            sofar = first_prompt + ids
            if consistent and p_ids[: len(sofar)] == sofar:
                gap = p_ids[len(sofar):]   # what the template put between the last turn and this one (observations)
                ids += gap + t_ids
                mask += [0] * len(gap) + [1] * len(t_ids)
                if lps is not None:
                    lp = c.get("logprobs")
                    lps = lps + [0.0] * len(gap) + [x["logprob"] for x in lp["content"]] if lp else None
            else:
                consistent = False
            text = c["message"]["content"]
            out = env.step(text)
            done = bool(out["done"])
            messages.append({"role": "assistant", "content": text})
            new_messages.append({"role": "assistant", "content": text})
            rewards.append((float(out["reward"] or 0.0), len(ids) - 1))
            obs = list(out.get("observations") or [])
            messages += obs
            if not done:
                new_messages += obs
            if len(first_prompt) + len(ids) >= max_len:
                stop = "length"
                break
        metrics = env.get_metrics()
        env.close()
        if not consistent:
            ids, mask, _ = get_response_ids_and_loss_mask_from_messages(new_messages, self.tokenizer)
            lps = None
            rew: Any = float(sum(r for r, _ in rewards))
        else:
            rew = [0.0] * len(ids)
            for r, i in rewards:
                if 0 <= i < len(rew):
                    rew[i] += r
        return {"prompt": first_prompt, "ids": ids, "mask": mask, "lps": lps, "reward": rew, "stop": stop, "metrics": metrics}

    async def generate(self, input_batch: GeneratorInput) -> GeneratorOutput:
        prompts, classes = input_batch["prompts"], input_batch["env_classes"]
        extras = input_batch.get("env_extras") or [{} for _ in prompts]
        tids = input_batch.get("trajectory_ids")
        sp = dict(input_batch.get("sampling_params") or self.cfg.sampling_params.to_dict())
        sem = asyncio.Semaphore(self.max_concurrency)
        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None)) as http:
            eps = await asyncio.gather(*[
                self._episode(http, sem, prompts[i], classes[i], extras[i], sp, tids[i].to_string() if tids else f"ep-{i}")
                for i in range(len(prompts))])
        responses, rewards = [e["ids"] for e in eps], [e["reward"] for e in eps]
        if any(isinstance(r, list) for r in rewards):  # one trajectory fell back to a scalar: spread it like the others
            rewards = [r if isinstance(r, list) else [0.0] * (len(e["ids"]) - 1) + [r] for r, e in zip(rewards, eps)]
        has_lp = all(e["lps"] is not None for e in eps)
        return GeneratorOutput(prompt_token_ids=[e["prompt"] for e in eps], response_ids=responses, rewards=rewards,
                               loss_masks=[e["mask"] for e in eps], stop_reasons=[e["stop"] for e in eps],
                               rollout_metrics=get_rollout_metrics(responses, rewards, [e["metrics"] for e in eps]),
                               rollout_logprobs=[e["lps"] for e in eps] if has_lp else None, trajectory_ids=tids,
                               rollout_expert_indices=None, is_last_step=None, env_metrics=[e["metrics"] for e in eps],
                               trajectory_generation_times=None, trajectory_time_splits=None, pixel_values=None,
                               image_grid_thw=None)
