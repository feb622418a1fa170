"""Rollout helpers: metrics over a generated batch, pass@n, prompt repetition with trajectory ids,
and merging of step-wise outputs (reference: skyrl/train/generators/utils.py:184-961)."""

from __future__ import annotations

from collections import defaultdict
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from .base import BatchMetadata, GeneratorInput, GeneratorOutput, TrajectoryID


def _traj_reward(r) -> float:
    return float(sum(r)) if isinstance(r, (list, tuple)) else float(r)


def get_rollout_metrics(responses: Sequence[Sequence[int]], rewards: Sequence[Union[float, Sequence[float]]],
                        env_metrics: Optional[Sequence[Dict[str, Any]]] = None,
                        env_classes: Optional[Sequence[str]] = None) -> Dict[str, float]:
    lens = np.array([len(r) for r in responses], dtype=np.float64) if len(responses) else np.zeros(1)
    scores = np.array([_traj_reward(r) for r in rewards], dtype=np.float64) if len(rewards) else np.zeros(1)
    pos, nonpos = lens[scores > 0], lens[scores <= 0]
    m = {
        "generate/min_num_tokens": float(lens.min()), "generate/max_num_tokens": float(lens.max()),
        "generate/avg_num_tokens": float(lens.mean()), "generate/std_num_tokens": float(lens.std()),
        "generate/avg_tokens_non_zero_rewards": float(pos.mean()) if len(pos) else 0.0,
        "generate/avg_tokens_zero_rewards": float(nonpos.mean()) if len(nonpos) else 0.0,
    }  # fmt: skip
    if env_metrics:
        agg: Dict[str, List[float]] = defaultdict(list)
        for em in env_metrics:
            for k, v in (em or {}).items():
                if isinstance(v, (int, float, bool)):
                    agg[k].append(float(v))
        for k, v in agg.items():
            m[f"environment/{k}"] = float(np.mean(v))
    return m


def compute_pass_at_n(rewards: Sequence[Union[float, Sequence[float]]], uids: Sequence[str]) -> float:
    """Fraction of prompts with at least one trajectory of positive total reward."""
    best: Dict[str, float] = {}
    for r, u in zip(rewards, uids):
        best[u] = max(best.get(u, float("-inf")), _traj_reward(r))
    return float(np.mean([1.0 if v > 0 else 0.0 for v in best.values()])) if best else 0.0


def get_metrics_from_generator_output(out: GeneratorOutput, uids: Sequence[str]) -> Dict[str, float]:
    rewards = out["rewards"]
    scores = [_traj_reward(r) for r in rewards]
    pos = [s for s in scores if s > 0]
    return {"avg_score": float(np.mean(scores)) if scores else 0.0, "pass_at_n": compute_pass_at_n(rewards, uids),
            "mean_positive_reward": float(np.mean(pos)) if pos else 0.0}


def prepare_generator_input(prompts: List[Any], n_samples_per_prompt: int, sampling_params: Optional[Dict[str, Any]],
                            default_env_class: str, training_phase: str, global_step: int,
                            prompt_token_ids: Optional[List[List[int]]] = None) -> Tuple[GeneratorInput, List[str]]:
    """Repeat every prompt ``n`` times; returns the generator input and the per-trajectory prompt uids.

    Each dataset item is ``{"prompt": conversation, "env_class": str?, "env_extras": dict?, "uid": str}``.
    """
    convs, classes, extras, tids, uids, pre = [], [], [], [], [], []
    for k, item in enumerate(prompts):
        uid = str(item.get("uid", k))
        for rep in range(n_samples_per_prompt):
            convs.append(item["prompt"])
            classes.append(item.get("env_class") or default_env_class)
            ex = dict(item.get("env_extras") or {})
            ex.setdefault("repetition_id", rep)
            extras.append(ex)
            tids.append(TrajectoryID(uid, rep))
            uids.append(uid)
            if prompt_token_ids is not None:
                pre.append(prompt_token_ids[k])
            elif item.get("prompt_token_ids") is not None:
                pre.append(item["prompt_token_ids"])
    gi = GeneratorInput(prompts=convs, env_classes=classes, env_extras=extras, sampling_params=sampling_params,
                        trajectory_ids=tids, batch_metadata=BatchMetadata(global_step, training_phase),
                        prompt_token_ids=pre if pre else None)
    return gi, uids


def concatenate_generator_outputs(outputs: List[GeneratorOutput]) -> GeneratorOutput:
    """Row-wise concatenation of several generator outputs (dynamic sampling, eval chunks)."""
    first = outputs[0]
    res = GeneratorOutput()
    for key in ("prompt_token_ids", "response_ids", "rewards", "loss_masks", "stop_reasons", "rollout_logprobs",
                "trajectory_ids", "is_last_step", "env_metrics", "trajectory_generation_times"):
        vals = [o.get(key) for o in outputs]
        if any(v is None for v in vals):
            res[key] = None
        else:
            res[key] = [x for v in vals for x in v]
    res["rollout_metrics"] = get_rollout_metrics(res["response_ids"], res["rewards"], res.get("env_metrics"))
    res["rollout_expert_indices"] = None
    res["pixel_values"] = res["image_grid_thw"] = None
    res["trajectory_time_splits"] = first.get("trajectory_time_splits")
    return res


def merge_stepwise_output(out: GeneratorOutput) -> GeneratorOutput:
    """Merge consecutive steps of one trajectory when each step's prompt extends the previous step's tokens.

    Step k+1 can be folded into step k when ``prompt_{k+1}`` starts with ``prompt_k + response_k``; the tokens in
    between (environment text added by the agent scaffold) become masked response tokens.  Steps whose context was
    rewritten stay separate rows.
    """
    tids = out.get("trajectory_ids")
    if not tids or out.get("is_last_step") is None:
        return out
    rows: List[Dict[str, Any]] = []
    cur: Optional[Dict[str, Any]] = None
    n = len(out["response_ids"])
    for i in range(n):
        p, r = list(out["prompt_token_ids"][i]), list(out["response_ids"][i])
        rew = out["rewards"][i]
        rew = list(rew) if isinstance(rew, (list, tuple)) else [0.0] * (len(r) - 1) + [float(rew)] if r else []
        m = list(out["loss_masks"][i])
        lp = list(out["rollout_logprobs"][i]) if out.get("rollout_logprobs") else None
        same = cur is not None and cur["tid"] == tids[i].to_string()
        full_prev = cur["prompt"] + cur["resp"] if cur is not None else None
        if same and p[: len(full_prev)] == full_prev:
            gap = p[len(full_prev):]
            cur["resp"] += gap + r
            cur["mask"] += [0] * len(gap) + m
            cur["rew"] += [0.0] * len(gap) + rew
            if cur["lp"] is not None and lp is not None:
                cur["lp"] += [0.0] * len(gap) + lp
            else:
                cur["lp"] = None
            cur["stop"] = out["stop_reasons"][i]
            cur["last"] = out["is_last_step"][i]
        else:
            if cur is not None:
                rows.append(cur)
            cur = {"tid": tids[i].to_string(), "tid_obj": tids[i], "prompt": p, "resp": r, "mask": m, "rew": rew, "lp": lp,
                   "stop": out["stop_reasons"][i], "last": out["is_last_step"][i]}
        if out["is_last_step"][i]:
            rows.append(cur)
            cur = None
    if cur is not None:
        rows.append(cur)
    merged = GeneratorOutput(
        prompt_token_ids=[x["prompt"] for x in rows], response_ids=[x["resp"] for x in rows],
        rewards=[x["rew"] for x in rows], loss_masks=[x["mask"] for x in rows], stop_reasons=[x["stop"] for x in rows],
        rollout_logprobs=[x["lp"] for x in rows] if all(x["lp"] is not None for x in rows) else None,
        trajectory_ids=[x["tid_obj"] for x in rows], is_last_step=[x["last"] for x in rows],
        rollout_metrics=out.get("rollout_metrics"), rollout_expert_indices=None, env_metrics=None,
        trajectory_generation_times=None, trajectory_time_splits=None, pixel_values=None, image_grid_thw=None)
    return merged
