"""Rollout helpers: metrics over a generated batch, pass@n, prompt repetition with trajectory ids,
and merging of step-wise outputs (reference: skyrl/train/generators/utils.py:184-961)."""

from __future__ import annotations

from collections import defaultdict
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from .base import BatchMetadata, GeneratorInput, GeneratorOutput, TrajectoryID
from ...utils.tokenizer import chat_template_ids


def _traj_reward(r) -> float:
    return float(sum(r)) if isinstance(r, (list, tuple)) else float(r)


def _aggregate_env_metrics(env_class: Optional[str], rows: List[Dict[str, Any]]) -> Dict[str, float]:
    """The environment class's own ``aggregate_metrics`` when the class is registered (an environment may want a sum or
    a maximum rather than a mean); the mean of every numeric entry otherwise."""
    if env_class is not None:
        try:
            from ...gym.registration import _load, registry

            spec = registry.get(env_class)
            agg = getattr(_load(spec.entry_point), "aggregate_metrics", None) if spec is not None else None
            if agg is not None:
                out = agg(rows)
                if out:
                    return {k: float(v) for k, v in out.items() if isinstance(v, (int, float, bool))}
        except Exception:  # noqa: BLE001 - metrics must never break a rollout
            pass
    acc: Dict[str, List[float]] = defaultdict(list)
    for em in rows:
        for k, v in em.items():
            if isinstance(v, (int, float, bool)):
                acc[k].append(float(v))
    return {k: float(np.mean(v)) for k, v in acc.items()}


def _time_stats(m: Dict[str, float], name: str, times) -> None:
    if times is None or len(times) == 0:
        return
    a = np.asarray(times, dtype=np.float64)
    m[f"generate/trajectory_time_{name}_mean"] = float(a.mean())
    m[f"generate/trajectory_time_{name}_p90"] = float(np.percentile(a, 90))
    m[f"generate/trajectory_time_{name}_max"] = float(a.max())


def get_rollout_metrics(responses: Sequence[Sequence[int]], rewards: Sequence[Union[float, Sequence[float]]],
                        env_metrics: Optional[Sequence[Dict[str, Any]]] = None,
                        env_classes: Optional[Sequence[str]] = None, loss_masks: Optional[Sequence[Sequence[int]]] = None,
                        trajectory_completion_times: Optional[Sequence[float]] = None,
                        trajectory_time_splits: Optional[Dict[str, Sequence[float]]] = None) -> Dict[str, float]:
    """Token statistics of a rollout batch (all tokens; with ``loss_masks`` also the model-generated ones and the
    lengths of the individual turns = runs of trained tokens), trajectory time statistics (mean / p90 / max of the
    end-to-end times, of every named split, and of the remainder ``other``), and the environments' own numeric
    metrics under ``environment/<name>``, aggregated per environment class by the class's own ``aggregate_metrics``
    when ``env_classes`` is given and averaged otherwise (reference: generators/utils.py:411-508, same metric names)."""
    lens = np.array([len(r) for r in responses], dtype=np.float64) if len(responses) else np.zeros(1)
    scores = np.array([_traj_reward(r) for r in rewards], dtype=np.float64) if len(rewards) else np.zeros(1)
    pos, zero = lens[scores > 0], lens[scores == 0]
    m = {
        "generate/min_num_tokens": float(lens.min()), "generate/max_num_tokens": float(lens.max()),
        "generate/avg_num_tokens": float(lens.mean()), "generate/std_num_tokens": float(lens.std()),
        "generate/avg_tokens_non_zero_rewards": float(pos.mean()) if len(pos) else 0.0,
        "generate/avg_tokens_zero_rewards": float(zero.mean()) if len(zero) else 0.0,
    }  # fmt: skip
    if loss_masks is not None and len(loss_masks):
        own = np.array([sum(1 for x in mk if x) for mk in loss_masks], dtype=np.float64)
        m.update({"generate/avg_assistant_tokens": float(own.mean()), "generate/min_assistant_tokens": float(own.min()),
                  "generate/max_assistant_tokens": float(own.max()), "generate/std_assistant_tokens": float(own.std())})
        turns = compute_turn_token_counts([list(mk) for mk in loss_masks])
        if turns:
            t = np.array(turns, dtype=np.float64)
            m.update({"generate/tokens_per_turn_mean": float(t.mean()), "generate/tokens_per_turn_std": float(t.std()),
                      "generate/tokens_per_turn_max": float(t.max())})
    _time_stats(m, "completion", trajectory_completion_times)
    for name, times in (trajectory_time_splits or {}).items():
        _time_stats(m, name, times)
    n_t = len(trajectory_completion_times) if trajectory_completion_times is not None else 0
    if n_t and trajectory_time_splits and all(len(v) == n_t for v in trajectory_time_splits.values()):
        other = np.asarray(trajectory_completion_times, dtype=np.float64).copy()
        for times in trajectory_time_splits.values():
            other -= np.asarray(times, dtype=np.float64)  # what no split accounts for: templating, tokenisation, queueing
        _time_stats(m, "other", other)
    if env_metrics:
        by_class: Dict[Optional[str], List[Dict[str, Any]]] = defaultdict(list)
        for i, em in enumerate(env_metrics):
            by_class[env_classes[i] if env_classes is not None and i < len(env_classes) else None].append(em or {})
        for cls, rows in by_class.items():
            for k, v in _aggregate_env_metrics(cls, rows).items():
                m[f"environment/{k}"] = v
    return m


def _outcome(r) -> float:
    """What decides whether a trajectory "passed": its scalar reward, or the reward on its last token (the outcome
    reward of a token-level list; earlier entries are shaping terms)."""
    if isinstance(r, (list, tuple)):
        if not len(r):
            raise ValueError("token-level rewards must be non-empty lists")
        return float(r[-1])
    return float(r)


def compute_pass_at_n(rewards: Sequence[Union[float, Sequence[float]]], uids: Sequence[str]) -> float:
    """Fraction of prompts with at least one trajectory whose outcome reward is positive."""
    best: Dict[str, float] = {}
    for r, u in zip(rewards, uids):
        best[u] = max(best.get(u, float("-inf")), _outcome(r))
    return float(np.mean([1.0 if v > 0 else 0.0 for v in best.values()])) if best else 0.0


def get_metrics_from_generator_output(out: GeneratorOutput, uids: Sequence[str]) -> Dict[str, float]:
    """``avg_score``: mean total reward per trajectory; ``pass_at_n``: see ``compute_pass_at_n``;
    ``mean_positive_reward``: mean over *all* trajectories of their positive reward mass (``max(r, 0)``, summed over
    tokens for token-level rewards).  Definitions of the reference (generators/utils.py:184-232)."""
    rewards = out["rewards"]
    if not len(rewards):
        raise ValueError("`rewards` must be a non-empty list")
    scores = [_traj_reward(r) for r in rewards]
    pos = [float(sum(max(float(x), 0.0) for x in r)) if isinstance(r, (list, tuple)) else max(float(r), 0.0) for r in rewards]
    return {"avg_score": float(np.mean(scores)), "pass_at_n": compute_pass_at_n(rewards, uids),
            "mean_positive_reward": float(np.mean(pos))}


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
    # per-component times: lists are joined per name; a chunk without them makes the whole field None
    splits = [o.get("trajectory_time_splits") for o in outputs]
    if any(sp is None for sp in splits):
        res["trajectory_time_splits"] = None
    else:
        names = list(splits[0])
        res["trajectory_time_splits"] = {k: [x for sp in splits for x in sp.get(k, [])] for k in names}
    routes = [o.get("rollout_expert_indices") for o in outputs]
    res["rollout_expert_indices"] = None if any(r is None for r in routes) else [x for r in routes for x in r]
    # aggregates are recomputed over the joined rows, never combined from the chunks' aggregates
    res["rollout_metrics"] = get_rollout_metrics(res["response_ids"], res["rewards"], res.get("env_metrics"),
                                                 loss_masks=res.get("loss_masks"),
                                                 trajectory_completion_times=res.get("trajectory_generation_times"),
                                                 trajectory_time_splits=res.get("trajectory_time_splits"))
    res["pixel_values"] = res["image_grid_thw"] = None
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


# ----------------------------------------------------------------------------- utilities for custom generators
# What a hand-written generator (an agent loop that talks to the engine through chat messages) needs in order to hand
# the trainer token ids, loss masks and rollout log-probs that are consistent with what the model saw.  Behavioural
# reference: skyrl/train/generators/utils.py:105-182 (chat templates, generation prompt), :349-395 (overlong
# filtering, turn counts), :567-774 (message encoding with a fixed base conversation), :783-804 (slicing).

# ChatML without the "You are a helpful assistant" default that some tokenizers insert when no system message is given:
# what a multi-turn rollout wants, because the conversation is tokenised piece by piece.
def _chatml(assistant_body: str) -> str:
    """ChatML template text.  ``assistant_body`` renders an assistant message's content; it sits, with the end-of-turn
    token, inside a ``generation`` block, so that ``apply_chat_template(..., return_assistant_tokens_mask=True)`` marks
    exactly the tokens the model produced (not the role header, not the newline after the end-of-turn token)."""
    return ("{%- for message in messages -%}"
            "{{- '<|im_start|>' + message['role'] + '\n' -}}"
            "{%- if message['role'] == 'assistant' -%}"
            "{%- generation -%}" + assistant_body + "{{- '<|im_end|>' -}}{%- endgeneration -%}"
            "{%- else -%}"
            "{{- message['content'] + '<|im_end|>' -}}"
            "{%- endif -%}"
            "{{- '\n' -}}"
            "{%- endfor -%}"
            "{%- if add_generation_prompt -%}{{- '<|im_start|>assistant\n' -}}{%- endif -%}")


_KEEP = "{{- message['content'] -}}"
# earlier assistant turns lose their <think>...</think> part (what Qwen3's own template does); the last message, if it
# is the assistant's, keeps it
_DROP_OLD_THINKING = ("{%- set body = message['content'] -%}"
                      "{%- if '</think>' in body and not (loop.last and message['role'] == 'assistant') -%}"
                      "{%- set body = body.split('</think>')[-1].lstrip('\n') -%}"
                      "{%- endif -%}"
                      "{{- body -}}")
_KEEP_REASONING_FIELD = ("{%- if message.get('reasoning_content') -%}"
                         "{{- '<think>\n' + message['reasoning_content'] + '\n</think>\n\n' -}}{%- endif -%}"
                         "{{- message['content'] -}}")

# ChatML without the "You are a helpful assistant" default that some tokenizers insert when no system message is given:
# what a multi-turn rollout wants, because the conversation is tokenised piece by piece.  Unlike the reference's
# templates of the same names these also honour ``add_generation_prompt``.
CUSTOM_CHAT_TEMPLATES: Dict[str, str] = {
    "chatml_no_default_system": _chatml(_KEEP),
    # keeps earlier turns' <think> blocks (Qwen3's own template drops them, which changes the tokens of past turns)
    "chatml_keep_thinking": _chatml(_KEEP_REASONING_FIELD),
    # the names the reference registers (generators/utils.py:66-102)
    "qwen3_with_thinking": _chatml(_KEEP),
    "qwen3_without_thinking": _chatml(_DROP_OLD_THINKING),
}


def get_custom_chat_template(chat_template_config: Optional[Any] = None) -> Optional[str]:
    """``{"source": "name" | "file", "name_or_path": ...}`` (dict or config object) -> Jinja template text, or None to
    keep the tokenizer's own template.  Files must be regular ``.jinja`` / ``.jinja2`` / ``.j2`` / ``.txt`` files."""
    import os

    if chat_template_config is None:
        return None
    get = chat_template_config.get if isinstance(chat_template_config, dict) else lambda k, d=None: getattr(chat_template_config, k, d)
    source, name = get("source"), get("name_or_path")
    if not source:
        raise ValueError("chat template config needs a 'source' ('name' or 'file')")
    if not name:
        return None
    if source == "name":
        if name not in CUSTOM_CHAT_TEMPLATES:
            raise ValueError(f"unknown chat template '{name}'; available: {sorted(CUSTOM_CHAT_TEMPLATES)}")
        return CUSTOM_CHAT_TEMPLATES[name]
    if source == "file":
        path = os.path.realpath(os.path.expanduser(str(name)))
        if not os.path.isfile(path) or os.path.splitext(path)[1].lower() not in (".jinja", ".jinja2", ".j2", ".txt"):
            raise ValueError(f"chat template file '{name}' must be an existing .jinja / .jinja2 / .j2 / .txt file")
        with open(path, encoding="utf-8") as f:
            return f.read()
    raise ValueError(f"chat template source must be 'name' or 'file', got '{source}'")


def get_generation_prompt_ids(tokenizer, tokenizer_kwargs: Optional[Dict[str, Any]] = None) -> List[int]:
    """Token ids the chat template appends to open an assistant turn (``<|im_start|>assistant\\n`` for ChatML): the
    difference between templating one user message with and without the generation prompt."""
    kw = dict(tokenizer_kwargs or {})
    if "enable_thinking" in kw:
        raise ValueError("enable_thinking changes the generation prompt per call: use encode_messages_subset")
    probe = [{"role": "user", "content": ""}]
    plain = chat_template_ids(tokenizer, probe, **kw)
    opened = chat_template_ids(tokenizer, probe, add_generation_prompt=True, **kw)
    return opened[len(plain):]


_BASE_CONVERSATION = [{"role": "system", "content": "."}, {"role": "user", "content": "."}]


def encode_messages_subset(messages: List[Dict[str, Any]], tokenizer, tokenizer_kwargs: Optional[Dict[str, Any]] = None) -> List[int]:
    """Token ids of ``messages`` as they appear *inside* a longer conversation: a fixed two-message base conversation is
    templated with and without them and the base's tokens are cut off, so a template that injects a default system
    prompt (or a BOS token) at the start of a conversation does not inject it in the middle of a trajectory.  If the
    last message is not an assistant message the generation prompt is *not* included."""
    if not messages:
        raise ValueError("messages must not be empty")
    kw = dict(tokenizer_kwargs or {})
    base = chat_template_ids(tokenizer, _BASE_CONVERSATION, add_generation_prompt=False, **kw)
    full = chat_template_ids(tokenizer, _BASE_CONVERSATION + list(messages), add_generation_prompt=False, **kw)
    if full[: len(base)] != base:
        raise ValueError("the chat template does not extend a conversation by appending tokens; give a custom template")
    return full[len(base):]


def get_response_ids_and_loss_mask_from_messages(messages: List[Dict[str, Any]], tokenizer,
                                                 assistant_logprobs: Optional[List[List[float]]] = None,
                                                 tokenizer_kwargs: Optional[Dict[str, Any]] = None):
    """``(response_ids, loss_mask, rollout_logprobs | None)`` for the messages that follow the prompt.

    Every message is encoded on its own with ``encode_messages_subset``.  Tokens of non-assistant messages are masked
    out.  In an assistant message the generation prompt that opens the turn is masked out (the model did not produce
    it), the tokens up to and including the end-of-turn token are trained on, and anything the template adds after
    that token (a newline in ChatML) is masked out again.  ``assistant_logprobs[i]`` are the engine's log-probs of the
    i-th assistant message's generated tokens: they are aligned to the trained positions (zeros elsewhere); when the
    counts disagree by the end-of-turn token -- engines that stop *before* emitting it -- the missing entry is 0."""
    if not messages:
        raise ValueError("messages must not be empty")
    gen_prompt = get_generation_prompt_ids(tokenizer, {k: v for k, v in (tokenizer_kwargs or {}).items() if k != "enable_thinking"})
    eos = getattr(tokenizer, "eos_token_id", None)
    ids: List[int] = []
    mask: List[int] = []
    lps: Optional[List[float]] = [] if assistant_logprobs is not None else None
    a_idx = 0
    for msg in messages:
        cur = encode_messages_subset([msg], tokenizer, tokenizer_kwargs)
        ids.extend(cur)
        if msg.get("role") != "assistant":
            mask.extend([0] * len(cur))
            if lps is not None:
                lps.extend([0.0] * len(cur))
            continue
        lead = len(gen_prompt) if cur[: len(gen_prompt)] == gen_prompt else 0
        end = len(cur)
        if eos is not None and eos in cur[lead:]:
            end = len(cur) - cur[::-1].index(eos)  # one past the last end-of-turn token
        n_train = end - lead
        mask.extend([0] * lead + [1] * n_train + [0] * (len(cur) - end))
        if lps is not None:
            given = list(assistant_logprobs[a_idx]) if a_idx < len(assistant_logprobs) else []
            if len(given) not in (n_train, n_train - 1):
                raise ValueError(f"assistant message {a_idx}: {len(given)} log-probs for {n_train} generated tokens")
            given = given + [0.0] * (n_train - len(given))
            lps.extend([0.0] * lead + given + [0.0] * (len(cur) - end))
        a_idx += 1
    return ids, mask, lps


def apply_overlong_filtering(loss_masks: List[List[int]], stop_reasons: List[str]) -> List[List[int]]:
    """DAPO overlong filtering: a response that did not end by itself (stop reason other than ``stop``) is not
    trained on at all.  Uses the engine's stop reasons, so it does not depend on a particular end-of-sequence id."""
    if len(loss_masks) != len(stop_reasons):
        raise ValueError("loss_masks and stop_reasons must have the same length")
    return [list(m) if r == "stop" else [0] * len(m) for m, r in zip(loss_masks, stop_reasons)]


def compute_turn_token_counts(loss_masks: List[List[int]]) -> List[int]:
    """Generated tokens per assistant turn over a batch: every maximal run of non-zero loss-mask entries is one turn
    (observation tokens are masked, so they separate the runs).  Fully masked trajectories contribute nothing."""
    counts: List[int] = []
    for m in loss_masks:
        run = 0
        for v in m:
            if v:
                run += 1
            elif run:
                counts.append(run)
                run = 0
        if run:
            counts.append(run)
    return counts


def slice_generator_output(out: GeneratorOutput, start: int, end: int) -> GeneratorOutput:
    """Rows ``[start, end)`` of every per-trajectory list of a generator output (scalars and ``None`` pass through)."""
    n = len(out["response_ids"])
    res: Dict[str, Any] = {}
    for k, v in out.items():
        if k == "trajectory_time_splits" and isinstance(v, dict):
            res[k] = {name: (t[start:end] if len(t) == n else t) for name, t in v.items()}
        else:
            res[k] = v[start:end] if isinstance(v, list) and len(v) == n else v
    return res  # type: ignore[return-value]


# ----------------------------------------------------------------------------- output validation
class GeneratorOutputError(ValueError):
    """A generator handed the trainer rows that do not fit together."""


def _tid(t) -> str:
    return t.to_string() if hasattr(t, "to_string") else str(t)


def validate_generator_output(num_prompts: int, out: GeneratorOutput, step_wise: bool = False) -> List[str]:
    """Checks a ``GeneratorOutput`` before it is turned into tensors, so that a hand-written generator fails with a
    message about its own output instead of an index error three layers down.  Returns warnings (conditions that are
    legal but usually a bug, e.g. every token masked out).  Reference: trainer_utils.py:672-826 (same rules).

    * at least one response; one response per prompt unless ``step_wise`` (then one per step);
    * every per-row field (``prompt_token_ids, loss_masks, rewards, stop_reasons, rollout_logprobs, trajectory_ids,
      is_last_step, rollout_expert_indices``), when given, has one entry per response;
    * per row: ``len(loss_mask) == len(response)``, token-level rewards and rollout log-probs have the response's
      length; rewards are all floats or all lists of floats, never a mixture;
    * step-wise: ``is_last_step`` and ``trajectory_ids`` present, the last row ends a trajectory, the rows of a
      trajectory are adjacent, and ``is_last_step`` is true exactly where the trajectory id changes."""
    resp = out.get("response_ids")
    if not resp:
        raise GeneratorOutputError("the generator returned no responses")
    n = len(resp)
    if not step_wise and n != num_prompts:
        raise GeneratorOutputError(f"{num_prompts} prompts but {n} responses")
    for key in ("prompt_token_ids", "loss_masks", "rewards", "stop_reasons", "rollout_logprobs", "trajectory_ids",
                "is_last_step", "rollout_expert_indices"):
        v = out.get(key)
        if isinstance(v, (list, tuple)) and len(v) != n:
            raise GeneratorOutputError(f"'{key}' has {len(v)} entries for {n} responses")
    masks, rewards, lps = out.get("loss_masks"), out.get("rewards"), out.get("rollout_logprobs")
    if masks is None or rewards is None:
        raise GeneratorOutputError("'loss_masks' and 'rewards' are required")
    kinds = {isinstance(r, (list, tuple)) for r in rewards}
    if len(kinds) > 1:
        raise GeneratorOutputError("rewards mix per-trajectory floats and per-token lists")
    per_token = kinds == {True}
    for i, r in enumerate(resp):
        if len(masks[i]) != len(r):
            raise GeneratorOutputError(f"row {i}: loss mask has {len(masks[i])} entries for {len(r)} response tokens")
        if per_token:
            if len(rewards[i]) != len(r):
                raise GeneratorOutputError(f"row {i}: {len(rewards[i])} token rewards for {len(r)} response tokens")
            if not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in rewards[i]):
                raise GeneratorOutputError(f"row {i}: token rewards must be numbers")
        elif not isinstance(rewards[i], (int, float)) or isinstance(rewards[i], bool):
            raise GeneratorOutputError(f"row {i}: reward must be a number or a list of numbers, got {type(rewards[i]).__name__}")
        if lps and lps[i] is not None and len(lps[i]) != len(r):
            raise GeneratorOutputError(f"row {i}: {len(lps[i])} rollout log-probs for {len(r)} response tokens")
    warnings: List[str] = []
    if not any(any(m) for m in masks):
        warnings.append("every response token is masked out of the loss: the policy loss will be 0/0")
    if step_wise:
        last, tids = out.get("is_last_step"), out.get("trajectory_ids")
        if last is None or tids is None:
            raise GeneratorOutputError("step-wise output needs 'is_last_step' and 'trajectory_ids'")
        if last[-1] is not True:
            raise GeneratorOutputError("the last row must be the final step of a trajectory (is_last_step[-1] is not True)")
        keys = [_tid(t) for t in tids]
        done: set = set()
        for i, k in enumerate(keys):
            if i and k != keys[i - 1]:
                done.add(keys[i - 1])
                if last[i - 1] is not True:
                    raise GeneratorOutputError(f"trajectory '{keys[i - 1]}' ends at row {i - 1} but is_last_step[{i - 1}] is not True")
            elif i and last[i - 1] is True:
                raise GeneratorOutputError(f"is_last_step[{i - 1}] is True but trajectory '{k}' continues at row {i}")
            if k in done:
                raise GeneratorOutputError(f"rows of trajectory '{k}' are not adjacent (it reappears at row {i})")
    return warnings
