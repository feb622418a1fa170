"""Dynamic sampling of the training batch: ``filter`` (DAPO) and ``replace`` (POLARIS) strategies.

Behavioural reference: skyrl/train/utils/trainer_utils.py:392-608 and ``RayPPOTrainer.handle_dynamic_sampling``
(skyrl/train/trainer.py:1584-1644).  A prompt group is *informative* when its samples' total rewards differ (or when
there is one sample per prompt).

* ``filter``: drop uninformative groups, keep the rest, and ask for another rollout batch until ``target_prompts``
  informative groups have been collected (then truncate to exactly that many groups' trajectories).
* ``replace``: if more than ``min_replace_ratio`` of the groups are informative, overwrite every uninformative group
  with a randomly drawn informative one (the batch keeps its size); otherwise ask for another rollout batch.

Process model: every rank holds its own share of the prompt batch, so ``target_prompts`` is the per-rank share and the
"keep sampling?" decision is made jointly (a rank that has enough waits for the others), which keeps every rank's
share equal and the ranks in step on the data loader.
"""

from __future__ import annotations

from collections import defaultdict
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from .generators.base import GeneratorOutput
from .generators.utils import concatenate_generator_outputs, get_rollout_metrics

_ROW_KEYS = ("prompt_token_ids", "response_ids", "rewards", "loss_masks", "stop_reasons", "rollout_logprobs",
             "trajectory_ids", "is_last_step", "env_metrics", "trajectory_generation_times", "rollout_expert_indices",
             "pixel_values", "image_grid_thw")


def select_rows(out: GeneratorOutput, idx: Sequence[int]) -> GeneratorOutput:
    """Rows ``idx`` (repeats allowed) of every per-trajectory field; rollout metrics are recomputed."""
    res = GeneratorOutput()
    for k, v in out.items():
        if k in _ROW_KEYS and isinstance(v, list):
            res[k] = [v[i] for i in idx]
        elif k == "trajectory_time_splits" and isinstance(v, dict):
            res[k] = {name: [times[i] for i in idx] for name, times in v.items()}  # per-trajectory lists by name
        else:
            res[k] = v
    if res.get("response_ids") is not None and res.get("rewards") is not None:
        res["rollout_metrics"] = get_rollout_metrics(res["response_ids"], res["rewards"], res.get("env_metrics"),
                                                     loss_masks=res.get("loss_masks"),
                                                     trajectory_completion_times=res.get("trajectory_generation_times"),
                                                     trajectory_time_splits=res.get("trajectory_time_splits"))
    return res


def _scores(out: GeneratorOutput) -> np.ndarray:
    return np.array([float(sum(r)) if isinstance(r, (list, tuple)) else float(r) for r in out["rewards"]], dtype=np.float64)


def group_informative(out: GeneratorOutput, uids: Sequence[str], n_samples_per_prompt: int) -> Dict[str, bool]:
    """uid -> whether the group's rewards have non-zero spread (always true with one sample per prompt)."""
    vals: Dict[str, List[float]] = defaultdict(list)
    for u, s in zip(uids, _scores(out)):
        vals[u].append(s)
    return {u: (n_samples_per_prompt == 1 or float(np.std(v)) > 0.0) for u, v in vals.items()}


class DynamicSampler:
    """State of one RL step's sampling rounds. ``handle`` returns ``(output, uids, keep_sampling)``."""

    def __init__(self, kind: str, target_prompts: int, n_samples_per_prompt: int, max_sample_batches: int = 30,
                 min_replace_ratio: float = 0.3, seed: int = 0, all_ranks_done=None):
        if kind not in ("filter", "replace"):
            raise ValueError(f"Invalid dynamic sampling type: {kind}")
        self.kind, self.target, self.n = kind, int(target_prompts), int(n_samples_per_prompt)
        self.max_batches, self.min_ratio = int(max_sample_batches), float(min_replace_ratio)
        self.rng = np.random.default_rng(seed)
        self.all_ranks_done = all_ranks_done or (lambda done: done)
        self.reset()

    def reset(self) -> None:
        self.rounds = 0
        self.collected: Optional[GeneratorOutput] = None
        self.collected_uids: List[str] = []
        self.collected_prompts = 0

    # ------------------------------------------------------------------ strategies
    def _filter(self, out: GeneratorOutput, uids: List[str]) -> Tuple[GeneratorOutput, List[str], bool]:
        good = group_informative(out, uids, self.n)
        if self.collected_prompts < self.target:
            keep = [i for i, u in enumerate(uids) if good[u]]
            part = select_rows(out, keep)
            if part.get("response_ids"):
                self.collected = part if self.collected is None else concatenate_generator_outputs([self.collected, part])
                self.collected_uids.extend(uids[i] for i in keep)
                self.collected_prompts += sum(1 for v in good.values() if v)
        done = self.all_ranks_done(self.collected_prompts >= self.target)
        if not done:
            return out, uids, True
        # exactly `target` groups: uids arrive group by group, so cut at the first trajectory of group target + 1
        seen: List[str] = []
        cut = len(self.collected_uids)
        for i, u in enumerate(self.collected_uids):
            if u not in seen:
                if len(seen) == self.target:
                    cut = i
                    break
                seen.append(u)
        final = select_rows(self.collected, list(range(cut)))
        return final, self.collected_uids[:cut], False

    def _replace(self, out: GeneratorOutput, uids: List[str]) -> Tuple[GeneratorOutput, List[str], bool]:
        good = group_informative(out, uids, self.n)
        rows: Dict[str, List[int]] = defaultdict(list)
        for i, u in enumerate(uids):
            rows[u].append(i)
        good_uids = [u for u in rows if good[u]]
        bad_uids = [u for u in rows if not good[u]]
        enough = len(good_uids) > len(rows) * self.min_ratio
        if not self.all_ranks_done(enough):
            return out, uids, True
        if not bad_uids or not enough:
            return out, uids, False
        # without replacement while the informative groups last, with replacement beyond that
        if len(bad_uids) <= len(good_uids):
            picks = list(self.rng.choice(len(good_uids), size=len(bad_uids), replace=False))
        else:
            picks = list(self.rng.choice(len(good_uids), size=len(bad_uids), replace=True))
        src = list(range(len(uids)))
        new_uids = list(uids)
        for b, k in zip(bad_uids, picks):
            g = good_uids[int(k)]
            for dst_i, src_i in zip(rows[b], rows[g]):
                src[dst_i] = src_i
                new_uids[dst_i] = f"{g}#r{b}"  # a distinct group id: the copy is normalised with its own statistics
        return select_rows(out, src), new_uids, False

    # ------------------------------------------------------------------ driver
    def handle(self, out: GeneratorOutput, uids: List[str]) -> Tuple[GeneratorOutput, List[str], bool]:
        self.rounds += 1
        res, ruids, keep = (self._filter if self.kind == "filter" else self._replace)(out, list(uids))
        if keep and self.max_batches > 0 and self.rounds >= self.max_batches:
            raise RuntimeError(f"dynamic sampling ({self.kind}) hit max_sample_batches={self.max_batches} without "
                               "collecting a full batch; check the difficulty distribution of the data")
        self.last_rounds = self.rounds
        if not keep:
            self.reset()
        return res, ruids, keep

    def metrics(self) -> Dict[str, float]:
        return {"dynamic_sampling/sample_batches": float(getattr(self, "last_rounds", self.rounds))}
