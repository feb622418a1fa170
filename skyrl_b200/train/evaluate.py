"""Evaluation loop: generate with the eval sampling parameters, aggregate per-dataset metrics and
optionally dump trajectories to JSONL (reference: skyrl/train/evaluate.py, trainer_utils.py:227-374)."""

from __future__ import annotations

import json
import os
from collections import defaultdict
from typing import Any, Dict, List

import numpy as np

from .generators.utils import get_metrics_from_generator_output, prepare_generator_input


def calculate_per_dataset_metrics(out, uids: List[str], data_sources: List[str], n_samples: int) -> Dict[str, float]:
    by_src: Dict[str, List[int]] = defaultdict(list)
    for i, s in enumerate(data_sources):
        by_src[s or "default"].append(i)
    m: Dict[str, float] = {}
    for src, idxs in by_src.items():
        sub = {"rewards": [out["rewards"][i] for i in idxs]}
        mm = get_metrics_from_generator_output(sub, [uids[i] for i in idxs])
        m[f"eval/{src}/avg_score"] = mm["avg_score"]
        m[f"eval/{src}/pass_at_{n_samples}"] = mm["pass_at_n"]
        m[f"eval/{src}/mean_positive_reward"] = mm["mean_positive_reward"]
    return m


async def evaluate(eval_dataset, generator, cfg, global_step: int, tokenizer=None, env=None, tracker=None
                   ) -> Dict[str, float]:
    g = cfg.generator
    first_out = None
    sp = g.eval_sampling_params.to_dict() if g.eval_sampling_params is not None else None
    bs = cfg.trainer.eval_batch_size
    items = list(eval_dataset.items)
    if env is not None and env.world_size > 1:
        items = items[env.rank :: env.world_size]
    all_rewards, all_uids, all_src, dumps = [], [], [], []
    for s in range(0, len(items), bs):
        chunk = items[s : s + bs]
        gi, uids = prepare_generator_input(chunk, g.eval_n_samples_per_prompt, sp, cfg.environment.env_class, "eval",
                                           global_step)
        out = await generator.generate(gi)
        if first_out is None:
            first_out = (out, uids)
        srcs = [(it.get("env_extras") or {}).get("data_source") for it in chunk for _ in range(g.eval_n_samples_per_prompt)]
        if g.step_wise_trajectories and out.get("is_last_step") is not None:
            # one row per step: score every trajectory by its last step (where the reward sits) and take the prompt uid
            # and data source from the trajectory id (reference: evaluate.py:178-300, ``evaluate_step_wise``)
            src_of = {t.instance_id: s for t, s in zip(gi["trajectory_ids"], srcs)} if gi.get("trajectory_ids") else {}
            keep = [i for i, last in enumerate(out["is_last_step"]) if last]
            tids = out.get("trajectory_ids") or []
            uids = [tids[i].instance_id if tids else uids[min(i, len(uids) - 1)] for i in keep]
            srcs = [src_of.get(u) for u in uids]
            out = {k: ([v[i] for i in keep] if isinstance(v, list) and len(v) == len(out["is_last_step"]) else v)
                   for k, v in out.items()}
        all_rewards.extend(out["rewards"])
        all_uids.extend(uids)
        all_src.extend(srcs)
        if cfg.trainer.dump_eval_results and tokenizer is not None:
            for p, r, rew, stop in zip(out["prompt_token_ids"], out["response_ids"], out["rewards"], out["stop_reasons"]):
                dumps.append({"prompt": tokenizer.decode(p), "response": tokenizer.decode(r),
                              "reward": float(np.sum(rew)), "stop_reason": stop})
    if env is not None and env.world_size > 1:
        # every rank evaluated its own slice of the set: merge the slices so that the metrics cover the whole set
        import torch.distributed as dist

        if dist.is_initialized():
            parts = [None] * env.world_size
            dist.all_gather_object(parts, (all_rewards, all_uids, all_src, dumps))
            all_rewards = [x for p in parts for x in p[0]]
            all_uids = [x for p in parts for x in p[1]]
            all_src = [x for p in parts for x in p[2]]
            dumps = [x for p in parts for x in p[3]]
    t = cfg.trainer
    if first_out is not None and (env is None or env.is_main) and (t.print_example_interval > 0 or t.num_logger_eval_samples > 0):
        # one decoded example to the log, up to ``num_logger_eval_samples`` trajectories to JSONL / the tracker's table
        # (reference: evaluate.py:105-125)
        import logging

        from ..utils.trajectory_logging import TrajectoryLogger

        tl = TrajectoryLogger(os.path.join(t.log_path, "trajectories"), tokenizer, max_rows=max(1, t.num_logger_eval_samples),
                              tracker=tracker)
        if t.print_example_interval > 0:
            row = tl.rows(*first_out)[0]
            logging.getLogger(__name__).info("eval example at step %d | reward %.3f\n--- prompt ---\n%s\n--- response ---\n%s",
                                             global_step, row["reward"], row["prompt"], row["response"])
        if t.num_logger_eval_samples > 0:
            tl.log(first_out[0], global_step, "eval", first_out[1])
    out_all = {"rewards": all_rewards}
    mm = get_metrics_from_generator_output(out_all, all_uids)
    metrics = {"eval/all/avg_score": mm["avg_score"], f"eval/all/pass_at_{g.eval_n_samples_per_prompt}": mm["pass_at_n"],
               "eval/all/mean_positive_reward": mm["mean_positive_reward"]}
    metrics.update(calculate_per_dataset_metrics(out_all, all_uids, all_src, g.eval_n_samples_per_prompt))
    if dumps and (env is None or env.is_main):
        d = os.path.join(cfg.trainer.export_path, "dumped_evals", f"global_step_{global_step}_evals")
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, "eval.jsonl"), "w") as f:
            for row in dumps:
                f.write(json.dumps(row) + "\n")
    return metrics
