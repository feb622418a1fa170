"""Synchronous PPO / GRPO controller.

One RL step (reference: ``RayPPOTrainer.train`` skyrl/train/trainer.py:271-601) is

    generate -> postprocess rewards -> tensorise -> forward (old policy / ref / critic) ->
    KL-in-reward -> advantages -> train critic + policy (mini-batches x epochs) -> checkpoint ->
    weight sync -> log

The process model is SPMD: every rank runs this controller on *its own shard* of the prompt batch
with its colocated generation engine, so no batch ever crosses a process boundary.  Ranks meet only
inside the sharded optimizer step (gradient reduce-scatter, parameter push) and when metrics are
averaged.  With the engine reading the trainer's parameter buffer in place, "weight sync" after an
update is the parameter push of the optimizer step itself plus a version bump that retires stale
prefix-cache entries.
"""

from __future__ import annotations

import asyncio
import logging
import math
import os
import time
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from ..algorithms import rl
from ..engine.llm_engine import EngineConfig, LLMEngine
from ..inference.local_client import LocalInferenceClient
from ..parallel.dist import DistEnv, get_env
from ..workers.worker import CriticWorker, PolicyWorker, RefWorker
from . import utils as tutils
from .batch import TrainingInputBatch, pad_training_input_batch
from .callbacks import CallbackHandler
from .dataset import PromptDataset, StatefulBatchIterator
from .generators.base import GeneratorInput, GeneratorInterface, GeneratorOutput
from .generators.skyrl_gym_generator import SkyRLGymGenerator
from .generators.utils import (compute_pass_at_n, get_metrics_from_generator_output, prepare_generator_input,
                               validate_generator_output)
from .preprocess import (compute_prompt_boundaries, compute_prompt_mini_batch_boundaries,
                         convert_prompts_responses_to_batch_tensors)
from .tracking import Tracking
from .utils import Timer

logger = logging.getLogger(__name__)


class PPOTrainer:
    def __init__(self, cfg, tracker: Optional[Tracking] = None, tokenizer=None, train_dataset: Optional[PromptDataset] = None,
                 eval_dataset: Optional[PromptDataset] = None, inference_engine_client=None,
                 generator: Optional[GeneratorInterface] = None, env: Optional[DistEnv] = None):
        self.cfg = cfg
        self.env = env or get_env()
        self.tracker = tracker
        self.tokenizer = tokenizer
        self.train_dataset, self.eval_dataset = train_dataset, eval_dataset
        self.inference_engine_client = inference_engine_client
        self.generator = generator
        self.policy: Optional[PolicyWorker] = None
        self.ref: Optional[RefWorker] = None
        self.critic: Optional[CriticWorker] = None
        self.engine: Optional[LLMEngine] = None
        self.global_step = 0
        self.all_metrics: Dict[str, float] = {}
        self.all_timings: Dict[str, float] = {}
        self.kl_controller = rl.get_kl_controller(cfg.trainer.algorithm) if cfg.trainer.algorithm.use_kl_in_reward else None
        self.train_iter: Optional[StatefulBatchIterator] = None
        from ..workers.dispatch import WorkerDispatch

        self.dispatch = WorkerDispatch(self)  # the reference's worker verbs by role name (trainer.dispatch.forward(...))
        self.callbacks = CallbackHandler([])  # add with trainer.callbacks.add(cb) (or append: it is list-like enough)
        self.dynamic_sampler = None
        tutils.validate_cfg(cfg, self.env.world_size)
        torch.manual_seed(cfg.trainer.seed + self.env.rank)
        np.random.seed(cfg.trainer.seed + self.env.rank)

    # ------------------------------------------------------------------ construction
    def build_models(self, policy_model=None, peer_ctx=None) -> None:
        """Create the policy (and optional ref / critic) workers and the colocated generation engine."""
        t = self.cfg.trainer
        a = t.algorithm
        if (peer_ctx is None and self.env.world_size > 1 and self.env.device.type == "cuda" and t.b200.fused_optimizer
                and policy_model is None):
            from ..parallel.peer import PeerContext

            peer_ctx = PeerContext(self.env.device)
        self.peer_ctx = peer_ctx
        self.policy = PolicyWorker(t, model=policy_model, model_path=t.policy.model.path, env=self.env, peer_ctx=peer_ctx,
                                   seed=t.seed)
        if a.use_kl_loss or a.use_kl_in_reward:
            self.ref = RefWorker(t, model_path=t.ref.model.path or t.policy.model.path, env=self.env, seed=t.seed)
        if a.advantage_estimator == "gae" or t.critic.model.path is not None:
            self.critic = CriticWorker(t, model_path=t.critic.model.path or t.policy.model.path, env=self.env,
                                       seed=t.seed + 1)
        if self.inference_engine_client is None:
            etp = int(self.cfg.generator.inference_engine.tensor_parallel_size or 1)
            if etp > 1 and (self.env.world_size % etp or not dist.is_initialized()):
                raise ValueError(f"generator.inference_engine.tensor_parallel_size={etp} must divide the world size "
                                 f"{self.env.world_size}")
            self.engine_tp = etp
            self.engine = self._build_engine(self.policy.engine_model(etp))
            self.inference_engine_client = LocalInferenceClient([self.engine], self.tokenizer)
        if self.generator is None:
            self.generator = SkyRLGymGenerator(self.cfg.generator, self.cfg.environment.skyrl_gym,
                                               self.inference_engine_client, self.tokenizer)

    def _build_engine(self, model) -> LLMEngine:
        g, ie, b = self.cfg.generator, self.cfg.generator.inference_engine, self.cfg.trainer.b200
        max_len = (g.max_input_length or self.cfg.trainer.max_prompt_length) + g.sampling_params.max_generate_length
        ecfg = EngineConfig(block_size=b.kv_block_size, gpu_memory_utilization=ie.gpu_memory_utilization,
                            max_num_seqs=ie.max_num_seqs, max_num_batched_tokens=max(ie.max_num_batched_tokens, max_len),
                            max_model_len=max_len, enable_prefix_caching=ie.enable_prefix_caching,
                            enforce_eager=ie.enforce_eager or not b.cuda_graph_decode,
                            return_routed_experts=bool(ie.enable_return_routed_experts),
                            # the ranks of one tensor-parallel engine must draw the same samples
                            seed=self.cfg.trainer.seed + self.env.rank // max(1, getattr(self, "engine_tp", 1)))
        spec = bool(self.cfg.trainer.mtp.enabled and b.speculative_decode and getattr(self, "engine_tp", 1) == 1
                    and not ie.enable_return_routed_experts and getattr(self.policy, "mtp_head", None) is not None)
        if spec:
            ecfg.num_speculative_tokens = 1  # one draft head: deeper settings of trainer.mtp.num_speculative_tokens run as 1
        if b.decode_graph_batch_sizes:
            ecfg.graph_batch_sizes = tuple(sorted(int(x) for x in b.decode_graph_batch_sizes))
        for k, v in (ie.engine_init_kwargs or {}).items():
            if hasattr(ecfg, k):
                setattr(ecfg, k, v)
        eos = [self.tokenizer.eos_token_id] if self.tokenizer is not None and self.tokenizer.eos_token_id is not None else []
        detok = (lambda ids: self.tokenizer.decode(ids, skip_special_tokens=False)) if self.tokenizer is not None else None
        eng = LLMEngine(model, ecfg, eos_token_ids=eos, detokenize=detok)
        if spec:
            eng.set_draft_head(self.policy.mtp_head)  # shared with the trainer: drafts follow every optimizer step
        if getattr(self, "engine_tp", 1) > 1:
            from ..engine.lockstep import LockstepEngine

            emesh = self.policy.engine_mesh
            eng = LockstepEngine(eng, emesh.tp_cpu_group, self.env.rank - emesh.tp_rank)
        return eng

    # ------------------------------------------------------------------ data
    def _local_prompts(self, global_batch: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
        """This rank's contiguous share of the global prompt batch (tail prompts dropped to keep shares equal)."""
        W, r = self.env.world_size, self.env.rank
        per = len(global_batch) // W
        return global_batch[r * per : (r + 1) * per]

    # ------------------------------------------------------------------ rollout
    async def _generate_lockstep(self, gen_input: GeneratorInput) -> GeneratorOutput:
        """Rollout through a tensor-parallel engine: the group's leader generates for the prompts of all its ranks
        while the others mirror its engine steps; every rank then keeps the rows of its own prompts."""
        emesh = self.policy.engine_mesh
        grp, tp = emesh.tp_cpu_group, emesh.tp_size
        parts: List[Any] = [None] * tp
        dist.all_gather_object(parts, dict(gen_input), group=grp)
        counts = [len(p["prompts"]) for p in parts]
        box: List[Any] = [None]
        if self.engine.is_leader:
            merged = GeneratorInput()
            for key in parts[0]:
                vals = [p.get(key) for p in parts]
                merged[key] = [x for v in vals for x in v] if all(isinstance(v, list) for v in vals) else vals[0]
            try:
                box[0] = await self.generator.generate(merged)
            finally:
                self.engine.end_generation()
        else:
            await asyncio.to_thread(self.engine.follow)
        dist.broadcast_object_list(box, src=self.engine.leader, group=grp)
        out = box[0]
        n_rows, n_in = len(out["response_ids"]), sum(counts)
        if n_rows != n_in:
            raise NotImplementedError("step-wise trajectories are not supported with a tensor-parallel engine")
        lo = sum(counts[: emesh.tp_rank])
        from .dynamic_sampling import select_rows

        return select_rows(out, list(range(lo, lo + counts[emesh.tp_rank])))

    async def generate(self, gen_input: GeneratorInput) -> GeneratorOutput:
        if getattr(self, "engine_tp", 1) > 1 and self.engine is not None:
            out = await self._generate_lockstep(gen_input)
        else:
            out = await self.generator.generate(gen_input)
        n = len(out["response_ids"])
        for key in ("prompt_token_ids", "rewards", "loss_masks"):
            if len(out[key]) != n:
                raise ValueError(f"generator output field '{key}' has {len(out[key])} rows, expected {n}")
        return out

    def postprocess_generator_output(self, out: GeneratorOutput, uids: List[str],
                                     metrics_generator_output: Optional[GeneratorOutput] = None,
                                     metrics_uids: Optional[List[str]] = None):
        """Scalar rewards -> last response token; reward metrics; optional merge of step-wise rows; optional
        zero-variance filter.  Returns ``(output, uids)`` -- ``uids`` gets shorter when step-wise rows are merged
        (reference: trainer.py:1013-1121).

        The reward metrics are computed over ``metrics_generator_output`` / ``metrics_uids`` when given (a superset of
        the trained rows: the fully-async trainer passes the groups it dropped so that the numbers stay comparable),
        and, for step-wise rollouts, over the last step of every trajectory only."""
        a, g = self.cfg.trainer.algorithm, self.cfg.generator
        m_out = metrics_generator_output if metrics_generator_output is not None else out
        m_uids = list(metrics_uids if metrics_uids is not None else uids)
        m_rewards = list(m_out["rewards"])
        if g.step_wise_trajectories and m_out.get("is_last_step") is not None:
            keep = [i for i, last in enumerate(m_out["is_last_step"]) if last]
            m_rewards, m_uids = [m_rewards[i] for i in keep], [m_uids[i] for i in keep]
        mm = get_metrics_from_generator_output({"rewards": m_rewards}, m_uids)
        m = {"reward/avg_raw_reward": mm["avg_score"], f"reward/avg_pass_at_{g.n_samples_per_prompt}": mm["pass_at_n"],
             "reward/mean_positive_reward": mm["mean_positive_reward"]}
        if g.merge_stepwise_output:
            if not g.step_wise_trajectories:
                raise ValueError("generator.merge_stepwise_output needs generator.step_wise_trajectories=true")
            from .generators.utils import merge_stepwise_output

            before = len(out["response_ids"])
            out = merge_stepwise_output(out)
            m["generate/num_seq_before_merge"], m["generate/num_seq_after_merge"] = float(before), float(len(out["response_ids"]))
            uids = [t.instance_id for t in out["trajectory_ids"]]
        per_token: List[List[float]] = []
        for r, resp in zip(out["rewards"], out["response_ids"]):
            if isinstance(r, (list, tuple)):
                per_token.append([float(x) for x in r])
            else:
                row = [0.0] * len(resp)
                if row:
                    row[-1] = float(r)
                per_token.append(row)
        if a.zero_variance_filter:
            scores = np.array([sum(r) for r in per_token], dtype=np.float64)
            groups: Dict[str, List[int]] = {}
            for i, u in enumerate(uids):
                groups.setdefault(u, []).append(i)
            masks = [list(x) for x in out["loss_masks"]]
            dropped = 0
            for idxs in groups.values():
                live = [i for i in idxs if any(masks[i])]
                if len(live) > 1 and float(np.ptp(scores[live])) <= a.zero_variance_filter_tol:
                    for i in live:
                        masks[i] = [0] * len(masks[i])
                    dropped += 1
            out["loss_masks"] = masks
            m["reward/zero_variance_groups"] = m["reward/num_zero_variance_filtered"] = float(dropped)
        out["rewards"] = per_token
        self.all_metrics.update(m)
        if out.get("rollout_metrics"):
            self.all_metrics.update(out["rollout_metrics"])
        return out, uids

    def convert_to_training_input(self, out: GeneratorOutput, uids: List[str]) -> TrainingInputBatch:
        pad_id = self.tokenizer.pad_token_id if self.tokenizer is not None and self.tokenizer.pad_token_id is not None else 0
        seq, att, rmask, rew, lmask, lps = convert_prompts_responses_to_batch_tensors(
            pad_id, out["prompt_token_ids"], out["response_ids"], out["rewards"], out["loss_masks"],
            out.get("rollout_logprobs"), max_seq_len=self.cfg.trainer.algorithm.max_seq_len)
        batch = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "rewards": rew,
                                    "loss_mask": lmask, "rollout_logprobs": lps})
        if out.get("rollout_expert_indices") is not None:
            # rollout-time expert choices, aligned with ``sequences`` (reference: dataset/preprocess.py:230-273)
            from ..models.router_replay import PAD, pad_routes

            routes = pad_routes(out["rollout_expert_indices"], att.sum(1).tolist(), seq.shape[1])
            batch["rollout_expert_indices"] = routes
            batch["router_padding_mask"] = routes[:, :, 0, 0] == PAD
        batch.metadata = {"uids": list(uids), "response_length": rmask.shape[1],
                          "is_last_step": out.get("is_last_step"),
                          "avg_response_length": float(rmask.sum(1).float().mean()),
                          "trajectory_ids": [t.to_string() for t in out["trajectory_ids"]] if out.get("trajectory_ids") else None}
        self.all_metrics["generate/avg_response_length"] = batch.metadata["avg_response_length"]
        return batch

    def handle_dynamic_sampling(self, out: GeneratorOutput, uids: List[str]):
        """DAPO ``filter`` / POLARIS ``replace`` (reference: trainer.py:1584-1644). Returns
        ``(output, uids, keep_sampling)``; with ``keep_sampling`` the caller rolls out the next prompt batch."""
        ds = self.cfg.trainer.algorithm.dynamic_sampling
        if self.dynamic_sampler is None:
            from .dynamic_sampling import DynamicSampler

            W = self.env.world_size

            def all_done(done: bool) -> bool:
                if not dist.is_initialized() or W == 1:
                    return done
                t = torch.tensor([1 if done else 0], dtype=torch.int32)
                dist.all_reduce(t, op=dist.ReduceOp.MIN)  # host tensor: gloo side of the process group
                return bool(t.item())

            share = max(1, self.cfg.trainer.train_batch_size * self._data_share() // W)
            self.dynamic_sampler = DynamicSampler(ds.type, share, self.cfg.generator.n_samples_per_prompt,
                                                  ds.max_sample_batches, ds.min_replace_ratio,
                                                  seed=self.cfg.trainer.seed + self.env.rank, all_ranks_done=all_done)
        res = self.dynamic_sampler.handle(out, uids)
        self.all_metrics.update(self.dynamic_sampler.metrics())
        return res

    # ------------------------------------------------------------------ forward passes
    def _skip_policy_forward(self) -> bool:
        """The old-policy forward can be skipped when the loss is anchored on the rollout log-probs and nothing else
        reads the old ones (reference: trainer.py:1279-1304; ``cispo`` qualifies only with the rollout anchor)."""
        a = self.cfg.trainer.algorithm
        if a.policy_loss_type == "cispo":
            anchored = a.cispo.cispo_anchor == "rollout"
        else:
            anchored = a.policy_loss_type in rl.LOSSES_WITHOUT_OLD_LOGPROBS
        return anchored and not a.use_kl_in_reward and not rl.off_policy_correction_enabled_cfg(a)

    def _forward_old(self, worker, role: str, batch: TrainingInputBatch) -> torch.Tensor:
        """Forward pass that produces "old" log-probs / values.  With ``recompute_old_logprobs_per_minibatch`` it runs
        mini-batch by mini-batch with the training packing, so the ratio is exactly 1 at the first inner step."""
        t = self.cfg.trainer
        if not t.recompute_old_logprobs_per_minibatch:
            return worker.forward(batch)["output"]
        dp = max(1, self.env.world_size // self._data_share())
        size = t.critic_mini_batch_size if role == "critic" else t.policy_mini_batch_size
        bounds = compute_prompt_mini_batch_boundaries(batch.metadata["uids"], max(1, size // dp))
        if len(bounds) <= 1 and t.micro_train_batch_size_per_gpu == t.micro_forward_batch_size_per_gpu:
            return worker.forward(batch, train_packing=True)["output"]
        parts = []
        for s, e in bounds:
            mini = batch.slice(s, e)
            mini.metadata = dict(batch.metadata)
            parts.append(worker.forward(mini, train_packing=True)["output"])
        return torch.cat(parts, 0)

    def _old_logprobs_from_train_forward(self) -> bool:
        """True when pi_old == pi_theta at the only optimizer step of this RL step (and nothing else needs pi_old)."""
        t = self.cfg.trainer
        single_update = self.num_policy_updates_per_step() == 1
        a = t.algorithm
        return (t.b200.reuse_train_forward_for_old_logprobs and single_update and not a.use_kl_in_reward
                and not rl.off_policy_correction_enabled_cfg(a) and a.policy_loss_type in ("regular", "dual_clip", "gspo",
                                                                                           "sapo", "cispo"))

    def fwd_logprobs_values_reward(self, batch: TrainingInputBatch) -> TrainingInputBatch:
        if self.critic is not None:
            batch["values"] = self._forward_old(self.critic, "critic", batch)
        if self.ref is not None:
            batch["base_action_log_probs"] = self._forward_old(self.ref, "ref", batch)
        if self._skip_policy_forward() and batch.get("rollout_logprobs") is not None:
            batch["action_log_probs"] = batch["rollout_logprobs"].clone()
        elif self._old_logprobs_from_train_forward():
            batch["action_log_probs"] = None  # filled by the worker from its own forward (identical weights)
            return batch
        else:
            batch["action_log_probs"] = self._forward_old(self.policy, "policy", batch)
        if batch.get("rollout_logprobs") is not None:
            d = (batch["action_log_probs"] - batch["rollout_logprobs"]).abs()
            mk = batch["loss_mask"]
            denom = mk.sum().clamp(min=1)
            mean = float((d * mk).sum() / denom)
            self.all_metrics["policy/rollout_train_logprobs_abs_diff_mean"] = mean
            self.all_metrics["policy/rollout_train_logprobs_abs_diff_std"] = float(
                ((((d - mean) ** 2) * mk).sum() / denom).sqrt())
        return batch

    def apply_reward_kl_penalty(self, batch: TrainingInputBatch) -> TrainingInputBatch:
        """reward_t -= beta * KL_t (reference: trainer.py:1409-1464)."""
        a = self.cfg.trainer.algorithm
        kl = rl.compute_approx_kl(batch["action_log_probs"], batch["base_action_log_probs"], loss_mask=batch["loss_mask"],
                                  kl_estimator_type=a.kl_estimator_type)
        mk = batch["loss_mask"]
        kl_mean = float(((kl * mk).sum(-1) / mk.sum(-1).clamp(min=1)).mean())
        beta = self.kl_controller.value
        batch["rewards"] = batch["rewards"] - beta * kl
        self.kl_controller.update(kl_mean, n_steps=batch.batch_size)
        self.all_metrics.update({"loss/avg_kl": kl_mean, "loss/avg_kl_max": float(kl.max()), "loss/kl_loss_coef": beta})
        return batch

    def compute_advantages_and_returns(self, batch: TrainingInputBatch) -> TrainingInputBatch:
        a = self.cfg.trainer.algorithm
        uids = np.array(batch.metadata["uids"], dtype=object)
        rew, rmask = batch["rewards"], batch["response_mask"].float()
        last = batch.metadata.get("is_last_step")
        dev = self.env.device if self.env.device.type == "cuda" else torch.device("cpu")
        if last is not None and self.cfg.generator.step_wise_trajectories:
            # step-wise: estimate on the last step of each trajectory, broadcast to its earlier steps
            last_t = torch.tensor(last, dtype=torch.bool)
            tids = batch.metadata.get("trajectory_ids")
            if tids is None:
                # rows of a trajectory are adjacent and end with its last step: number the trajectories by counting the
                # last steps seen before each row
                seen, tids = 0, []
                for is_last in last:
                    tids.append(seen)
                    seen += int(bool(is_last))
            adv_l, ret_l = rl.compute_advantages_and_returns(
                rew[last_t].to(dev), rmask[last_t].to(dev), uids[last_t.numpy()], a.advantage_estimator, a,
                values=batch["values"][last_t].to(dev) if batch.get("values") is not None else None,
                grpo_norm_by_std=a.grpo_norm_by_std, gamma=a.gamma, lambd=a.lambd)
            adv_l, ret_l = adv_l.cpu(), ret_l.cpu()
            scalar = {}
            k = 0
            for i, is_last in enumerate(last):
                if is_last:
                    live = rmask[i] > 0
                    scalar[tids[i]] = (float(adv_l[k][live[-adv_l.shape[1]:]].mean()) if live.any() else 0.0)
                    k += 1
            adv = torch.stack([rmask[i] * scalar.get(tids[i], 0.0) for i in range(len(last))])
            ret = adv.clone()
        else:
            adv, ret = rl.compute_advantages_and_returns(
                rew.to(dev), rmask.to(dev), uids, a.advantage_estimator, a,
                values=batch["values"].to(dev) if batch.get("values") is not None else None,
                grpo_norm_by_std=a.grpo_norm_by_std, gamma=a.gamma, lambd=a.lambd)
            adv, ret = adv.cpu(), ret.cpu()
        batch["advantages"], batch["returns"] = adv, ret
        mk = batch["loss_mask"]
        scores = rew.sum(-1)
        self.all_metrics.update({
            "reward/avg_rewards": float(scores.mean()),
            "loss/avg_advantages": float((adv * mk).sum() / mk.sum().clamp(min=1)),
            "loss/avg_advantages_abs": float((adv.abs() * mk).sum() / mk.sum().clamp(min=1)),
        })
        return batch

    # ------------------------------------------------------------------ training
    def _normalize_advantages(self, mini: TrainingInputBatch, boundaries=None) -> TrainingInputBatch:
        """Optional batch z-score, then bake the loss reduction into the advantages (reference: trainer.py:1467-1507)."""
        a, t = self.cfg.trainer.algorithm, self.cfg.trainer
        adv, mk = mini["advantages"], mini["loss_mask"]
        if a.advantage_batch_normalize:
            n = mk.sum().clamp(min=1)
            mean = (adv * mk).sum() / n
            var = (((adv - mean) ** 2) * mk).sum() / n
            adv = (adv - mean) * torch.rsqrt(var + 1e-8)
        # token counts are global quantities: sum them across the data-parallel ranks.  The ranks of one tensor /
        # sequence / pipeline parallel group hold the same merged batch, so a sum over the world counts every batch
        # ``tp`` times and the number of distinct data shards is ``world / tp``
        W, tp = self.env.world_size, self._data_share()
        if a.loss_reduction == "token_mean":
            tot = mk.sum().double().reshape(1)
            if dist.is_initialized() and W > 1:
                dist.all_reduce(tot)  # host tensor: travels over the gloo side of the process group
                tot = tot / tp
            mini["advantages"] = adv / tot.float().clamp(min=1)
        else:
            scaled = rl.apply_loss_reduction_to_advantages_minibatch(
                adv, mk, a.loss_reduction, t.micro_train_batch_size_per_gpu, a.max_seq_len or adv.shape[1], boundaries)
            mini["advantages"] = scaled / (W // tp)
        return mini

    def _data_share(self) -> int:
        """How many ranks train on the same data shard (the policy's tensor / sequence / pipeline group size)."""
        return int(self.policy.tp_size) if self.policy is not None else 1

    def num_policy_updates_per_step(self) -> int:
        """Optimizer steps per RL step = mini-batches x epochs (reference: trainer.py:777-779)."""
        t = self.cfg.trainer
        return max(1, t.train_batch_size // max(1, t.policy_mini_batch_size)) * t.update_epochs_per_batch

    def _execute_training_step(self, role: str, batch: TrainingInputBatch) -> Dict[str, float]:
        t = self.cfg.trainer
        worker = self.policy if role == "policy" else self.critic
        # this rank's batch holds train_batch_size / dp prompts, dp = number of distinct data shards
        dp = max(1, self.env.world_size // self._data_share())
        mini_prompts = (t.policy_mini_batch_size if role == "policy" else t.critic_mini_batch_size) // dp
        mini_prompts = max(1, mini_prompts)
        uids = batch.metadata["uids"]
        bounds = compute_prompt_mini_batch_boundaries(uids, mini_prompts)
        all_status: List[Dict[str, float]] = []
        for _epoch in range(t.update_epochs_per_batch):
            for (s, e) in bounds:
                mini = batch.slice(s, e)
                mini.metadata = dict(batch.metadata)
                mini.metadata["uids"] = uids[s:e]
                if role == "policy":
                    pb = [(a - s, b - s) for a, b in compute_prompt_boundaries(uids[s:e])]
                    mini = self._normalize_advantages(mini, pb)
                    mini = self._balance_tokens(mini)
                status = worker.forward_backward(mini, **({"step_follows": True} if role == "policy" else {}))
                gn = worker.optim_step()
                if gn is not None:
                    status["grad_norm"] = float(gn)
                all_status.append({k: v for k, v in status.items() if isinstance(v, (int, float))})
        keys = set().union(*[s.keys() for s in all_status]) if all_status else set()
        return {k: float(np.mean([s[k] for s in all_status if k in s])) for k in keys}

    def _balance_tokens(self, mini: TrainingInputBatch) -> TrainingInputBatch:
        """Pure data parallelism: re-deal the mini-batch's rows so that every rank trains on about the same number of
        tokens.  Runs after the loss reduction has been folded into the advantages, so each row carries all that its
        loss term needs and the summed gradient is unchanged."""
        W = self.env.world_size
        if (W <= 1 or not dist.is_initialized() or self._data_share() != 1
                or not getattr(self.cfg.trainer.b200, "balance_tokens_across_ranks", False)
                or getattr(self.policy, "pipe", None) is not None):
            return mini
        from .balance import balance_rows_across_ranks

        out, rep = balance_rows_across_ranks(mini, self.env.rank, W)
        metrics = getattr(self, "all_metrics", None)
        if rep is not None and metrics is not None:
            mean = max(1.0, rep["mean_tokens"])
            metrics["policy/token_imbalance_before"] = rep["max_tokens_before"] / mean
            metrics["policy/token_imbalance_after"] = rep["max_tokens_after"] / mean
        return out

    def train_critic_and_policy(self, batch: TrainingInputBatch) -> Dict[str, float]:
        m: Dict[str, float] = {}
        if self.critic is not None:
            with Timer("critic_train", self.all_timings):
                for k, v in self._execute_training_step("critic", batch).items():
                    m[f"critic/{k}"] = v
        with Timer("policy_train", self.all_timings):
            for k, v in self._execute_training_step("policy", batch).items():
                m[f"policy/{k}"] = v
        return m

    def sync_weights(self) -> None:
        """Make the freshly trained weights visible to the generation engine(s)."""
        c = self.inference_engine_client
        if self.engine is None and self.policy is not None and hasattr(c, "fetch_weights"):
            # stand-alone rollout servers: publish the weights and have every server load them
            from ..weight_sync.remote import RemoteWeightSync

            if getattr(self, "_remote_sync", None) is None:
                ie = self.cfg.generator.inference_engine
                in_box = getattr(self, "rollout_servers_in_box", False) or ie.weight_sync_backend == "peer"
                if ie.weight_sync_backend == "delta":
                    transport = "delta"
                elif in_box and self.env.device.type == "cuda":
                    transport = "peer"  # the servers' GPUs are NVLink peers: push the blocks straight into their buffers
                else:
                    transport = "path"
                sd = getattr(ie.delta_weight_sync, "sync_dir", "") or None
                model = None if transport == "peer" else self.policy.engine_model()
                self._remote_sync = RemoteWeightSync(c, model, transport, sd, is_main=self.env.is_main,
                                                     peer_plan=self.policy.remote_push_plan)
            if self._remote_sync.transport != "peer":
                self.policy.refresh_engine_model()
            asyncio.run(self._remote_sync.sync()) if not self._in_event_loop() else None
            if self._remote_sync.last_push_ms is not None:
                self.all_metrics["timing/weight_sync_kernel_ms"] = float(self._remote_sync.last_push_ms)
            return
        if self.policy is not None:
            self.policy.refresh_engine_model()  # TP shards / LoRA adapters -> the engine's own layout
            ms = getattr(self.policy, "last_weight_sync_ms", None)
            if ms is not None:
                self.all_metrics["timing/weight_sync_kernel_ms"] = float(ms)
        if hasattr(c, "increment_weight_version"):
            c.increment_weight_version()

    def _gather_over_tp(self, out: GeneratorOutput, uids: List[str]):
        """Every rank generated for its own prompts; ranks of one tensor-parallel group train on the same data, so
        they exchange their rollouts and continue with the concatenation (in rank order, identical on each)."""
        import torch.distributed as tdist

        mesh = self.policy.mesh
        parts: List[Any] = [None] * mesh.tp_size
        tdist.all_gather_object(parts, (out, uids), group=mesh.tp_group)
        merged: Dict[str, Any] = {}
        for key in parts[0][0]:
            vals = [p[0].get(key) for p in parts]
            if all(isinstance(v, list) for v in vals):
                merged[key] = [x for v in vals for x in v]
            else:
                merged[key] = vals[mesh.tp_rank]
        return merged, [u for p in parts for u in p[1]]

    @staticmethod
    def _in_event_loop() -> bool:
        try:
            asyncio.get_running_loop()
            return True
        except RuntimeError:
            return False

    async def sync_weights_async(self) -> None:
        """``sync_weights`` for callers already inside an event loop (remote servers need awaited HTTP calls)."""
        c = self.inference_engine_client
        if self.engine is None and self.policy is not None and hasattr(c, "fetch_weights"):
            self.sync_weights()  # builds the helper; the transfer itself is awaited here
            await self._remote_sync.sync()
            if self._remote_sync.last_push_ms is not None:
                self.all_metrics["timing/weight_sync_kernel_ms"] = float(self._remote_sync.last_push_ms)
        else:
            self.sync_weights()

    # ------------------------------------------------------------------ one RL step
    async def train_step_async(self, prompts: List[Dict[str, Any]], prompt_token_ids=None) -> Dict[str, float]:
        cfg = self.cfg
        self.all_metrics, self.all_timings = {}, {}
        t_step = time.time()
        gen_input, uids = prepare_generator_input(prompts, cfg.generator.n_samples_per_prompt, None,
                                                  cfg.environment.env_class, "train", self.global_step, prompt_token_ids)
        with Timer("generate", self.all_timings):
            out = await self.generate(gen_input)
        for w in validate_generator_output(len(gen_input["prompts"]), out, bool(cfg.generator.step_wise_trajectories)):
            logger.warning("generator output: %s", w)
        if self.policy is not None and self.policy.tp_size > 1:
            out, uids = self._gather_over_tp(out, uids)
        if out.get("trajectory_ids") and len(out["response_ids"]) != len(uids):
            uids = [t.instance_id for t in out["trajectory_ids"]]  # step-wise outputs have one row per step
        if cfg.trainer.algorithm.dynamic_sampling.type is not None:
            out, uids, keep_sampling = self.handle_dynamic_sampling(out, uids)
            if keep_sampling:  # not enough informative prompt groups yet: the caller supplies the next prompt batch
                m = dict(self.all_metrics)
                m.update({f"timing/{k}": v for k, v in self.all_timings.items()})
                m["trainer/keep_sampling"] = 1.0
                return m
        with Timer("postprocess", self.all_timings):
            out, uids = self.postprocess_generator_output(out, uids)
            self._log_examples(out, uids)
            batch = self.convert_to_training_input(out, uids)
        with Timer("fwd_logprobs_values_reward", self.all_timings):
            batch = self.fwd_logprobs_values_reward(batch)
        if cfg.trainer.algorithm.use_kl_in_reward and self.ref is not None:
            batch = self.apply_reward_kl_penalty(batch)
        with Timer("compute_advantages_and_returns", self.all_timings):
            batch = self.compute_advantages_and_returns(batch)
        if cfg.trainer.dump_data_batch:
            with Timer("dump_data_batch", self.all_timings):
                self.dump_data(batch, f"global_step_{self.global_step}_training_input")
        with Timer("train_critic_and_policy", self.all_timings):
            self.all_metrics.update(self.train_critic_and_policy(batch))
        with Timer("sync_weights", self.all_timings):
            await self.sync_weights_async()
        n_tokens = int(batch["attention_mask"].sum())
        n_gen = int(batch["response_mask"].sum())
        self.all_timings["step"] = time.time() - t_step
        tt = max(1e-9, self.all_timings.get("train_critic_and_policy", 0.0))
        self.all_metrics["trainer/tokens_per_second_per_gpu"] = n_tokens / tt
        self.all_metrics["trainer/num_tokens"] = float(n_tokens)
        self.all_metrics["trainer/num_generated_tokens"] = float(n_gen)
        self.global_step += 1
        self.all_metrics["trainer/global_step"] = float(self.global_step)
        metrics = dict(self.all_metrics)
        metrics.update({f"timing/{k}": v for k, v in self.all_timings.items()})
        self._last_batch = batch
        return metrics

    def train_step(self, prompts: List[Dict[str, Any]], prompt_token_ids=None) -> Dict[str, float]:
        return asyncio.run(self.train_step_async(prompts, prompt_token_ids))

    # ------------------------------------------------------------------ full loop
    def train(self) -> None:
        asyncio.run(self.train_async())

    async def train_async(self) -> None:
        t = self.cfg.trainer
        assert self.train_dataset is not None, "train() needs a train_dataset"
        self.train_iter = StatefulBatchIterator(self.train_dataset, t.train_batch_size, shuffle=True, seed=t.seed)
        if self.load_checkpoints() > 0:
            await self.sync_weights_async()  # remote servers learn about the restored weights before the first rollout
        if t.eval_before_train and self.eval_dataset is not None and self.global_step == 0:
            self._log(await self.eval_async(), self.global_step)
        total = t.epochs * len(self.train_iter)
        if t.max_training_steps is not None:
            total = min(total, t.max_training_steps)
        self.total_steps, self.steps_per_epoch, self.epoch = total, len(self.train_iter), self.train_iter.epoch
        self.callbacks.fire("on_train_start", self)
        self.policy.start_profile()
        if getattr(t.policy, "record_memory", False):
            self.policy.record_memory_history(True)
        done = False
        while self.train_iter.epoch < t.epochs and not done:
            self.epoch = self.train_iter.epoch
            self.callbacks.fire("on_epoch_start", self)
            for global_batch in self.train_iter:
                self.callbacks.fire("on_step_start", self, batch=global_batch)
                metrics = await self.train_step_async(self._local_prompts(global_batch))
                if metrics.get("trainer/keep_sampling"):
                    continue  # dynamic sampling wants more rollouts before this RL step can train
                ctl = self.callbacks.fire("on_step_end", self, batch=getattr(self, "_last_batch", None), metrics=metrics)
                want_save, want_eval, stop = ctl.should_save, ctl.should_evaluate, ctl.should_stop
                ctl.reset()
                if self.eval_dataset is not None and (want_eval or (t.eval_interval > 0 and self.global_step % t.eval_interval == 0)):
                    self.callbacks.fire("on_eval_start", self)
                    ev = await self.eval_async()
                    metrics.update(ev)
                    self.callbacks.fire("on_eval_end", self, metrics=ev)
                self.callbacks.fire("on_log", self, logs=metrics)
                self._log(metrics, self.global_step)
                self.policy.profile_step()  # one profiler step per RL step
                if want_save or (t.ckpt_interval > 0 and self.global_step % t.ckpt_interval == 0):
                    self.save_checkpoints()
                if t.hf_save_interval > 0 and self.global_step % t.hf_save_interval == 0:
                    self.save_models()
                if self.global_step >= total or stop:
                    done = True
                    break
            self.callbacks.fire("on_epoch_end", self)
            if t.update_ref_every_epoch and self.ref is not None:
                self.update_ref_with_policy()
        if t.ckpt_interval > 0:
            self.save_checkpoints()
        summary = self.policy.stop_profile()
        if summary and self.env.is_main:
            print(summary)
        if getattr(t.policy, "record_memory", False):
            self.policy.dump_memory_snapshot(os.path.join(t.log_path, "memory_snapshots"), f"step{self.global_step}")
        self.callbacks.fire("on_train_end", self)

    def _log_examples(self, out: GeneratorOutput, uids: List[str]) -> None:
        """Rank 0: one decoded example every ``trainer.print_example_interval`` steps (reference: trainer.py:394-403) and
        up to ``trainer.num_logger_train_samples`` trajectories per step as JSONL under ``{log_path}/trajectories`` and
        as a tracker table (reference: trainer.py:405-417; ``-1`` = off)."""
        t = self.cfg.trainer
        if not self.env.is_main or not out.get("response_ids"):
            return
        every = t.print_example_interval
        if every > 0 and self.global_step % every == 0:
            from ..utils.trajectory_logging import TrajectoryLogger

            row = TrajectoryLogger(os.path.join(t.log_path, "trajectories"), self.tokenizer, max_rows=1).rows(out, uids)[0]
            logger.info("step %d example | reward %.3f | stop %s | %d tokens\n--- prompt ---\n%s\n--- response ---\n%s",
                        self.global_step, row["reward"], row["stop_reason"], row["response_length"], row["prompt"],
                        row["response"])
        if t.num_logger_train_samples > 0:
            from ..utils.trajectory_logging import TrajectoryLogger

            TrajectoryLogger(os.path.join(t.log_path, "trajectories"), self.tokenizer, max_rows=t.num_logger_train_samples,
                             tracker=self.tracker).log(out, self.global_step, "train", uids)

    def dump_data(self, batch: TrainingInputBatch, file_name: str) -> str:
        """``trainer.dump_data_batch``: the training batch of this rank, as the byte form that
        ``TrainingInputBatch.from_bytes`` reads back, under ``{export_path}/dumped_data`` (reference: trainer.py:1236-1242)."""
        d = os.path.join(self.cfg.trainer.export_path, "dumped_data")
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, f"{file_name}_rank{self.env.rank}.bin" if self.env.world_size > 1 else f"{file_name}.bin")
        with open(path, "wb") as f:
            f.write(batch.to_bytes())
        return path

    def init_weight_sync_state(self) -> None:
        """Kept for trainer subclasses written against the reference: there is no state to set up here."""
        self.dispatch.init_weight_sync_state(self.inference_engine_client)

    def _log(self, metrics: Dict[str, float], step: int) -> None:
        if self.tracker is not None and self.env.is_main:
            self.tracker.log(metrics, step)

    async def eval_async(self) -> Dict[str, float]:
        from .evaluate import evaluate

        return await evaluate(self.eval_dataset, self.generator, self.cfg, self.global_step, self.tokenizer, self.env,
                              tracker=self.tracker)

    def eval(self) -> Dict[str, float]:
        return asyncio.run(self.eval_async())

    def update_ref_with_policy(self) -> None:
        self.ref.backload()
        self.ref.model.flat_params.copy_(self.policy.model.flat_params)

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoints(self) -> None:
        """``{ckpt_path}/global_step_N/{policy,critic}/`` + ``data.pt`` + ``trainer_state.pt``; pointer written last."""
        t = self.cfg.trainer
        d = os.path.join(t.ckpt_path, f"{tutils.GLOBAL_STEP_PREFIX}{self.global_step}")
        os.makedirs(d, exist_ok=True)
        self.policy.save_checkpoint(os.path.join(d, "policy"), tag=str(self.global_step))
        if self.critic is not None:
            self.critic.save_checkpoint(os.path.join(d, "critic"), tag=str(self.global_step))
        if self.env.is_main:
            if self.train_iter is not None:
                torch.save(self.train_iter.state_dict(), os.path.join(d, "data.pt"))
            torch.save({"global_step": self.global_step, "config": self.cfg.to_dict()}, os.path.join(d, "trainer_state.pt"))
        if dist.is_initialized():
            dist.barrier()
        if self.env.is_main:
            tutils.write_latest(t.ckpt_path, self.global_step)
            tutils.cleanup_old_checkpoints(t.ckpt_path, t.max_ckpts_to_keep, self.global_step)
        self.callbacks.fire("on_save", self, ckpt_path=d)

    def load_checkpoints(self) -> int:
        d = tutils.resolve_resume_path(self.cfg.trainer)
        if d is None:
            return 0
        state = torch.load(os.path.join(d, "trainer_state.pt"), weights_only=False)
        step_from_dir = int(os.path.basename(os.path.normpath(d))[len(tutils.GLOBAL_STEP_PREFIX):])
        if state["global_step"] != step_from_dir:
            raise ValueError(f"checkpoint {d} is inconsistent: trainer_state says step {state['global_step']}")
        self.policy.load_checkpoint(os.path.join(d, "policy"))
        if self.critic is not None and os.path.isdir(os.path.join(d, "critic")):
            self.critic.load_checkpoint(os.path.join(d, "critic"))
        if self.train_iter is not None and os.path.exists(os.path.join(d, "data.pt")):
            self.train_iter.load_state_dict(torch.load(os.path.join(d, "data.pt"), weights_only=False))
        self.global_step = int(state["global_step"])
        self.sync_weights()
        return self.global_step

    def save_models(self) -> None:
        d = os.path.join(self.cfg.trainer.export_path, f"{tutils.GLOBAL_STEP_PREFIX}{self.global_step}", "policy")
        self.policy.save_hf_model(d, self.tokenizer)


# familiar name for users of the reference
RayPPOTrainer = PPOTrainer
