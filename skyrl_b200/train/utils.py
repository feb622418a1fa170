"""Trainer utilities: timers, config validation, checkpoint bookkeeping.

``Timer`` names are public metric names (``timing/<name>``), as in the reference
(skyrl/train/utils/utils.py:32-56).  ``validate_cfg`` re-implements the cross-field checks of
``validate_cfg`` / ``validate_batch_sizes`` (skyrl/train/utils/utils.py:58-478) for the process model
used here (SPMD ranks instead of Ray actor groups).
"""

from __future__ import annotations

import math
import os
import shutil
import time
from typing import Dict, List, Optional

import torch

from ..algorithms import rl

GLOBAL_STEP_PREFIX = "global_step_"
LATEST_FILE = "latest_ckpt_global_step.txt"


class Timer:
    """``with Timer("generate", timings): ...`` accumulates wall-clock seconds into ``timings[name]``."""

    def __init__(self, name: str, store: Optional[Dict[str, float]] = None, sync_cuda: bool = False):
        self.name, self.store, self.sync = name, store, sync_cuda

    def __enter__(self):
        if self.sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        self.t0 = time.time()
        return self

    def __exit__(self, *exc):
        if self.sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        self.elapsed = time.time() - self.t0
        if self.store is not None:
            self.store[self.name] = self.store.get(self.name, 0.0) + self.elapsed
        return False

    async def __aenter__(self):
        return self.__enter__()

    async def __aexit__(self, *exc):
        return self.__exit__(*exc)


class CudaTimer:
    """Device-side duration in milliseconds measured with CUDA events on the current stream."""

    def __init__(self, device=None):
        self.device = device
        self.enabled = torch.cuda.is_available()

    def __enter__(self):
        if self.enabled:
            self.s, self.e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.s.record()
        else:
            self.t0 = time.time()
        return self

    def __exit__(self, *exc):
        if self.enabled:
            self.e.record()
            self.e.synchronize()
            self.elapsed_ms = self.s.elapsed_time(self.e)
        else:
            self.elapsed_ms = (time.time() - self.t0) * 1e3
        return False


def dp_sizes(cfg, world_size: int) -> Dict[str, int]:
    t = cfg.trainer
    if t.strategy == "megatron":
        m = t.policy.megatron_config
        denom = m.tensor_model_parallel_size * m.pipeline_model_parallel_size * m.context_parallel_size
    else:
        denom = t.policy.sequence_parallel_size
    if world_size % denom != 0:
        raise ValueError(f"world size {world_size} is not divisible by the model-parallel size {denom}")
    return {"policy": world_size // denom, "ref": world_size // max(1, t.ref.sequence_parallel_size),
            "critic": world_size // max(1, t.critic.sequence_parallel_size)}


def validate_batch_sizes(cfg, world_size: int) -> None:
    t, g = cfg.trainer, cfg.generator
    n = g.n_samples_per_prompt
    dp = dp_sizes(cfg, world_size)
    if t.train_batch_size < t.policy_mini_batch_size:
        raise ValueError(f"train_batch_size ({t.train_batch_size}) must be >= policy_mini_batch_size "
                         f"({t.policy_mini_batch_size})")
    if t.train_batch_size % t.policy_mini_batch_size != 0:
        raise ValueError("train_batch_size must be divisible by policy_mini_batch_size")
    for role, mini in (("policy", t.policy_mini_batch_size), ("critic", t.critic_mini_batch_size)):
        if role == "critic" and t.critic.model.path is None:
            continue
        per_gpu = mini * n // dp[role]
        if mini * n % dp[role] != 0 or per_gpu <= 0:
            raise ValueError(f"{role}_mini_batch_size * n_samples_per_prompt ({mini}*{n}) must be a positive multiple "
                             f"of the data-parallel size {dp[role]}")
        if t.max_tokens_per_microbatch <= 0 and per_gpu % t.micro_train_batch_size_per_gpu != 0:
            raise ValueError(f"{role} mini-batch per GPU ({per_gpu}) must be divisible by "
                             f"micro_train_batch_size_per_gpu ({t.micro_train_batch_size_per_gpu})")
        train_per_gpu = t.train_batch_size * n // dp[role]
        if train_per_gpu % per_gpu != 0:
            raise ValueError(f"{role}: per-GPU train batch ({train_per_gpu}) must be divisible by the per-GPU "
                             f"mini-batch ({per_gpu})")
    lcm = math.lcm(dp["policy"], dp["ref"])
    if t.train_batch_size * n < lcm:
        raise ValueError(f"train_batch_size * n_samples_per_prompt must be >= lcm(dp_policy, dp_ref) = {lcm}")


def validate_cfg(cfg, world_size: int = 1) -> None:
    t, g, a = cfg.trainer, cfg.generator, cfg.trainer.algorithm
    if t.strategy == "fsdp2":
        t.strategy = "fsdp"
    if t.strategy not in ("fsdp", "megatron"):
        raise ValueError(f"unknown trainer.strategy '{t.strategy}' (expected fsdp or megatron)")
    if t.sequence_parallel_backend not in ("ulysses", "context"):
        raise ValueError("sequence_parallel_backend must be 'ulysses' (heads exchanged by all-to-all) or 'context' "
                         "(keys / values all-gathered: context parallelism)")
    if a.advantage_estimator not in rl.AdvantageEstimatorRegistry.list_available():
        raise ValueError(f"unknown advantage_estimator '{a.advantage_estimator}'; available: "
                         f"{rl.AdvantageEstimatorRegistry.list_available()}")
    if a.policy_loss_type not in rl.PolicyLossRegistry.list_available():
        raise ValueError(f"unknown policy_loss_type '{a.policy_loss_type}'; available: "
                         f"{rl.PolicyLossRegistry.list_available()}")
    if a.loss_reduction not in ("token_mean", "token_mean_legacy", "sequence_mean", "seq_mean_token_sum_norm", "prompt_mean"):
        raise ValueError(f"invalid loss_reduction '{a.loss_reduction}'")
    if a.kl_estimator_type not in ("k1", "abs", "k2", "k3"):
        raise ValueError(f"invalid kl_estimator_type '{a.kl_estimator_type}'")
    if a.use_kl_in_reward and a.use_kl_loss:
        raise ValueError("use_kl_in_reward and use_kl_loss are mutually exclusive")
    if t.max_training_steps is not None and t.max_training_steps <= 0:
        raise ValueError(f"max_training_steps must be > 0, got {t.max_training_steps}")
    lp = g.sampling_params.logprobs
    if lp is not None and (isinstance(lp, bool) or not isinstance(lp, int) or lp > 1 or lp < 0):
        raise ValueError(f"`logprobs` if set should be 0 or 1 (both return only the chosen token's logprob), got {lp!r}")
    if g.max_input_length is not None and g.max_input_length < t.max_prompt_length:
        raise ValueError(f"generator.max_input_length ({g.max_input_length}) must be at least trainer.max_prompt_length "
                         f"({t.max_prompt_length})")
    for name, sp in (("sampling_params", g.sampling_params), ("eval_sampling_params", g.eval_sampling_params)):
        if sp is not None and float(sp.repetition_penalty) != 1.0:
            raise ValueError(f"generator.{name}.repetition_penalty={sp.repetition_penalty}: the built-in engine applies no "
                             "repetition penalty; leave it at 1.0")
    ie = g.inference_engine
    for key in ("pipeline_parallel_size", "expert_parallel_size"):
        if int(getattr(ie, key) or 1) != 1:
            raise ValueError(f"generator.inference_engine.{key}={getattr(ie, key)}: the built-in engine shards by tensor "
                             "parallelism only (tensor_parallel_size); use more engines for more throughput")
    if int(ie.data_parallel_size or 1) != 1:
        raise ValueError("generator.inference_engine.data_parallel_size: engine replicas are counted by num_engines here "
                         "(one per GPU when colocated); leave data_parallel_size at 1")
    if ie.enable_pd or int(ie.num_prefill or 0) > 0:
        raise ValueError("prefill/decode disaggregation (enable_pd, num_prefill) is not available")
    if t.mtp.enabled and t.mtp.num_speculative_tokens < 1:
        raise ValueError("trainer.mtp.num_speculative_tokens must be >= 1 when trainer.mtp.enabled")
    if t.update_epochs_per_batch < 1:
        raise ValueError("trainer.update_epochs_per_batch must be >= 1")
    if g.n_samples_per_prompt < 1 or g.eval_n_samples_per_prompt < 1:
        raise ValueError("generator.n_samples_per_prompt and eval_n_samples_per_prompt must be >= 1")
    if a.advantage_estimator == "gae" and t.critic.model.path is None:
        raise ValueError("advantage_estimator='gae' needs a critic: set trainer.critic.model.path")
    if a.use_tis:
        raise ValueError("`use_tis` was replaced by trainer.algorithm.off_policy_correction.tis_ratio_type")
    oc = a.off_policy_correction
    if oc.tis_ratio_type not in (None, "token", "sequence"):
        raise ValueError(f"invalid tis_ratio_type '{oc.tis_ratio_type}'")
    if oc.sequence_mask_metric not in (None, "geometric", "product"):
        raise ValueError(f"invalid sequence_mask_metric '{oc.sequence_mask_metric}'")
    if a.dynamic_sampling.type not in (None, "filter", "replace"):
        raise ValueError(f"invalid dynamic_sampling.type '{a.dynamic_sampling.type}'")
    if g.step_wise_trajectories and g.batched:
        raise ValueError("step_wise_trajectories requires the non-batched generator")
    for node in (t.policy, t.critic, t.ref):
        prof = getattr(node, "torch_profiler_config", None)
        if prof is not None:
            prof.validate()
    if t.policy.megatron_config.moe_enable_routing_replay and not g.inference_engine.enable_return_routed_experts:
        raise ValueError("rollout router replay needs generator.inference_engine.enable_return_routed_experts=true")
    if g.inference_engine.enable_return_routed_experts and g.step_wise_trajectories:
        raise ValueError("step_wise_trajectories does not support enable_return_routed_experts=true")
    if g.max_turns > 1 and g.batched:
        raise ValueError("generator.batched=true only supports max_turns=1")
    if t.fully_async.enabled:
        if t.placement.colocate_all:
            raise ValueError("fully-async training needs disjoint trainer and rollout GPUs (placement.colocate_all=false)")
        ok_losses = {"rollout_is", "dppo"}
        if not (a.policy_loss_type in ok_losses or (a.policy_loss_type == "cispo" and a.cispo.cispo_anchor == "rollout")
                or oc.tis_ratio_type is not None):
            raise ValueError("fully-async training needs a rollout-anchored objective: policy_loss_type in "
                             "{rollout_is, dppo}, cispo with cispo_anchor=rollout, or a TIS off-policy correction")
        fa = t.fully_async
        B = t.policy_mini_batch_size
        if not (B <= fa.num_parallel_generation_workers <= B * (fa.max_staleness_steps + 1)):
            raise ValueError("fully_async.num_parallel_generation_workers must lie in "
                             f"[{B}, {B * (fa.max_staleness_steps + 1)}] (mini-batch size .. mini-batch * (staleness+1))")
    validate_parallel_cfg(cfg, world_size)
    validate_batch_sizes(cfg, world_size)


def validate_parallel_cfg(cfg, world_size: int = 1) -> None:
    """Model-parallel settings that this build supports (reference: validate_megatron_cfg, train/utils/utils.py:194-232)."""
    t = cfg.trainer
    mc = t.policy.megatron_config
    tp, pp, cp, ep = (int(getattr(mc, k, 1) or 1) for k in ("tensor_model_parallel_size", "pipeline_model_parallel_size",
                                                              "context_parallel_size", "expert_model_parallel_size"))
    sp = int(t.policy.sequence_parallel_size or 1)
    if t.strategy != "megatron":
        if max(tp, pp, cp, ep) > 1:
            raise ValueError("tensor / pipeline / context / expert parallel sizes need trainer.strategy=megatron")
    else:
        if sp > 1:
            raise ValueError("policy.sequence_parallel_size (Ulysses) belongs to strategy=fsdp; with strategy=megatron "
                             "sequence parallelism is implied by tensor_model_parallel_size > 1")
        if pp > 1 and (tp > 1 or ep > 1):
            raise ValueError("pipeline parallelism cannot be combined with tensor or expert parallelism in this build")
        if cp > 1 and max(tp, pp, ep) > 1:
            raise ValueError("context parallelism cannot be combined with tensor, pipeline or expert parallelism in this build")
        if tp > 1 and ep > 1:
            raise ValueError("tensor and expert parallelism cannot be combined in this build")
        if t.policy.model.lora.rank > 0 and (tp > 1 or ep > 1 or pp > 1):
            raise ValueError("LoRA is supported with the data-parallel strategy only")
    for name, size in (("tensor_model_parallel_size", tp), ("expert_model_parallel_size", ep),
                       ("pipeline_model_parallel_size", pp), ("policy.sequence_parallel_size", sp),
                       ("context_parallel_size", cp)):
        if size > 1 and world_size % size != 0:
            raise ValueError(f"{name}={size} does not divide the number of ranks ({world_size})")
        if size > 8:
            raise ValueError(f"{name}={size}: model-parallel groups span at most the 8 GPUs of one NVSwitch domain")
    if sp > 1 and t.policy.model.lora.rank > 0:
        raise ValueError("LoRA together with sequence parallelism is not supported")


# ----------------------------------------------------------------------------- checkpoints
def list_checkpoint_steps(ckpt_path: str) -> List[int]:
    if not os.path.isdir(ckpt_path):
        return []
    out = []
    for d in os.listdir(ckpt_path):
        if d.startswith(GLOBAL_STEP_PREFIX) and d[len(GLOBAL_STEP_PREFIX):].isdigit():
            out.append(int(d[len(GLOBAL_STEP_PREFIX):]))
    return sorted(out)


def cleanup_old_checkpoints(ckpt_path: str, max_to_keep: int, current_step: int) -> None:
    """Keep the newest ``max_to_keep`` step directories (reference: trainer_utils.py:154-190)."""
    if max_to_keep is None or max_to_keep < 0:
        return
    steps = [s for s in list_checkpoint_steps(ckpt_path) if s <= current_step]
    for s in steps[: max(0, len(steps) - max_to_keep)]:
        shutil.rmtree(os.path.join(ckpt_path, f"{GLOBAL_STEP_PREFIX}{s}"), ignore_errors=True)


def write_latest(ckpt_path: str, step: int) -> None:
    """The pointer file is written last and atomically, so a crash never leaves it ahead of the data."""
    tmp = os.path.join(ckpt_path, LATEST_FILE + ".tmp")
    with open(tmp, "w") as f:
        f.write(str(step))
    os.replace(tmp, os.path.join(ckpt_path, LATEST_FILE))


def resolve_resume_path(cfg_trainer) -> Optional[str]:
    """``none`` | ``latest`` | ``from_path`` -> checkpoint directory or None (reference: trainer.py:1722-1833)."""
    mode = (cfg_trainer.resume_mode or "none").lower()
    if mode == "none":
        return None
    if mode == "latest":
        p = os.path.join(cfg_trainer.ckpt_path, LATEST_FILE)
        if not os.path.exists(p):
            return None
        step = int(open(p).read().strip())
        d = os.path.join(cfg_trainer.ckpt_path, f"{GLOBAL_STEP_PREFIX}{step}")
        if not os.path.isdir(d):
            raise FileNotFoundError(f"{LATEST_FILE} points at step {step} but {d} does not exist")
        return d
    if mode == "from_path":
        d = cfg_trainer.resume_path
        if not d or not os.path.isdir(d):
            raise FileNotFoundError(f"resume_path '{d}' does not exist")
        if not os.path.basename(os.path.normpath(d)).startswith(GLOBAL_STEP_PREFIX):
            raise ValueError(f"resume_path must be a '{GLOBAL_STEP_PREFIX}N' directory, got '{d}'")
        return d
    raise ValueError(f"invalid resume_mode '{cfg_trainer.resume_mode}'")
