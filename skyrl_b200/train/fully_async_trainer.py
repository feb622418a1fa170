"""Fully asynchronous RL: generation never waits for training.

``W`` generation workers (coroutines, one prompt group each) feed a bounded queue; the trainer consumes
mini-batches of ``B`` groups, updates the policy, pushes weights to the rollout engines *while requests are in
flight* (pause-keep -> transfer -> resume) and raises the admission capacity.  Staleness is bounded by admission
control, not by discarding data.  Behavioural reference: skyrl/train/fully_async_trainer.py
(``_AsyncStalenessManager`` :115-234 with the capacity rule :181-187, ``_AsyncDataloader`` :237-326, loop
:432-732, checkpoint extras :1151-1202, constraints :353-404).
"""

from __future__ import annotations

import asyncio
import os
import time
from typing import Any, Dict, List, Optional, Set

import numpy as np
import torch

from . import utils as tutils
from .batch import TrainingInputBatch
from .generators.utils import concatenate_generator_outputs, prepare_generator_input
from .trainer import PPOTrainer
from .utils import Timer


class AsyncStalenessManager:
    """Admission control.  A new rollout may start iff

        capacity = min(W - running, (S + current_step) * B - (accepted + running)) > 0

    with W generation workers, S = max_staleness_steps, B = mini-batch size in prompt groups.  Invariant:
    ``submitted == accepted + filtered + running``.
    """

    def __init__(self, max_workers: int, max_staleness_steps: int, mini_batch_size: int):
        self.W, self.S, self.B = max_workers, max_staleness_steps, mini_batch_size
        self.current_step = 1
        self.submitted = self.accepted = self.filtered = self.running = 0
        self._cond = asyncio.Condition()

    def capacity(self) -> int:
        return min(self.W - self.running, (self.S + self.current_step) * self.B - (self.accepted + self.running))

    def check_invariant(self) -> None:
        assert self.submitted == self.accepted + self.filtered + self.running, (
            f"staleness accounting broken: submitted={self.submitted} accepted={self.accepted} "
            f"filtered={self.filtered} running={self.running}")

    async def acquire_submission_slot(self) -> None:
        async with self._cond:
            await self._cond.wait_for(lambda: self.capacity() > 0)
            self.running += 1
            self.submitted += 1

    async def on_rollout_accepted(self) -> None:
        async with self._cond:
            self.running -= 1
            self.accepted += 1
            self._cond.notify_all()

    async def on_rollout_filtered(self) -> None:
        """A finished rollout that will not be trained on (e.g. zero-variance group) frees its budget."""
        async with self._cond:
            self.running -= 1
            self.filtered += 1
            self._cond.notify_all()

    async def on_rollout_cancelled(self) -> None:
        async with self._cond:
            self.running -= 1
            self.submitted -= 1
            self._cond.notify_all()

    async def notify_capacity_change(self, new_step: int) -> None:
        async with self._cond:
            self.current_step = new_step
            self._cond.notify_all()

    def state_dict(self) -> Dict[str, int]:
        return {"current_step": self.current_step, "accepted": self.accepted, "filtered": self.filtered}

    def load_state_dict(self, sd: Dict[str, int]) -> None:
        self.current_step = sd["current_step"]
        # in-flight rollouts of the previous run are lost: restart the accounting from what was consumed
        self.accepted, self.filtered = sd["accepted"], sd["filtered"]
        self.submitted, self.running = self.accepted + self.filtered, 0


class AsyncDataloader:
    """Shared prompt iterator for the generation workers: one item at a time under a lock, skipping uids that
    were already consumed before a restart; epochs roll over transparently."""

    def __init__(self, dataset, seed: int = 42, epochs: int = 1, consumed_uids: Optional[Set[str]] = None,
                 rank: int = 0, world: int = 1):
        """``rank`` / ``world``: every training rank feeds its own generation workers from a disjoint slice of each
        epoch's permutation (the permutation itself is the same on all ranks)."""
        self.ds, self.seed, self.epochs = dataset, seed, epochs
        self.rank, self.world = rank, max(1, world)
        self.epoch = 0
        self.consumed: Set[str] = set(consumed_uids or ())
        self._order = self._make_order()
        self._pos = 0
        self._lock = asyncio.Lock()

    def _make_order(self) -> np.ndarray:
        idx = np.arange(len(self.ds))
        np.random.default_rng(self.seed + self.epoch).shuffle(idx)
        return idx[self.rank :: self.world]

    def epoch_uid(self, uid: str) -> str:
        return f"{self.epoch}:{uid}"

    async def next(self) -> Optional[Dict[str, Any]]:
        async with self._lock:
            while True:
                if self._pos >= len(self._order):
                    self.epoch += 1
                    if self.epoch >= self.epochs:
                        return None
                    self._order, self._pos = self._make_order(), 0
                item = self.ds[int(self._order[self._pos])]
                self._pos += 1
                key = self.epoch_uid(item["uid"])
                if key in self.consumed:
                    continue
                out = dict(item)
                out["_consumed_key"] = key
                return out


class FullyAsyncPPOTrainer(PPOTrainer):
    def __init__(self, *args, weight_transfer=None, **kwargs):
        """``weight_transfer``: callable run between pause and resume that moves the new weights to the engines."""
        super().__init__(*args, **kwargs)
        fa = self.cfg.trainer.fully_async
        self.B = max(1, self.cfg.trainer.policy_mini_batch_size // self.env.world_size)
        self.W = fa.num_parallel_generation_workers
        self.S = fa.max_staleness_steps
        if not (self.B <= self.W <= self.B * (self.S + 1)):
            raise ValueError(f"num_parallel_generation_workers ({self.W}) must lie in [{self.B}, {self.B * (self.S + 1)}]")
        self.staleness = AsyncStalenessManager(self.W, self.S, self.B)
        self.weight_transfer = weight_transfer
        self.consumed_uids: Set[str] = set()
        self.filtered_uids: Set[str] = set()
        self._queue: Optional[asyncio.Queue] = None
        self._stop = False
        self.async_metrics: Dict[str, float] = {}

    # ------------------------------------------------------------------ generation side
    async def _generation_worker(self, loader: AsyncDataloader) -> None:
        g = self.cfg.generator
        while not self._stop:
            await self.staleness.acquire_submission_slot()
            item = None
            try:
                item = await loader.next()
                if item is None or self._stop:
                    await self.staleness.on_rollout_cancelled()
                    return
                gi, uids = prepare_generator_input([item], g.n_samples_per_prompt, None, self.cfg.environment.env_class,
                                                   "train", self.global_step)
                t0 = time.monotonic()
                out = await self.generator.generate(gi)
                group = {"out": out, "uids": uids, "key": item["_consumed_key"], "gen_time": time.monotonic() - t0,
                         "weight_version_start": getattr(self.inference_engine_client, "weight_version", 0),
                         "step_at_submit": self.staleness.current_step}
                if self.cfg.trainer.fully_async.sample_full_batch and self._zero_variance(out):
                    self.filtered_uids.add(item["_consumed_key"])
                    await self.staleness.on_rollout_filtered()
                    continue
                await self._queue.put(group)
                await self.staleness.on_rollout_accepted()
            except asyncio.CancelledError:
                await self.staleness.on_rollout_cancelled()
                return
            except Exception:
                # a crashed generation worker must not leave the trainer waiting for ever on a short batch
                self._stop = True
                self._worker_error = True
                await self.staleness.on_rollout_cancelled()
                raise

    def _zero_variance(self, out) -> bool:
        """All *live* trajectories of the group (those with a non-zero loss mask) earned the same total reward, within
        the tolerance: nothing to learn from.  A single live trajectory is kept (reference: fully_async_trainer.py
        ``_should_keep_group``)."""
        masks = out.get("loss_masks") or [[1]] * len(out["rewards"])
        scores = [float(np.sum(r)) if isinstance(r, (list, tuple)) else float(r)
                  for r, m in zip(out["rewards"], masks) if any(m)]
        return len(scores) > 1 and (max(scores) - min(scores)) <= self.cfg.trainer.algorithm.zero_variance_filter_tol

    async def _collect_mini_batch(self) -> Optional[List[Dict[str, Any]]]:
        groups = []
        while len(groups) < self.B:
            if self._stop and self._queue.empty():
                return None
            try:
                groups.append(await asyncio.wait_for(self._queue.get(), timeout=0.05))
            except asyncio.TimeoutError:
                if all(t.done() for t in self._workers) and self._queue.empty():
                    return None if not groups else None
        return groups

    def convert_groups_to_training_input(self, groups: List[Dict[str, Any]]) -> TrainingInputBatch:
        if self.policy is not None and self.policy.tp_size > 1:
            # ranks of one tensor / sequence parallel group train on one batch: the union of what each collected
            import torch.distributed as dist

            parts: List[Any] = [None] * self.policy.mesh.tp_size
            dist.all_gather_object(parts, groups, group=self.policy.mesh.tp_group)
            groups = [g for p in parts for g in p]
        out = concatenate_generator_outputs([g["out"] for g in groups])
        uids = [u for g in groups for u in g["uids"]]
        out, uids = self.postprocess_generator_output(out, uids)
        batch = self.convert_to_training_input(out, uids)
        stale = [self.staleness.current_step - g["step_at_submit"] for g in groups]
        self.all_metrics.update({"async/staleness_mean": float(np.mean(stale)), "async/staleness_max": float(max(stale)),
                                 "async/group_gen_time_mean": float(np.mean([g["gen_time"] for g in groups])),
                                 "async/queue_depth": float(self._queue.qsize())})
        return batch

    # ------------------------------------------------------------------ trainer side
    def _train_on_batch(self, batch: TrainingInputBatch) -> Dict[str, float]:
        batch = self.fwd_logprobs_values_reward(batch)
        if self.cfg.trainer.algorithm.use_kl_in_reward and self.ref is not None:
            batch = self.apply_reward_kl_penalty(batch)
        batch = self.compute_advantages_and_returns(batch)
        return self.train_critic_and_policy(batch)

    async def sync_weights_in_flight(self) -> None:
        """pause(keep) -> transfer -> resume; in-flight requests continue on the new weights."""
        c = self.inference_engine_client
        if self.weight_transfer is None and self.engine is None and hasattr(c, "fetch_weights"):
            # stand-alone rollout servers (other ranks of this launch, or another machine): the remote sync helper
            # pauses them with their requests kept, moves the weights (peer push / delta / export) and resumes them
            await self.sync_weights_async()
            return
        await c.pause("keep", clear_cache=self.cfg.trainer.fully_async.clear_kv_cache_on_weight_sync)
        try:
            if self.weight_transfer is not None:
                await asyncio.to_thread(self.weight_transfer)
            if hasattr(c, "increment_weight_version"):
                c.increment_weight_version()
        finally:
            await c.resume()  # generation must restart even when the transfer failed

    async def train_async(self) -> None:
        t = self.cfg.trainer
        assert self.train_dataset is not None
        self.load_checkpoints()
        loader = AsyncDataloader(self.train_dataset, seed=t.seed, epochs=t.epochs, consumed_uids=self.consumed_uids,
                                 rank=self.env.rank, world=self.env.world_size)
        self._queue = asyncio.Queue(maxsize=self.B * (self.S + 1))
        self._stop, self._worker_error = False, False
        self._workers = [asyncio.create_task(self._generation_worker(loader)) for _ in range(self.W)]
        max_steps = t.max_training_steps
        try:
            while True:
                self.all_metrics, self.all_timings = {}, {}
                with Timer("wait_for_generation_buffer", self.all_timings):
                    groups = await self._collect_mini_batch()
                if groups is None:
                    break
                with Timer("convert_to_training_input", self.all_timings):
                    batch = await asyncio.to_thread(self.convert_groups_to_training_input, groups)
                with Timer("train_critic_and_policy", self.all_timings):
                    self.all_metrics.update(await asyncio.to_thread(self._train_on_batch, batch))
                with Timer("sync_weights", self.all_timings):
                    await self.sync_weights_in_flight()
                for g in groups:
                    self.consumed_uids.add(g["key"])
                self.all_metrics["trainer/num_tokens"] = float(batch["attention_mask"].sum())
                self.all_metrics["trainer/num_generated_tokens"] = float(batch["loss_mask"].sum())
                self.global_step += 1
                await self.staleness.notify_capacity_change(self.global_step + 1)
                self.staleness.check_invariant()
                metrics = dict(self.all_metrics)
                metrics.update({f"timing/{k}": v for k, v in self.all_timings.items()})
                metrics["trainer/global_step"] = float(self.global_step)
                ctl = self.callbacks.fire("on_step_end", self, metrics=metrics)
                want_save = ctl.should_save
                ctl.reset()
                self.callbacks.fire("on_log", self, logs=metrics)
                self._log(metrics, self.global_step)
                if want_save and not (t.ckpt_interval > 0 and self.global_step % t.ckpt_interval == 0):
                    self.save_checkpoints()
                if t.ckpt_interval > 0 and self.global_step % t.ckpt_interval == 0:
                    self.save_checkpoints()
                if max_steps is not None and self.global_step >= max_steps:
                    break
        finally:
            self._stop = True
            for w in self._workers:
                w.cancel()
            res = await asyncio.gather(*self._workers, return_exceptions=True)
            errs = [r for r in res if isinstance(r, Exception) and not isinstance(r, asyncio.CancelledError)]
            if errs:
                raise errs[0]

    # ------------------------------------------------------------------ checkpoint extras
    def save_checkpoints(self) -> None:
        super().save_checkpoints()
        if self.env.is_main:
            d = os.path.join(self.cfg.trainer.ckpt_path, f"{tutils.GLOBAL_STEP_PREFIX}{self.global_step}")
            torch.save({"consumed_uids": sorted(self.consumed_uids), "filtered_uids": sorted(self.filtered_uids),
                        "staleness": self.staleness.state_dict()}, os.path.join(d, "fully_async_state.pt"))

    def load_checkpoints(self) -> int:
        step = super().load_checkpoints()
        d = tutils.resolve_resume_path(self.cfg.trainer)
        if d is not None and os.path.exists(os.path.join(d, "fully_async_state.pt")):
            st = torch.load(os.path.join(d, "fully_async_state.pt"), weights_only=False)
            self.consumed_uids, self.filtered_uids = set(st["consumed_uids"]), set(st["filtered_uids"])
            self.staleness.load_state_dict(st["staleness"])
        return step


class FullyAsyncTrainerSim(FullyAsyncPPOTrainer):
    """No model: 'training' sleeps for ``simulate_training_step_seconds`` and weight sync for
    ``simulate_weight_sync_seconds`` -- measures what the rollout side alone can deliver
    (reference: skyrl/train/fully_async_trainer_sim.py:21-117)."""

    def build_models(self, *a, **k) -> None:
        from .generators.skyrl_gym_generator import SkyRLGymGenerator

        if self.generator is None:
            self.generator = SkyRLGymGenerator(self.cfg.generator, self.cfg.environment.skyrl_gym,
                                               self.inference_engine_client, self.tokenizer)

    def _train_on_batch(self, batch):
        time.sleep(self.cfg.trainer.fully_async.simulate_training_step_seconds)
        return {"sim/trained_tokens": float(batch["attention_mask"].sum())}

    async def sync_weights_in_flight(self) -> None:
        c = self.inference_engine_client
        await c.pause("keep")
        try:
            await asyncio.sleep(self.cfg.trainer.fully_async.simulate_weight_sync_seconds)
            if hasattr(c, "increment_weight_version"):
                c.increment_weight_version()
        finally:
            await c.resume()

    def save_checkpoints(self) -> None:
        return None

    def load_checkpoints(self) -> int:
        return 0
