"""One-step-off-policy trainer: rollouts for batch ``k+1`` are generated while batch ``k`` is trained on.

Reference: examples/train/async/async_trainer.py:19-200 (``AsyncRayPPOTrainer``: an ``asyncio.Queue(maxsize=1)``
between a generation task and the training loop, weight sync between steps gated by two events).  The same protocol
is kept; what differs is where the two halves run.  The reference needs disjoint GPU sets for trainer and rollout
engines (``colocate_all`` must be false).  Here both share each GPU: the engine generates from its *own copy* of the
weights (refreshed between steps, which is the weight sync), so the optimizer may update the training parameters while
decode kernels of the next batch are in flight on another stream; training runs in a worker thread so the event loop
keeps scheduling engine steps.
"""

from __future__ import annotations

import asyncio
from typing import Any, Dict, List, Optional

import torch

from ..models.decoder import CausalLM
from .generators.utils import prepare_generator_input
from .trainer import PPOTrainer
from .utils import Timer
from .dataset import StatefulBatchIterator


class OneStepOffPPOTrainer(PPOTrainer):
    def build_models(self, policy_model=None, peer_ctx=None) -> None:
        super().build_models(policy_model, peer_ctx)
        eng = self.engine
        if eng is not None and eng.model is self.policy.model:
            # give the engine a private copy so that in-place optimizer updates never race with decoding
            m = self.policy.model
            copy = CausalLM(m.args, device=self.env.device, dtype=m.flat_params.dtype, seed=None)
            copy.flat_params.copy_(m.flat_params)
            self.policy._engine_copy = copy
            self.engine = self._build_engine(copy)
            self.inference_engine_client.engines = [self.engine]
            del eng

    def sync_weights(self) -> None:
        m, ec = self.policy.model, getattr(self.policy, "_engine_copy", None)
        if ec is not None and ec.flat_params.numel() == m.flat_params.numel() and not hasattr(m, "lora_rank") \
                and self.policy.mesh is None:
            ec.flat_params.copy_(m.flat_params)
            c = self.inference_engine_client
            if hasattr(c, "increment_weight_version"):
                c.increment_weight_version()
            return
        super().sync_weights()

    async def _generate_loop(self, it, buffer: asyncio.Queue, sync_finished: asyncio.Event, ack: asyncio.Event,
                             n_batches: int) -> None:
        cfg = self.cfg
        for k, global_batch in enumerate(it):
            if k >= n_batches:
                break
            prompts = self._local_prompts(global_batch)
            gi, uids = prepare_generator_input(prompts, cfg.generator.n_samples_per_prompt, None, cfg.environment.env_class,
                                               "train", self.global_step)
            out = await self.generate(gi)
            await buffer.put((out, uids))  # blocks while the previous batch has not been taken
            ack.set()  # the engine is idle: weights may be swapped now
            await sync_finished.wait()
            sync_finished.clear()
        await buffer.put(None)

    def _train_on(self, out, uids) -> Dict[str, float]:
        out, uids = self.postprocess_generator_output(out, uids)
        batch = self.convert_to_training_input(out, uids)
        batch = self.fwd_logprobs_values_reward(batch)
        if self.cfg.trainer.algorithm.use_kl_in_reward and self.ref is not None:
            batch = self.apply_reward_kl_penalty(batch)
        batch = self.compute_advantages_and_returns(batch)
        m = self.train_critic_and_policy(batch)
        m["trainer/num_tokens"] = float(batch["attention_mask"].sum())
        return m

    async def train_async(self) -> None:
        t = self.cfg.trainer
        assert self.train_dataset is not None, "train() needs a train_dataset"
        self.train_iter = StatefulBatchIterator(self.train_dataset, t.train_batch_size, shuffle=True, seed=t.seed)
        self.load_checkpoints()
        total = t.epochs * len(self.train_iter)
        if t.max_training_steps is not None:
            total = min(total, t.max_training_steps)
        self.staleness: List[int] = []
        while self.global_step < total and self.train_iter.epoch < t.epochs:
            buffer: asyncio.Queue = asyncio.Queue(maxsize=1)
            sync_finished, ack = asyncio.Event(), asyncio.Event()
            remaining = total - self.global_step
            gen_task = asyncio.create_task(self._generate_loop(iter(self.train_iter), buffer, sync_finished, ack, remaining))
            try:
                while True:
                    item = await buffer.get()
                    if item is None:
                        break
                    out, uids = item
                    self.all_metrics, self.all_timings = {}, {}
                    gen_version = out.get("weight_version", None)
                    with Timer("train_critic_and_policy", self.all_timings):
                        metrics = await asyncio.to_thread(self._train_on, out, uids)
                    await ack.wait()  # generation of the next batch finished (or the loop ended)
                    ack.clear()
                    with Timer("sync_weights", self.all_timings):
                        self.sync_weights()
                    sync_finished.set()
                    self.global_step += 1
                    self.all_metrics.update(metrics)
                    self.all_metrics["trainer/global_step"] = float(self.global_step)
                    self.all_metrics.update({f"timing/{k}": v for k, v in self.all_timings.items()})
                    self._log(dict(self.all_metrics), self.global_step)
                    if t.ckpt_interval > 0 and self.global_step % t.ckpt_interval == 0:
                        self.save_checkpoints()
                    if self.global_step >= total:
                        break
            finally:
                if not gen_task.done():
                    gen_task.cancel()
                    try:
                        await gen_task
                    except (asyncio.CancelledError, Exception):  # noqa: BLE001
                        pass
