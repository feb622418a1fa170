"""Dry run at the longest sequences a configuration allows: no rollout, every row is ``max_input_length`` prompt tokens
plus ``max_generate_length`` response tokens, pushed through the same forward passes, advantage computation, policy /
critic update and weight sync as a real step.  A configuration that survives this does not run out of memory when a
batch of maximum-length responses shows up mid-run.  Prints the step time and the peak device memory per rank.

    python -m skyrl_b200.launch --nproc-per-node 8 examples/train_scripts/full_context/main_full_ctx.py \\
        trainer.policy.model.path=qwen2.5-7b ... num_dummy_steps=2

Counterpart in the reference: examples/train_scripts/full_context/{main_full_ctx,trainer_full_ctx}.py.
"""

import random
import sys
import time

import torch

from skyrl_b200.config.config import SkyRLTrainConfig
from skyrl_b200.entrypoints.main_base import BasePPOExp
from skyrl_b200.train.trainer import PPOTrainer


class FullCtxTrainer(PPOTrainer):
    num_dummy_steps = 2

    def _max_length_output(self, seed: int):
        cfg = self.cfg
        rng = random.Random(seed + 977 * self.env.rank)
        n_prompts = max(1, cfg.trainer.train_batch_size // self.env.world_size)
        n = cfg.generator.n_samples_per_prompt
        P, R = cfg.generator.max_input_length, cfg.generator.sampling_params.max_generate_length
        vocab = len(self.tokenizer)
        prompts, uids = [], []
        for i in range(n_prompts):
            p = [rng.randrange(4, vocab) for _ in range(P)]
            prompts += [p] * n
            uids += [f"full-{self.env.rank}-{i}"] * n
        rows = len(prompts)
        out = {"prompt_token_ids": prompts, "response_ids": [[rng.randrange(4, vocab) for _ in range(R)] for _ in range(rows)],
               "rewards": [float(rng.randrange(2)) for _ in range(rows)], "loss_masks": [[1] * R for _ in range(rows)],
               "stop_reasons": ["length"] * rows, "rollout_metrics": None, "rollout_logprobs": None}
        return out, uids

    def train(self) -> None:
        for step in range(self.num_dummy_steps):
            self.all_metrics, self.all_timings = {}, {}
            t0 = time.time()
            out, uids = self._max_length_output(step)
            out, uids = self.postprocess_generator_output(out, uids)
            batch = self.convert_to_training_input(out, uids)
            batch = self.fwd_logprobs_values_reward(batch)
            if self.cfg.trainer.algorithm.use_kl_in_reward and self.ref is not None:
                batch = self.apply_reward_kl_penalty(batch)
            batch = self.compute_advantages_and_returns(batch)
            status = self.train_critic_and_policy(batch)
            self.sync_weights()
            self.global_step += 1
            peak = torch.cuda.max_memory_allocated() / 2**30 if torch.cuda.is_available() else 0.0
            print(f"[full-context] rank {self.env.rank} step {step + 1}/{self.num_dummy_steps}: "
                  f"{batch['sequences'].shape[0]} rows x {batch['sequences'].shape[1]} tokens, "
                  f"{time.time() - t0:.2f} s, peak {peak:.1f} GiB, grad_norm {status.get('policy/grad_norm', float('nan')):.4f}",
                  flush=True)


class FullCtxExp(BasePPOExp):
    def get_train_dataset(self):
        return None  # nothing is read: the rows are synthesised at the configured maximum lengths

    def get_eval_dataset(self):
        return None

    def get_trainer(self, cfg, tracker, tokenizer, train_dataset, eval_dataset, inference_engine_client, generator):
        tr = FullCtxTrainer(cfg, tracker=tracker, tokenizer=tokenizer, train_dataset=None, eval_dataset=None,
                            inference_engine_client=inference_engine_client, generator=generator, env=self.env)
        tr.num_dummy_steps = self.num_dummy_steps
        return tr


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("num_dummy_steps=")]
    steps = [int(a.split("=", 1)[1]) for a in sys.argv[1:] if a.startswith("num_dummy_steps=")]
    exp = FullCtxExp.__new__(FullCtxExp)
    exp.num_dummy_steps = steps[0] if steps else 2
    FullCtxExp.__init__(exp, SkyRLTrainConfig.from_cli_overrides(args))
    exp.run()
