#!/usr/bin/env bash
# GRPO with a draft head trained beside the policy (soft cross-entropy on detached trunk states) and used by the
# colocated engine for speculative decoding: one guess per step, kept when the token sampled from the target equals it.
# The engine reads the head the trainer updates, so there is no drafter reload after a weight sync.
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.main_base \
  trainer.policy.model.path=$MODEL \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=gsm8k \
  trainer.mtp.enabled=true \
  trainer.mtp.num_speculative_tokens=1 \
  trainer.mtp.loss_weight=0.1 \
  trainer.b200.speculative_decode=true \
  trainer.train_batch_size=256 \
  trainer.policy_mini_batch_size=64 \
  generator.n_samples_per_prompt=8 \
  generator.batched=true \
  trainer.max_prompt_length=512 \
  generator.sampling_params.max_generate_length=1024 \
  trainer.algorithm.advantage_estimator=grpo \
  trainer.algorithm.use_kl_loss=false \
  trainer.logger=console \
  "$@"
