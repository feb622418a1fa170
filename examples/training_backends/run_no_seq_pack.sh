#!/usr/bin/env bash
# Row-count micro-batches instead of token-budget packing: every micro-batch holds micro_*_batch_size_per_gpu rows
# (trainer.max_tokens_per_microbatch=-1); the rows of a micro-batch are still concatenated without padding tokens.
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.main_base \
  trainer.policy.model.path=$MODEL \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=gsm8k \
  trainer.max_tokens_per_microbatch=-1 \
  trainer.micro_train_batch_size_per_gpu=4 \
  trainer.micro_forward_batch_size_per_gpu=16 \
  trainer.b200.microbatch_packing=balanced \
  trainer.train_batch_size=256 \
  trainer.policy_mini_batch_size=64 \
  generator.n_samples_per_prompt=8 \
  generator.batched=true \
  trainer.algorithm.advantage_estimator=grpo \
  trainer.logger=console \
  "$@"
