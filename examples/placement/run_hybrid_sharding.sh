#!/usr/bin/env bash
# Hybrid sharding of the optimizer: shard groups of FSDP_SIZE ranks, replicated across groups (the reduced gradient
# shard is all-reduced between replicas).  Fewer peers per reduce-scatter and per parameter push than full sharding.
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.main_base \
  trainer.policy.model.path=$MODEL \
  trainer.policy.fsdp_config.fsdp_size=${FSDP_SIZE:-4} \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=gsm8k \
  trainer.train_batch_size=1024 \
  trainer.policy_mini_batch_size=256 \
  generator.n_samples_per_prompt=5 \
  trainer.algorithm.advantage_estimator=grpo \
  trainer.policy.optimizer_config.lr=1.0e-6 \
  trainer.logger=console \
  "$@"
