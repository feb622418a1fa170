#!/usr/bin/env bash
# Multi-turn GSM8K: the environment answers a wrong attempt with a hint and scores every turn; the per-turn rewards
# land on the last token of each assistant turn, and observation tokens are masked out of the loss.
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.main_base \
  trainer.policy.model.path=$MODEL \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=gsm8k_multi_turn \
  generator.max_turns=3 \
  generator.use_conversation_multi_turn=true \
  generator.batched=false \
  trainer.train_batch_size=256 \
  trainer.policy_mini_batch_size=64 \
  generator.n_samples_per_prompt=5 \
  trainer.max_prompt_length=512 \
  generator.max_input_length=4096 \
  generator.sampling_params.max_generate_length=512 \
  trainer.algorithm.advantage_estimator=grpo \
  trainer.algorithm.use_kl_loss=false \
  trainer.policy.optimizer_config.lr=1.0e-6 \
  trainer.logger=console \
  trainer.epochs=10 \
  "$@"
