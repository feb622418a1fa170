#!/usr/bin/env bash
# GRPO where the rollout loop talks to the policy through /v1/chat/completions (template for agent-scaffold adapters).
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU examples/train_integrations/openai_chat/main_chat.py \
  trainer.policy.model.path=$MODEL \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=gsm8k \
  generator.batched=false \
  generator.max_turns=1 \
  trainer.train_batch_size=256 \
  trainer.policy_mini_batch_size=64 \
  generator.n_samples_per_prompt=8 \
  trainer.max_prompt_length=512 \
  generator.sampling_params.max_generate_length=1024 \
  trainer.algorithm.advantage_estimator=grpo \
  trainer.algorithm.use_kl_loss=false \
  trainer.logger=console \
  "$@"
