#!/usr/bin/env bash
# Student = MODEL, teacher = TEACHER (same tokenizer).  Rewards are the teacher-student log-prob gap per token.
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU examples/on_policy_distillation/main_on_policy_distill.py \
  trainer.policy.model.path=$MODEL \
  trainer.ref.model.path=${TEACHER:-qwen2.5-7b} \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=gsm8k \
  trainer.algorithm.advantage_estimator=token_rewards \
  trainer.algorithm.use_kl_in_reward=true \
  trainer.algorithm.use_kl_loss=false \
  trainer.algorithm.policy_loss_type=rollout_is \
  trainer.train_batch_size=256 \
  trainer.policy_mini_batch_size=256 \
  generator.n_samples_per_prompt=4 \
  trainer.max_prompt_length=512 \
  generator.sampling_params.max_generate_length=1024 \
  trainer.policy.optimizer_config.lr=1.0e-6 \
  trainer.logger=console \
  trainer.epochs=10 \
  "$@"
