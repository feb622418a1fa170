#!/usr/bin/env bash
# PPO with a learned critic (GAE advantages).
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}      # preset name (random init) or a local HF checkpoint directory
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.main_base \
  trainer.policy.model.path=$MODEL \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=gsm8k \
  trainer.train_batch_size=1024 \
  trainer.policy_mini_batch_size=256 \
  generator.n_samples_per_prompt=5 \
  trainer.max_prompt_length=512 \
  generator.sampling_params.max_generate_length=1024 \
  trainer.policy.optimizer_config.lr=1.0e-6 \
  trainer.max_tokens_per_microbatch=32768 \
  generator.inference_engine.gpu_memory_utilization=0.6 \
  trainer.logger=console \
  trainer.algorithm.advantage_estimator=gae \
  trainer.critic.model.path=$MODEL \
  trainer.critic.optimizer_config.lr=5.0e-6 \
  trainer.critic_mini_batch_size=256 \
  trainer.algorithm.use_kl_loss=false \
  trainer.algorithm.use_kl_in_reward=true \
  "$@"
