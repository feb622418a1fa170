#!/usr/bin/env bash
# PPO with a critic and a reference model on a TP=4 x DP=2 mesh, rollouts through TP=2 engines in lock step; after each
# update one kernel per trainer rank re-lays its TP4 shards out into the TP2 engines' buffers (vocabulary-parallel
# fused LM head on the trainer side).
set -euo pipefail
MODEL=${MODEL:-qwen2.5-7b}
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.main_base \
  trainer.policy.model.path=$MODEL \
  trainer.strategy=megatron \
  trainer.policy.megatron_config.tensor_model_parallel_size=4 \
  trainer.critic.megatron_config.tensor_model_parallel_size=4 \
  trainer.ref.megatron_config.tensor_model_parallel_size=4 \
  trainer.b200.vocab_parallel_lm_head=true \
  generator.inference_engine.tensor_parallel_size=2 \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=gsm8k \
  trainer.algorithm.advantage_estimator=gae \
  trainer.algorithm.use_kl_loss=true \
  trainer.train_batch_size=128 \
  trainer.policy_mini_batch_size=128 \
  trainer.critic_mini_batch_size=128 \
  generator.n_samples_per_prompt=4 \
  trainer.max_prompt_length=1024 \
  generator.sampling_params.max_generate_length=4096 \
  trainer.max_tokens_per_microbatch=16384 \
  trainer.policy.optimizer_config.lr=1.0e-6 \
  trainer.critic.optimizer_config.lr=5.0e-6 \
  trainer.logger=console \
  "$@"
