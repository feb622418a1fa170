#!/usr/bin/env bash
# MoE GRPO with rollout router replay: the engine records which experts every generated token was routed to and the
# trainer replays those choices in its forward pass, so training sees the rollout's routing, not a re-drawn one.
set -euo pipefail
MODEL=${MODEL:-qwen3-30b-a3b}
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.main_base \
  trainer.policy.model.path=$MODEL \
  trainer.strategy=megatron \
  trainer.policy.megatron_config.expert_model_parallel_size=$NGPU \
  generator.inference_engine.enable_return_routed_experts=true \
  trainer.policy.megatron_config.moe_enable_routing_replay=true \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=gsm8k \
  trainer.train_batch_size=128 \
  trainer.policy_mini_batch_size=128 \
  generator.n_samples_per_prompt=8 \
  trainer.max_prompt_length=512 \
  generator.sampling_params.max_generate_length=1024 \
  trainer.algorithm.advantage_estimator=grpo \
  trainer.algorithm.use_kl_loss=false \
  trainer.policy.optimizer_config.lr=1.0e-6 \
  trainer.logger=console \
  "$@"
