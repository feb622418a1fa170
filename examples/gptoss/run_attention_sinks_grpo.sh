#!/usr/bin/env bash
# GRPO on a model whose attention layers carry learned sink logits (one per query head, GPT-OSS style).  MODEL may be a
# preset with attention_sinks=true (tiny-sinks) or an HF checkpoint directory whose config.json sets
# "attention_sinks": true and whose tensors include model.layers.N.self_attn.sinks.  Data parallel only.
set -euo pipefail
MODEL=${MODEL:-tiny-sinks}
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.main_base \
  trainer.policy.model.path=$MODEL \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=gsm8k \
  trainer.train_batch_size=256 \
  trainer.policy_mini_batch_size=64 \
  generator.n_samples_per_prompt=5 \
  trainer.max_prompt_length=512 \
  generator.sampling_params.max_generate_length=512 \
  trainer.algorithm.advantage_estimator=grpo \
  trainer.algorithm.use_kl_loss=false \
  trainer.policy.optimizer_config.lr=1.0e-6 \
  trainer.logger=console \
  "$@"
