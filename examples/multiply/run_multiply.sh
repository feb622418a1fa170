#!/usr/bin/env bash
# Custom environment end to end: python examples/multiply/multiply_dataset.py --out $DATA, then this script.
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}
DATA=${DATA:-$HOME/data/multiply}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU examples/multiply/main_multiply.py \
  trainer.policy.model.path=$MODEL \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=multiply \
  generator.max_turns=2 \
  generator.use_conversation_multi_turn=true \
  generator.batched=false \
  trainer.train_batch_size=256 \
  trainer.policy_mini_batch_size=64 \
  generator.n_samples_per_prompt=8 \
  trainer.max_prompt_length=256 \
  generator.sampling_params.max_generate_length=128 \
  trainer.policy.optimizer_config.lr=1.0e-6 \
  trainer.algorithm.advantage_estimator=grpo \
  trainer.algorithm.use_kl_loss=false \
  trainer.logger=console \
  trainer.epochs=10 \
  "$@"
