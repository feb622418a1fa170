#!/usr/bin/env bash
# Evaluation-only run over the validation set.
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}      # preset name (random init) or a local HF checkpoint directory
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.main_generate \
  trainer.policy.model.path=$MODEL \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=gsm8k \
  generator.eval_n_samples_per_prompt=4 \
  "$@"
