#!/usr/bin/env bash
# Supervised fine-tuning on chat data with sequence packing.
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}      # preset name (random init) or a local HF checkpoint directory
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.main_sft \
  model.path=$MODEL \
  dataset_name=${SFT_DATA:-$HOME/data/sft/train.jsonl} \
  batch_size=256 \
  max_length=4096 \
  use_sequence_packing=true \
  max_tokens_per_microbatch=32768 \
  optimizer_config.lr=1.0e-5 \
  num_epochs=1 \
  placement.num_gpus_per_node=$NGPU \
  train_on_what=all_assistant_messages \
  "$@"
