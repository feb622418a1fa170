#!/usr/bin/env bash
# SFT with a perplexity logger and an early-stop callback (examples/callbacks/main_sft_with_callbacks.py).
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU examples/callbacks/main_sft_with_callbacks.py \
  model.path=$MODEL \
  dataset_name=${SFT_DATA:-$HOME/data/sft/train.jsonl} \
  batch_size=128 \
  max_length=2048 \
  use_sequence_packing=true \
  max_tokens_per_microbatch=32768 \
  optimizer_config.lr=1.0e-5 \
  num_epochs=1 \
  placement.num_gpus_per_node=$NGPU \
  "$@"
