#!/usr/bin/env bash
# Stand-alone rollout servers (one per GPU) and a session-affine router.
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}      # preset name (random init) or a local HF checkpoint directory
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.serve \
  trainer.policy.model.path=$MODEL \
  generator.inference_engine.gpu_memory_utilization=0.85 \
  "$@"
