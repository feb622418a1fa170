#!/usr/bin/env bash
# Memory check before a long run: two steps on rows of maximum length (no rollout, no dataset).
set -euo pipefail
MODEL=${MODEL:-qwen2.5-7b}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU examples/train_scripts/full_context/main_full_ctx.py \
  trainer.policy.model.path=$MODEL \
  trainer.train_batch_size=256 \
  trainer.policy_mini_batch_size=64 \
  generator.n_samples_per_prompt=8 \
  trainer.max_prompt_length=2048 \
  generator.sampling_params.max_generate_length=8192 \
  trainer.max_tokens_per_microbatch=32768 \
  trainer.algorithm.advantage_estimator=grpo \
  trainer.algorithm.use_kl_loss=true \
  trainer.gradient_checkpointing=true \
  trainer.logger=console \
  trainer.resume_mode=none \
  "$@"
