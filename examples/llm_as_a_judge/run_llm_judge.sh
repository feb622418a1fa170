#!/usr/bin/env bash
# GRPO where the reward comes from a judge model behind an OpenAI-compatible endpoint (environment "llm_judge").
# JUDGE_URL may point at a hosted model or at this package's own server:
#   python -m skyrl_b200.launch --nproc-per-node 1 -m skyrl_b200.entrypoints.serve trainer.policy.model.path=/path/to/judge
# Dataset rows need reward_spec.ground_truth (shown to the judge) and may carry the question in extra_info.question.
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}
export SKYRL_B200_JUDGE_URL=${JUDGE_URL:-http://127.0.0.1:8000}

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.main_base \
  trainer.policy.model.path=$MODEL \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=llm_judge \
  trainer.train_batch_size=256 \
  trainer.policy_mini_batch_size=64 \
  generator.n_samples_per_prompt=5 \
  trainer.max_prompt_length=512 \
  generator.sampling_params.max_generate_length=1024 \
  trainer.algorithm.advantage_estimator=grpo \
  trainer.algorithm.use_kl_loss=false \
  trainer.policy.optimizer_config.lr=1.0e-6 \
  trainer.logger=console \
  "$@"
