#!/usr/bin/env bash
# Long-context REPL environment whose code may query the policy (llm_query) and spawn child episodes (rlm_query).
# Dataset rows: prompt (the question), env_extras.context (the document), reward_spec.ground_truth.
set -euo pipefail
MODEL=${MODEL:-qwen2.5-7b}
DATA=${DATA:-$HOME/data/rlm}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU examples/rlm/main_rlm.py \
  trainer.policy.model.path=$MODEL \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=rlm \
  environment.skyrl_gym.max_env_workers=64 \
  generator.max_turns=10 \
  generator.batched=false \
  generator.use_conversation_multi_turn=true \
  trainer.train_batch_size=128 \
  trainer.policy_mini_batch_size=32 \
  generator.n_samples_per_prompt=8 \
  trainer.max_prompt_length=2048 \
  generator.max_input_length=16384 \
  generator.sampling_params.max_generate_length=1024 \
  trainer.max_tokens_per_microbatch=32768 \
  trainer.algorithm.advantage_estimator=grpo \
  trainer.algorithm.use_kl_loss=false \
  trainer.logger=console \
  "$@"
