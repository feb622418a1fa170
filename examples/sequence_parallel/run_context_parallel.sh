#!/usr/bin/env bash
# Long-context GRPO with context parallelism: every rank of a group owns a slice of each packed sequence with all
# attention heads and all-gathers the keys / values of the tokens before it.  Unlike Ulysses, the group size does not
# have to divide the number of key/value heads (Qwen2.5-1.5B has two; CP=4 works).
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.main_base \
  trainer.policy.model.path=$MODEL \
  trainer.policy.sequence_parallel_size=${CP:-4} \
  trainer.ref.sequence_parallel_size=${CP:-4} \
  trainer.sequence_parallel_backend=context \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=gsm8k \
  trainer.train_batch_size=128 \
  trainer.policy_mini_batch_size=128 \
  generator.n_samples_per_prompt=4 \
  trainer.max_prompt_length=2048 \
  generator.sampling_params.max_generate_length=16384 \
  trainer.max_tokens_per_microbatch=32768 \
  trainer.algorithm.advantage_estimator=grpo \
  trainer.algorithm.use_kl_loss=true \
  trainer.policy.optimizer_config.lr=1.0e-6 \
  trainer.logger=console \
  "$@"
