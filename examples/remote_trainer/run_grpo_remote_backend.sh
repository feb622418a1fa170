#!/usr/bin/env bash
# GRPO with the RL loop on this machine and the model behind a Tinker-compatible training service
# (skyrl_b200/integrations/remote_trainer).  Start the service first, e.g. on the GPU machine:
#   python -m skyrl_b200.tinker.api --base-model Qwen/Qwen2.5-1.5B-Instruct --port 8000
set -euo pipefail
SERVICE_URL=${SERVICE_URL:-http://127.0.0.1:8000}
DATA_DIR=${DATA_DIR:-$HOME/data/gsm8k}

python -m skyrl_b200.integrations.remote_trainer.entrypoint \
  --service-url "$SERVICE_URL" \
  data.train_data="['$DATA_DIR/train.parquet']" \
  data.val_data="['$DATA_DIR/validation.parquet']" \
  trainer.policy.model.path=Qwen/Qwen2.5-1.5B-Instruct \
  trainer.algorithm.advantage_estimator=grpo \
  trainer.algorithm.use_kl_loss=false \
  trainer.train_batch_size=256 \
  trainer.policy_mini_batch_size=64 \
  trainer.policy.optimizer_config.lr=1.0e-6 \
  trainer.epochs=20 \
  trainer.eval_interval=5 \
  trainer.ckpt_interval=10 \
  trainer.max_prompt_length=512 \
  generator.n_samples_per_prompt=5 \
  generator.sampling_params.max_generate_length=1024 \
  generator.sampling_params.temperature=1.0 \
  environment.env_class=gsm8k \
  trainer.logger=console \
  "$@"
