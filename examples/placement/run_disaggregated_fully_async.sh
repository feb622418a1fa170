#!/usr/bin/env bash
# One launch, two roles: the first half of the GPUs trains (sharded optimizer + Ulysses sequence parallelism), the
# second half only rolls out (one engine + server per GPU).  Weights reach the running engines by peer stores between
# pause(keep) and resume; generation continues while the trainer works on the previous batch (fully asynchronous).
set -euo pipefail
MODEL=${MODEL:-qwen2.5-7b}
DATA=${DATA:-$HOME/data/gsm8k}
NGPU=${NGPU:-8}   # = NTRAIN + NROLLOUT

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.main_base \
  trainer.policy.model.path=$MODEL \
  trainer.placement.colocate_all=false \
  trainer.placement.policy_num_gpus_per_node=${NTRAIN:-4} \
  generator.inference_engine.num_engines=${NROLLOUT:-4} \
  trainer.policy.sequence_parallel_size=${NTRAIN:-4} \
  trainer.fully_async.enabled=true \
  trainer.fully_async.max_staleness_steps=1 \
  trainer.algorithm.policy_loss_type=rollout_is \
  trainer.algorithm.use_kl_loss=false \
  data.train_data=["$DATA/train.parquet"] \
  data.val_data=["$DATA/validation.parquet"] \
  environment.env_class=gsm8k \
  trainer.train_batch_size=64 \
  trainer.policy_mini_batch_size=64 \
  generator.n_samples_per_prompt=4 \
  trainer.max_prompt_length=1024 \
  generator.sampling_params.max_generate_length=8192 \
  generator.inference_engine.enable_prefix_caching=true \
  trainer.policy.optimizer_config.lr=1.0e-6 \
  trainer.logger=console \
  "$@"
