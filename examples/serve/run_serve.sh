#!/usr/bin/env bash
# Stand-alone rollout servers: one engine + HTTP server per GPU and, on rank 0, a session-affine router in front.
# Clients (a trainer with generator.inference_engine.external_proxy_url, or any OpenAI-style client) talk to the router.
set -euo pipefail
MODEL=${MODEL:-qwen2.5-1.5b}
NGPU=${NGPU:-8}

python -m skyrl_b200.launch --nproc-per-node $NGPU -m skyrl_b200.entrypoints.serve \
  trainer.policy.model.path=$MODEL \
  generator.inference_engine.num_engines=$NGPU \
  generator.inference_engine.tensor_parallel_size=1 \
  generator.inference_engine.gpu_memory_utilization=0.85 \
  generator.inference_engine.max_num_seqs=512 \
  generator.inference_engine.enable_prefix_caching=true \
  trainer.max_prompt_length=2048 \
  generator.sampling_params.max_generate_length=2048 \
  "$@"
