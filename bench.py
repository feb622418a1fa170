#!/usr/bin/env python
"""Headline benchmark: one GRPO step (rollout + train + weight sync) of the Qwen2.5-1.5B-architecture
configuration, per-GPU work fixed (weak scaling): 32 prompts x 8 samples per GPU, 512-token uniform-random
prompts, responses of a length drawn uniformly in [256, 1024], Bernoulli(0.5) rewards, bf16, random init.

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Rank 0 prints one JSON line.  ``value`` is (generated + trained tokens) / second summed over all GPUs, timed
with CUDA events around exactly K steps (max over ranks); ``e2e`` is the same quantity from the host wall
clock around the same public-API calls (``PPOTrainer.train_step``), whose inputs start in pinned host memory
and whose metrics are read back to the host every step.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

METRIC = "rl_step_tokens_per_sec"
MODEL = "qwen2.5-1.5b"
PROMPTS_PER_GPU, N_SAMPLES, PROMPT_LEN, RESP_MIN, RESP_MAX = 32, 8, 512, 256, 1024

# The other headline configurations.  Every entry fixes the per-GPU work (weak scaling); the parallel layout is the named
# one when enough GPUs are present and is shrunk (and reported as such) on smaller runs.
CONFIGS = {
    # GRPO, Qwen2.5-1.5B, colocated sharded data parallel (the default, also selected by no --config at all)
    2: dict(model="qwen2.5-1.5b", prompts_per_gpu=32, n=8, prompt_len=512, resp_min=256, resp_max=1024, tp=1, engine_tp=1,
            algo="grpo"),
    # PPO with critic and reference model, Qwen2.5-7B, TP=4 x DP=2 training, TP=2 rollout engines, vocabulary-parallel
    # fused LM head, GAE(gamma=1, lambda=0.95), N(0, 1) reward on the last token; 128 prompts x 4 samples at 8 GPUs
    3: dict(model="qwen2.5-7b", prompts_per_gpu=16, n=4, prompt_len=1024, resp_min=4096, resp_max=4096, tp=4, engine_tp=2,
            algo="ppo"),
    # GRPO, Qwen3-30B-A3B, expert parallel over all ranks; 64 prompts x 8 samples at 8 GPUs
    4: dict(model="qwen3-30b-a3b", prompts_per_gpu=8, n=8, prompt_len=1024, resp_min=2048, resp_max=2048, tp=1, engine_tp=1,
            algo="grpo", ep="world"),
}


def reference_arm() -> None:
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference installs with --no-deps into baseline/_ref but its public API cannot import here: "
                      "ray, omegaconf, cloudpathlib, megatron-core and the pinned vllm 0.26 weight-transfer API are not "
                      "installed and there is no network"}))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.path = gpu_index, None, f"/tmp/sb_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
            except ValueError:
                continue
            for n, v in zip(names, p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        busy = [c for c in sm if c > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--config", type=int, default=2, choices=sorted(CONFIGS), help="headline configuration (BASELINE numbering)")
    ap.add_argument("--model", default=None)
    ap.add_argument("--prompts-per-gpu", type=int, default=None)
    ap.add_argument("--n-samples", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--resp-len", type=int, default=None, help="fixed response length (overrides the configuration's range)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the separately timed end-to-end steps (long configurations)")
    ap.add_argument("--max-tokens-per-microbatch", type=int, default=32768)
    ap.add_argument("--tp", type=int, default=None, help="tensor-parallel size of the training model (1 = sharded data parallel)")
    ap.add_argument("--ep", type=int, default=None, help="expert-parallel size (MoE models)")
    ap.add_argument("--pp", type=int, default=1, help="pipeline-parallel size of the training model")
    ap.add_argument("--sp", type=int, default=1, help="Ulysses sequence-parallel size of the training model")
    ap.add_argument("--engine-tp", type=int, default=None, help="tensor-parallel size of each rollout engine (lock-step ranks, "
                    "all-reduce in the o-proj / down-proj GEMM epilogues)")
    ap.add_argument("--reuse-train-forward", action="store_true",
                    help="take old log-probs from the training forward (exact with one optimizer update per step); "
                         "off by default so the step runs the same separate old-policy forward the reference does")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return

    import torch

    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.ops import _lib
    from skyrl_b200.parallel import dist as pdist
    from skyrl_b200.train.trainer import PPOTrainer
    from skyrl_b200.utils.tokenizer import SyntheticTokenizer

    env = pdist.init_distributed()
    world = env.world_size
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node")
    from skyrl_b200.models.decoder import PRESETS

    spec = CONFIGS[args.config]
    args.model = args.model or spec["model"]
    P = args.prompts_per_gpu or spec["prompts_per_gpu"]
    n = args.n_samples or spec["n"]
    PROMPT_LEN = args.prompt_len or spec["prompt_len"]
    RESP_MIN, RESP_MAX = (args.resp_len, args.resp_len) if args.resp_len else (spec["resp_min"], spec["resp_max"])

    def fit(want: int) -> int:  # largest power-of-two layout size <= want that divides the world
        k = 1
        while k * 2 <= want and world % (k * 2) == 0:
            k *= 2
        return k

    args.tp = fit(args.tp if args.tp is not None else spec["tp"])
    args.engine_tp = fit(args.engine_tp if args.engine_tp is not None else spec["engine_tp"])
    args.ep = args.ep if args.ep is not None else (world if spec.get("ep") == "world" and world > 1 else 1)
    ppo = spec["algo"] == "ppo"
    margs = PRESETS[args.model]
    cfg = SkyRLTrainConfig.from_cli_overrides([
        f"trainer.policy.model.path={args.model}", f"trainer.train_batch_size={P * world}",
        f"trainer.policy_mini_batch_size={P * world}", f"generator.n_samples_per_prompt={n}",
        f"trainer.max_prompt_length={PROMPT_LEN}", f"generator.sampling_params.max_generate_length={RESP_MAX}",
        "generator.sampling_params.temperature=1.0", "generator.batched=true",
        *(["trainer.algorithm.advantage_estimator=gae", "trainer.algorithm.gamma=1.0", "trainer.algorithm.lambd=0.95",
           f"trainer.critic.model.path={args.model}", f"trainer.critic_mini_batch_size={P * world}",
           "trainer.algorithm.use_kl_loss=true", "trainer.algorithm.kl_loss_coef=0.001",
           "trainer.critic.optimizer_config.lr=5e-6", "environment.env_class=synthetic_gaussian",
           "trainer.b200.vocab_parallel_lm_head=true"] if ppo else
          ["trainer.algorithm.advantage_estimator=grpo", "trainer.algorithm.use_kl_loss=false",
           "environment.env_class=synthetic_bernoulli"]),
        "trainer.algorithm.policy_loss_type=regular",
        "trainer.policy.optimizer_config.lr=1e-6", f"trainer.max_tokens_per_microbatch={args.max_tokens_per_microbatch}",
        "trainer.gradient_checkpointing=false",
        f"generator.inference_engine.max_num_seqs={P * n}", "generator.inference_engine.gpu_memory_utilization=0.25",
        "generator.inference_engine.enable_prefix_caching=false", "trainer.resume_mode=none", "trainer.seed=0",
        "trainer.logger=console", *(["trainer.strategy=megatron",
                                    f"trainer.policy.megatron_config.tensor_model_parallel_size={args.tp}"] if args.tp > 1 else []),
        *(["trainer.strategy=megatron", f"trainer.policy.megatron_config.expert_model_parallel_size={args.ep}"]
          if args.ep > 1 else []),
        *(["trainer.strategy=megatron", f"trainer.policy.megatron_config.pipeline_model_parallel_size={args.pp}"]
          if args.pp > 1 else []),
        *([f"trainer.policy.sequence_parallel_size={args.sp}", f"trainer.ref.sequence_parallel_size={args.sp}"]
          if args.sp > 1 else []),
        *([f"generator.inference_engine.tensor_parallel_size={args.engine_tp}"] if args.engine_tp > 1 else []),
        f"trainer.b200.reuse_train_forward_for_old_logprobs={'true' if args.reuse_train_forward else 'false'}"])
    tok = SyntheticTokenizer(margs.vocab_size)
    trainer = PPOTrainer(cfg, tokenizer=tok, env=env)
    trainer.build_models()

    g = torch.Generator().manual_seed(1234 + env.rank)
    e2e_steps = 0 if args.no_e2e else args.steps
    total_steps = args.warmup + args.steps + e2e_steps  # warm-up, device-timed steps, then separately timed end-to-end steps
    # all step inputs live in pinned host memory; every step copies its own slice to the device
    prompt_store = torch.randint(4, margs.vocab_size, (total_steps, P, PROMPT_LEN), generator=g, dtype=torch.int32)
    len_store = torch.randint(RESP_MIN, RESP_MAX + 1, (total_steps, P * n), generator=g, dtype=torch.int32)
    if torch.cuda.is_available():
        prompt_store, len_store = prompt_store.pin_memory(), len_store.pin_memory()

    def make_step_inputs(s: int):
        rows = prompt_store[s].tolist()
        lens = len_store[s].tolist()
        items = []
        for i, ids in enumerate(rows):
            items.append({"prompt": [{"role": "user", "content": ids}], "prompt_token_ids": ids, "uid": f"s{s}r{env.rank}p{i}",
                          "env_extras": {"p": 0.5, "seed": s * 100003 + env.rank * 1009 + i}})
        return items, lens

    def run_step(s: int):
        items, lens = make_step_inputs(s)
        # per-sample response length: EOS is forced by capping the sample at its drawn length
        k = 0
        per_item = []
        for it in items:
            per_item.append(lens[k : k + n])
            k += n
        trainer.generator._per_sample_max_tokens = per_item
        m = trainer.train_step(items)
        if env.is_main:
            import sys

            print("[bench] step %d: " % s + ", ".join(f"{k[7:]}={v:.3f}" for k, v in m.items() if k.startswith("timing/")) +
                  f", gen_tokens={m['trainer/num_generated_tokens']:.0f}" +
                  (f", alloc_retries={torch.cuda.memory_stats().get('num_alloc_retries', 0)}"
                   f", max_alloc_gb={torch.cuda.max_memory_allocated() / 2**30:.1f}"
                   f", reserved_gb={torch.cuda.memory_reserved() / 2**30:.1f}" if torch.cuda.is_available() else ""),
                  file=sys.stderr, flush=True)
        return m

    # per-sample lengths are passed through env_extras["sampling_params"], one entry per repetition
    from skyrl_b200.train.generators import utils as gutils

    orig_prepare = gutils.prepare_generator_input

    def prepare_with_lengths(prompts, n_samples, sp, env_class, phase, step, prompt_token_ids=None):
        gi, uids = orig_prepare(prompts, n_samples, sp, env_class, phase, step, prompt_token_ids)
        per_item = getattr(trainer.generator, "_per_sample_max_tokens", None)
        if per_item is not None:
            flat = [L for row in per_item for L in row]
            for ex, L in zip(gi["env_extras"], flat):
                ex["sampling_params"] = {"max_generate_length": int(L), "ignore_eos": True}
        return gi, uids

    import skyrl_b200.train.trainer as trainer_mod

    trainer_mod.prepare_generator_input = prepare_with_lengths

    for s in range(args.warmup):
        run_step(s)
    pdist.barrier()
    sampler = ClockSampler(env.local_rank)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if env.is_main:
        sampler.start()
    l0 = _lib.LAUNCH_COUNT
    t0 = time.perf_counter()
    if torch.cuda.is_available():
        ev0.record()
    tokens = 0.0
    gen_tokens = 0.0
    last = {}
    for s in range(args.warmup, args.warmup + args.steps):
        last = run_step(s)
        tokens += last["trainer/num_tokens"] + last["trainer/num_generated_tokens"]
        gen_tokens += last["trainer/num_generated_tokens"]
    if torch.cuda.is_available():
        ev1.record()
        torch.cuda.synchronize()
    pdist.barrier()
    dev_wall = time.perf_counter() - t0
    launches = _lib.LAUNCH_COUNT - l0
    # end-to-end pass: the same public call (trainer.train_step) on fresh prompts, timed on the host clock from before
    # the step's inputs leave pinned host memory until its metrics (loss, reward, token counts) are back on the host
    h0, d0 = _lib.H2D_BYTES, _lib.D2H_BYTES
    pdist.barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    t1 = time.perf_counter()
    e2e_tokens = 0.0
    for s in range(args.warmup + args.steps, total_steps):
        m = run_step(s)
        e2e_tokens += m["trainer/num_tokens"] + m["trainer/num_generated_tokens"]
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    pdist.barrier()
    wall = max(1e-9, time.perf_counter() - t1)
    e2e_all = pdist.all_reduce_sum_scalar(e2e_tokens, env.device)
    dev_s = ev0.elapsed_time(ev1) / 1e3 if torch.cuda.is_available() else dev_wall
    clocks = sampler.stop() if env.is_main else {}
    dev_s = pdist.all_reduce_max_scalar(dev_s, env.device)
    wall = pdist.all_reduce_max_scalar(wall, env.device)
    tokens_all = pdist.all_reduce_sum_scalar(tokens, env.device)
    gen_all = pdist.all_reduce_sum_scalar(gen_tokens, env.device)
    # ranks of a tensor / sequence / pipeline parallel group train on one merged batch and each of them reports it:
    # count that batch once (expert-parallel ranks keep their own data)
    share = max(args.tp, args.sp, args.pp)
    tokens_all, gen_all, e2e_all = tokens_all / share, gen_all / share, e2e_all / share
    K = max(1, args.steps)
    if env.is_main:
        status = _lib.status_read_clear() if torch.cuda.is_available() else 0
        out = {
            "metric": METRIC, "value": tokens_all / dev_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_s * 1e3 / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform-random token ids, %s rewards, random-init weights)"
            % ("N(0,1)" if ppo else "Bernoulli(0.5)"),
            "config": {"model": args.model, "baseline_config": args.config, "algorithm": spec["algo"],
                       "engine_tensor_parallel": args.engine_tp,
                       "global_batch": P * n * world, "seq_len": PROMPT_LEN + RESP_MAX,
                       "parallelism": (f"dp{world} x ep{args.ep} (fused expert dispatch/combine)" if args.ep > 1 else
                                       f"dp{world // args.pp} x pp{args.pp} (layer stages)" if args.pp > 1 else
                                       f"dp{world // args.sp} x sp{args.sp} (Ulysses, fused projections)" if args.sp > 1 else
                                       f"dp{world} (sharded optimizer, colocated engine per GPU)" if args.tp == 1 else
                                       f"dp{world // args.tp} x tp{args.tp} (fused GEMM collectives, colocated engine per GPU)"),
                       "prompts_per_gpu": P, "n_samples_per_prompt": n, "prompt_len": PROMPT_LEN,
                       "response_len": f"uniform[{RESP_MIN},{RESP_MAX}]", "tokens_counted": "generated + trained "
                       "(prompt+response) tokens per step", "generated_tokens_per_step": gen_all / K,
                       "l2_policy": "inputs larger than L2 (3.1 GB of weights, >10 GB of KV and activations per step)",
                       "phase_seconds_last_step": {k[7:]: round(v, 4) for k, v in last.items() if k.startswith("timing/")}},
            "clocks": clocks,
            "e2e": {"value": (e2e_all / wall) if e2e_steps else None, "timed_with": "host clock over %d further steps" % e2e_steps, "unit": "tokens/s", "h2d_bytes_per_step": (_lib.H2D_BYTES - h0) / max(1, e2e_steps),
                    "d2h_bytes_per_step": (_lib.D2H_BYTES - d0) / max(1, e2e_steps)},
            "gpu_launches": launches, "device_status": status, "impl": "ours",
            # trainer -> rollout weight sync: the colocated engine reads the parameter buffer the optimizer's fused
            # push just wrote, so the separate sync phase only bumps the weight version
            "weight_sync_ms": float(last["timing/weight_sync_kernel_ms"]) if "timing/weight_sync_kernel_ms" in last
            else 1e3 * float(last.get("timing/sync_weights", 0.0)),
        }
        print(json.dumps(out), flush=True)
    pdist.shutdown()


if __name__ == "__main__":
    main()
