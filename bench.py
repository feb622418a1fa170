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
    # long-context multi-turn agent GRPO, disaggregated and fully asynchronous: half of the GPUs train (sharded optimizer +
    # Ulysses sequence parallelism over all of them), the other half only roll out (one unsharded engine each), weights
    # are pushed over NVLink into the running engines; 8 turns of 1024 generated + 512 observation tokens, env tokens
    # masked, Bernoulli(0.3) reward at the end; 32 trajectories x 4 samples per update at 4 + 4 GPUs
    5: dict(model="qwen2.5-7b", prompts_per_gpu=8, n=4, prompt_len=512, turns=8, turn_tokens=1024, obs_tokens=512, algo="grpo"),
}


def _phase_anchor(argv, timeout_s: int):
    """Runs one kernel micro-benchmark of this repo in a child process and returns its JSON line (or the failure)."""
    try:
        p = subprocess.run([sys.executable, "-m", "skyrl_b200.benchmarks.bench_kernels", *argv], capture_output=True,
                           text=True, timeout=timeout_s, cwd=os.path.dirname(os.path.abspath(__file__)))
        for line in reversed(p.stdout.strip().splitlines()):
            if line.startswith("{"):
                return json.loads(line)
        return {"error": (p.stderr or p.stdout)[-300:]}
    except Exception as e:  # noqa: BLE001 - the reference line must be printed whatever happens here
        return {"error": f"{type(e).__name__}: {e}"[:300]}


def reference_arm() -> None:
    """No complete RL step can run through the reference here, so the arm reports ``unavailable``.  What of the
    reference does run on this machine is timed as *phase anchors* on the same tensors as this repo's kernels and
    attached under ``phase_anchors``: its own Triton fused LM-head kernel (and its materialised-logits path), loaded
    unmodified from ``baseline/_ref``, and flash-attn, the library behind its training attention.  These are not a
    reference value for the metric."""
    out = {"impl": "reference", "unavailable":
           "reference installs with --no-deps into baseline/_ref but its public API cannot import here: "
           "ray, omegaconf, cloudpathlib, megatron-core and the pinned vllm 0.26 weight-transfer API are not "
           "installed and there is no network"}
    if int(os.environ.get("RANK", "0")) != 0:
        return  # one line per job
    try:
        import torch

        if torch.cuda.is_available() and os.environ.get("SKYRL_B200_REFERENCE_ANCHORS", "1") == "1":
            out["phase_anchors"] = {
                "note": "same tensors, CUDA events, L2 flushed between iterations; not the reference arm",
                "fused_lm_head_logprob_T8192_V151936_H1536": _phase_anchor(
                    ["--which", "lmhead", "--impl", "both", "--tokens", "8192", "--iters", "3"], 240),
                "training_attention_16x8192_tokens": _phase_anchor(
                    ["--which", "attn", "--impl", "both", "--seqs", "16", "--seqlen", "8192", "--iters", "3"], 120),
            }
    except Exception as e:  # noqa: BLE001
        out["phase_anchors"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    print(json.dumps(out))


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


def run_disaggregated(args) -> None:
    """Configuration 5.  The ranks of the launch split into a training world and a rollout world before any process
    group exists (see ``entrypoints/main_base.py::split_roles``); rollout ranks serve until the trainer shuts them down."""
    import torch

    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.models.decoder import PRESETS

    spec = CONFIGS[5]
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if world < 2 or world != args.gpus:
        raise SystemExit("--config 5 splits the launch into training and rollout ranks: it needs --gpus >= 2 under torchrun")
    n_train = world // 2
    n_roll = world - n_train
    model = args.model or spec["model"]
    margs = PRESETS[model]
    P, n = args.prompts_per_gpu or spec["prompts_per_gpu"], args.n_samples or spec["n"]
    turns, turn_tok, obs_tok = args.turns or spec["turns"], args.resp_len or spec["turn_tokens"], args.obs_tokens or spec["obs_tokens"]
    plen = args.prompt_len or spec["prompt_len"]
    max_len = plen + turns * turn_tok + (turns - 1) * (obs_tok + 4) + 64
    sp_size = 1
    while sp_size * 2 <= n_train and margs.num_kv_heads % (sp_size * 2) == 0:
        sp_size *= 2
    port = int(os.environ.get("MASTER_PORT", "29500"))
    base = port + 100
    urls = [f"http://127.0.0.1:{base + j}" for j in range(n_roll)]
    W_gen = P * 2  # generation workers per training rank: one mini-batch in training, one in flight
    cfg = SkyRLTrainConfig.from_cli_overrides([
        f"trainer.policy.model.path={model}", f"trainer.train_batch_size={P * n_train}",
        f"trainer.policy_mini_batch_size={P * n_train}", f"generator.n_samples_per_prompt={n}",
        f"trainer.max_prompt_length={plen}", f"generator.sampling_params.max_generate_length={turn_tok}",
        'generator.sampling_params.additional_kwargs={"ignore_eos": true}', "generator.sampling_params.temperature=1.0",
        f"generator.max_turns={turns}", f"generator.max_input_length={max_len}", "generator.batched=false",
        "generator.use_conversation_multi_turn=true", "environment.env_class=synthetic_multiturn",
        "trainer.algorithm.advantage_estimator=grpo", "trainer.algorithm.use_kl_loss=false",
        "trainer.algorithm.policy_loss_type=rollout_is", "trainer.policy.optimizer_config.lr=1e-6",
        f"trainer.max_tokens_per_microbatch={args.max_tokens_per_microbatch}", "trainer.gradient_checkpointing=false",
        f"trainer.policy.sequence_parallel_size={sp_size}", "trainer.fully_async.enabled=true",
        "trainer.fully_async.max_staleness_steps=1", f"trainer.fully_async.num_parallel_generation_workers={W_gen}",
        "trainer.placement.colocate_all=false", f"trainer.placement.policy_num_gpus_per_node={n_train}",
        f"generator.inference_engine.num_engines={n_roll}", f"generator.inference_engine.max_num_seqs={4 * P * n}",
        "generator.inference_engine.gpu_memory_utilization=0.6", "generator.inference_engine.enable_prefix_caching=true",
        f"generator.inference_engine.max_num_batched_tokens={max(16384, max_len)}", "trainer.resume_mode=none",
        "trainer.seed=0", "trainer.logger=console", f"trainer.max_training_steps={args.warmup + args.steps}",
        "trainer.epochs=1000000", "trainer.ckpt_interval=0", "trainer.hf_save_interval=0", "trainer.eval_interval=0"])
    os.environ["SKYRL_B200_ROLLOUT_BASE_PORT"] = str(base)
    if rank >= n_train:
        # rollout world: its rank 0 hosts the rendezvous store of that world (torchrun's agent store belongs to the
        # full launch and stays with the training world)
        os.environ.pop("TORCHELASTIC_USE_AGENT_STORE", None)
        os.environ.update(WORLD_SIZE=str(n_roll), RANK=str(rank - n_train), MASTER_PORT=str(port + 1), SKYRL_B200_ROLE="rollout")
        from skyrl_b200.entrypoints.serve import InferenceOnlyEntrypoint

        cfg.trainer.placement.colocate_all = True
        InferenceOnlyEntrypoint(cfg, base_port=base).run(with_router=False)
        return
    os.environ.update(WORLD_SIZE=str(n_train), RANK=str(rank), SKYRL_B200_ROLE="train")
    from skyrl_b200.entrypoints.main_base import _shutdown_servers, _wait_for_servers
    from skyrl_b200.inference.remote_client import RemoteInferenceClient
    from skyrl_b200.ops import _lib
    from skyrl_b200.parallel import dist as pdist
    from skyrl_b200.train.dataset import PromptDataset
    from skyrl_b200.train.fully_async_trainer import FullyAsyncPPOTrainer
    from skyrl_b200.utils.tokenizer import SyntheticTokenizer

    env = pdist.init_distributed()
    tok = SyntheticTokenizer(margs.vocab_size)
    g = torch.Generator().manual_seed(4321)
    n_items = (args.warmup + args.steps + 4) * P * n_train * 2
    rows = []
    for i in range(n_items):
        ids = torch.randint(4, margs.vocab_size, (plen,), generator=g).tolist()
        rows.append({"prompt": [{"role": "user", "content": ids}], "prompt_token_ids": ids, "uid": f"t{i}",
                     "env_class": "synthetic_multiturn", "max_turns": turns, "obs_tokens": obs_tok,
                     "vocab_size": margs.vocab_size, "p": 0.3, "seed": 7919 * i + 1})
    ds = PromptDataset(rows, None, None)
    _wait_for_servers(urls)
    client = RemoteInferenceClient(urls, tokenizer=tok, model_name=model)
    trainer = FullyAsyncPPOTrainer(cfg, tokenizer=tok, train_dataset=ds, inference_engine_client=client, env=env)
    trainer.rollout_servers_in_box = True
    trainer.build_models()

    class Clock:
        """Step boundaries on the device clock: an event after every update, tokens from the step's metrics."""

        def __init__(self):
            self.events, self.tokens, self.gen, self.sync_ms, self.wall = [], [], [], [], []

        def on_step_end(self, tr, m):
            ev = torch.cuda.Event(enable_timing=True) if torch.cuda.is_available() else None
            if ev is not None:
                ev.record()
            self.events.append(ev)
            self.wall.append(time.perf_counter())
            self.tokens.append(m.get("trainer/num_tokens", 0.0))
            self.gen.append(m.get("trainer/num_generated_tokens", 0.0))
            self.sync_ms.append(m.get("timing/weight_sync_kernel_ms", 1e3 * m.get("timing/sync_weights", 0.0)))
            if env.is_main:
                print("[bench] update %d: " % len(self.events) + ", ".join(f"{k[7:]}={v:.3f}" for k, v in m.items()
                      if k.startswith("timing/")) + f", tokens={self.tokens[-1]:.0f}, staleness_max={m.get('async/staleness_max', 0):.0f}",
                      file=sys.stderr, flush=True)

        on_train_begin = on_train_end = lambda self, *a: None

    clock = Clock()
    trainer.callbacks.append(clock)
    sampler = ClockSampler(env.local_rank)
    if env.is_main:
        sampler.start()
    l0 = _lib.LAUNCH_COUNT
    try:
        trainer.train()
        W, K = args.warmup, args.steps
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            dev_s = clock.events[W - 1].elapsed_time(clock.events[W + K - 1]) / 1e3
        else:
            dev_s = clock.wall[W + K - 1] - clock.wall[W - 1]
        dev_s = pdist.all_reduce_max_scalar(dev_s, env.device)
        share = max(1, trainer.policy.tp_size)
        tokens = pdist.all_reduce_sum_scalar(sum(clock.tokens[W : W + K]), env.device) / share
        gen = pdist.all_reduce_sum_scalar(sum(clock.gen[W : W + K]), env.device) / share
        clocks = sampler.stop() if env.is_main else {}
        if env.is_main:
            status = _lib.status_read_clear() if torch.cuda.is_available() else 0
            print(json.dumps({
                "metric": METRIC, "value": (tokens + gen) / dev_s, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": dev_s * 1e3 / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic (uniform-random token ids, Bernoulli(0.3) reward at episode end, "
                "random-init weights)",
                "config": {"model": model, "baseline_config": 5, "algorithm": "grpo (rollout-anchored loss), fully asynchronous",
                           "parallelism": f"{n_train} training ranks (sharded optimizer x Ulysses sp{sp_size}) + {n_roll} "
                           "rollout-only ranks (one unsharded engine each)", "global_batch": P * n * n_train,
                           "trajectory": f"{turns} turns x ({turn_tok} generated + {obs_tok} observation tokens), prompt {plen}",
                           "seq_len": max_len, "tokens_counted": "trained (prompt + response) + generated tokens of the "
                           "updates in the timed window", "max_staleness_steps": 1,
                           "l2_policy": "inputs larger than L2 (15 GB of weights per rank)"},
                "clocks": clocks, "e2e": {"value": None, "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                                          "note": "the timed window is already end to end: requests and results cross HTTP"},
                "gpu_launches": _lib.LAUNCH_COUNT - l0, "device_status": status, "impl": "ours",
                "weight_sync_ms": float(sum(clock.sync_ms[W : W + K]) / max(1, K))}), flush=True)
    finally:
        if env.is_main:
            _shutdown_servers(urls)
        pdist.shutdown()


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
    ap.add_argument("--prefix-caching", type=int, default=1,
                    help="engine prefix cache: the n samples of a prompt share its key/value blocks and it is prefilled once")
    ap.add_argument("--no-e2e", action="store_true", help="skip the separately timed end-to-end steps (long configurations)")
    ap.add_argument("--turns", type=int, default=None, help="config 5: turns per trajectory")
    ap.add_argument("--obs-tokens", type=int, default=None, help="config 5: observation tokens appended after every turn")
    ap.add_argument("--max-tokens-per-microbatch", type=int, default=32768)
    ap.add_argument("--tp", type=int, default=None, help="tensor-parallel size of the training model (1 = sharded data parallel)")
    ap.add_argument("--ep", type=int, default=None, help="expert-parallel size (MoE models)")
    ap.add_argument("--pp", type=int, default=1, help="pipeline-parallel size of the training model")
    ap.add_argument("--sp", type=int, default=1, help="sequence-parallel size of the training model")
    ap.add_argument("--sp-backend", default="ulysses", choices=["ulysses", "context"],
                    help="ulysses: heads exchanged by all-to-all; context: keys / values all-gathered (context parallelism)")
    ap.add_argument("--engine-tp", type=int, default=None, help="tensor-parallel size of each rollout engine (lock-step ranks, "
                    "all-reduce in the o-proj / down-proj GEMM epilogues)")
    ap.add_argument("--reuse-train-forward", action="store_true",
                    help="take old log-probs from the training forward (exact with one optimizer update per step); "
                         "off by default so the step runs the same separate old-policy forward the reference does")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return
    if args.config == 5:
        run_disaggregated(args)
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
        f"generator.inference_engine.enable_prefix_caching={'true' if args.prefix_caching else 'false'}",
        "trainer.resume_mode=none", "trainer.seed=0",
        "trainer.logger=console", *(["trainer.strategy=megatron",
                                    f"trainer.policy.megatron_config.tensor_model_parallel_size={args.tp}"] if args.tp > 1 else []),
        *(["trainer.strategy=megatron", f"trainer.policy.megatron_config.expert_model_parallel_size={args.ep}"]
          if args.ep > 1 else []),
        *(["trainer.strategy=megatron", f"trainer.policy.megatron_config.pipeline_model_parallel_size={args.pp}"]
          if args.pp > 1 else []),
        *([f"trainer.policy.sequence_parallel_size={args.sp}", f"trainer.ref.sequence_parallel_size={args.sp}",
           f"trainer.sequence_parallel_backend={args.sp_backend}"] if args.sp > 1 else []),
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
                       "engine_tensor_parallel": args.engine_tp, "engine_prefix_caching": bool(args.prefix_caching),
                       "global_batch": P * n * world, "seq_len": PROMPT_LEN + RESP_MAX,
                       "parallelism": (f"dp{world} x ep{args.ep} (fused expert dispatch/combine)" if args.ep > 1 else
                                       f"dp{world // args.pp} x pp{args.pp} (layer stages)" if args.pp > 1 else
                                       (f"dp{world // args.sp} x cp{args.sp} (context parallel, key/value all-gather)" if args.sp_backend == "context"
                                        else f"dp{world // args.sp} x sp{args.sp} (Ulysses, fused projections)") if args.sp > 1 else
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
