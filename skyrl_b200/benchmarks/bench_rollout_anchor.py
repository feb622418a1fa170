"""Rollout phase anchor: the headline benchmark's generation workload, through this repo's engine and through the
vLLM installed on the machine (the role the reference fills with vLLM, skyrl/backends/skyrl_train/inference_servers/
vllm_server_actor.py; the image carries vLLM 0.22, not the reference's pinned 0.26).

    python -m skyrl_b200.benchmarks.bench_rollout_anchor --impl ours
    python -m skyrl_b200.benchmarks.bench_rollout_anchor --impl vllm

Workload = one GPU's share of BASELINE config 2: 32 prompts x 8 samples, each prompt 512 uniform-random token ids,
each sample forced to a length drawn uniformly in [256, 1024] (EOS ignored), temperature 1.0, chosen-token log-probs
returned, Qwen2.5-1.5B architecture with random weights, bf16.  One untimed round first (graph capture, compilation),
then ``--rounds`` timed rounds on fresh prompts; the time is the host clock around the blocking generate call, with a
device synchronisation on both sides where the caller owns the device.  This is a *phase anchor*: it compares the
generation phase only, not the RL step.
"""

from __future__ import annotations

import argparse
import json
import os
import tempfile
import time

import torch

from skyrl_b200.models.decoder import PRESETS


def workload(vocab: int, prompts: int, n: int, plen: int, lo: int, hi: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    p = torch.randint(4, vocab, (prompts, plen), generator=g).tolist()
    lens = torch.randint(lo, hi + 1, (prompts * n,), generator=g).tolist()
    rows = [p[i // n] for i in range(prompts * n)]
    return rows, lens


def run_ours(args, a):
    from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams
    from skyrl_b200.models.decoder import CausalLM

    m = CausalLM(a, device="cuda", dtype=torch.bfloat16, seed=0)
    S = args.prompts * args.n
    max_len = args.prompt_len + args.resp_max
    eng = LLMEngine(m, EngineConfig(block_size=32, max_num_seqs=S, max_model_len=max_len,
                                    max_num_batched_tokens=max(16384, max_len), gpu_memory_utilization=0.4,
                                    sync_interval=args.sync_interval))
    times, toks = [], []
    for r in range(args.rounds + 1):
        rows, lens = workload(a.vocab_size, args.prompts, args.n, args.prompt_len, args.resp_min, args.resp_max, 100 + r)
        sps = [SamplingParams(max_tokens=L, temperature=1.0, ignore_eos=True, logprobs=1) for L in lens]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = eng.generate(rows, sps)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        n_tok = sum(len(o.token_ids) for o in outs)
        assert n_tok == sum(lens), (n_tok, sum(lens))
        assert all(len(o.logprobs) == len(o.token_ids) for o in outs)
        if r > 0:
            times.append(dt)
            toks.append(n_tok)
    return times, toks


def run_vllm(args, a):
    os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
    from vllm import LLM, SamplingParams

    d = tempfile.mkdtemp(prefix="sb_vllm_model_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(a.to_hf_config(), f)
    S = args.prompts * args.n
    llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", seed=0,
              max_model_len=args.prompt_len + args.resp_max, max_num_seqs=S, gpu_memory_utilization=0.6,
              enable_prefix_caching=False, max_num_batched_tokens=16384)
    times, toks = [], []
    for r in range(args.rounds + 1):
        rows, lens = workload(a.vocab_size, args.prompts, args.n, args.prompt_len, args.resp_min, args.resp_max, 100 + r)
        sps = [SamplingParams(max_tokens=L, min_tokens=L, temperature=1.0, ignore_eos=True, logprobs=0, detokenize=False)
               for L in lens]
        t0 = time.perf_counter()
        outs = llm.generate([{"prompt_token_ids": p} for p in rows], sps, use_tqdm=False)
        dt = time.perf_counter() - t0
        n_tok = sum(len(o.outputs[0].token_ids) for o in outs)
        assert n_tok == sum(lens), (n_tok, sum(lens))
        if r > 0:
            times.append(dt)
            toks.append(n_tok)
    return times, toks


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "vllm"])
    ap.add_argument("--model", default="qwen2.5-1.5b")
    ap.add_argument("--prompts", type=int, default=32)
    ap.add_argument("--n", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--resp-min", type=int, default=256)
    ap.add_argument("--resp-max", type=int, default=1024)
    ap.add_argument("--rounds", type=int, default=3)
    ap.add_argument("--sync-interval", type=int, default=16, help="ours: decode steps between host harvests")
    args = ap.parse_args()
    a = PRESETS[args.model]
    times, toks = (run_ours if args.impl == "ours" else run_vllm)(args, a)
    best = min(range(len(times)), key=lambda i: times[i])
    out = {"impl": args.impl, "model": args.model, "sequences": args.prompts * args.n, "prompt_len": args.prompt_len,
           "response_len": f"uniform[{args.resp_min},{args.resp_max}]", "rounds": len(times),
           "seconds_per_round": [round(t, 4) for t in times], "generated_tokens_per_round": toks,
           "gen_tokens_per_s_mean": sum(toks) / sum(times), "gen_tokens_per_s_best": toks[best] / times[best]}
    if args.impl == "ours":
        out["sync_interval"] = args.sync_interval
    if args.impl == "vllm":
        import vllm

        out["vllm_version"] = vllm.__version__
    print("ROLLOUT_ANCHOR " + json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
