"""Training micro-benchmark: forward + backward (+ fused LM-head logprob) of one packed micro-batch, reporting
ms, model TFLOP/s and the fraction of the measured bf16 GEMM peak.

    python -m skyrl_b200.benchmarks.bench_train_step --model qwen2.5-1.5b --seqs 28 --seqlen 1152 --iters 3
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from skyrl_b200.models.decoder import PRESETS, CausalLM


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-1.5b")
    ap.add_argument("--seqs", type=int, default=28)
    ap.add_argument("--seqlen", type=int, default=1152)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--forward-only", action="store_true")
    ap.add_argument("--peak-tflops", type=float, default=float(os.environ.get("SB_BF16_TFLOPS", "1376.9")))
    args = ap.parse_args()
    a = PRESETS[args.model]
    m = CausalLM(a, device="cuda", dtype=torch.bfloat16, seed=0)
    m.attach_main_grad(torch.zeros(m.flat_numel, device="cuda", dtype=torch.float32))
    T = args.seqs * args.seqlen
    ids = torch.randint(4, a.vocab_size, (T,), device="cuda", dtype=torch.int32)
    pos = torch.arange(args.seqlen, device="cuda", dtype=torch.int32).repeat(args.seqs)
    cu = torch.arange(0, T + 1, args.seqlen, device="cuda", dtype=torch.int32)
    n_resp = T * 5 // 9
    pred = torch.randperm(T, device="cuda")[:n_resp].sort().values
    tgt = torch.randint(4, a.vocab_size, (n_resp,), device="cuda", dtype=torch.int32)

    def step():
        with torch.set_grad_enabled(not args.forward_only):
            h = m(ids, pos, cu, args.seqlen)
            lp, _ = m.token_logprobs(h[pred], tgt)
            if not args.forward_only:
                lp.sum().backward()

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.iters):
        step()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / args.iters
    dense = m.num_parameters() - a.vocab_size * a.hidden_size * (1 if a.tie_word_embeddings else 2)
    attn = 2 * 2 * a.num_layers * a.num_heads * a.head_dim * args.seqlen / 2  # causal QK^T + PV per token
    fwd = T * (2 * dense + attn) + n_resp * 2 * a.vocab_size * a.hidden_size
    flops = fwd if args.forward_only else 3 * fwd
    print(json.dumps({"model": args.model, "tokens": T, "mode": "fwd" if args.forward_only else "fwd+bwd", "ms": ms,
                      "tflops": flops / ms / 1e9, "fraction_of_measured_bf16_peak": flops / ms / 1e9 / args.peak_tflops,
                      "tokens_per_s": T / ms * 1e3}))


if __name__ == "__main__":
    main()
