"""Decode-step micro-benchmark: fills the engine with ``--seqs`` sequences of ``--ctx`` context tokens and
times decode steps (CUDA-graph replay or eager), reporting ms/step, tokens/s and the HBM roofline fraction
(weights + KV bytes that a step must read, over the measured copy bandwidth).

    python -m skyrl_b200.benchmarks.bench_decode_step --model qwen2.5-1.5b --seqs 256 --ctx 900 --steps 32
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m skyrl_b200.benchmarks.bench_decode_step \
        --model qwen2.5-7b --seqs 128 --ctx 3000 --tp 2      # tensor-parallel engine (one rank per GPU)
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams
from skyrl_b200.models.decoder import PRESETS, CausalLM


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-1.5b")
    ap.add_argument("--seqs", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=900)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--no-fused", action="store_true", help="plain GEMMs instead of split-K + fused consumers")
    ap.add_argument("--mlp-block", action="store_true", help="persistent o-proj..down-proj kernel per layer")
    ap.add_argument("--hbm-gbs", type=float, default=float(os.environ.get("SB_HBM_GBS", "6543.4")))
    ap.add_argument("--tp", type=int, default=1, help="engine tensor-parallel size (= number of ranks launched)")
    args = ap.parse_args()
    a = PRESETS[args.model]
    rank = 0
    if args.tp > 1:
        from skyrl_b200.engine.tp_model import TPEngineModel
        from skyrl_b200.parallel import dist as pdist
        from skyrl_b200.parallel import tensor_parallel as tpm
        from skyrl_b200.parallel.peer import PeerContext

        env = pdist.init_distributed()
        assert env.world_size == args.tp, "launch one rank per tensor-parallel shard"
        rank = env.rank
        tp = tpm.TPGroup(PeerContext(env.device), None)
        m = TPEngineModel(a, tp, device=env.device, dtype=torch.bfloat16)
        m.flat_params.normal_(0.0, 0.02)  # timing only: the shards need no consistent full model
        for name, prm in m.named_flat_views():
            if name.split(".")[-1] in ("ln1", "ln2", "final_norm"):
                prm.data.fill_(1.0)
    else:
        m = CausalLM(a, device="cuda", dtype=torch.bfloat16, seed=None)
        m.flat_params.normal_(0.0, 0.02)  # timing only: drawn on the device (a host generator takes minutes for 7B)
        for name, prm in m.named_flat_views():
            if name.split(".")[-1] in ("ln1", "ln2", "final_norm"):
                prm.data.fill_(1.0)
    max_len = args.ctx + args.steps * 3 + 64
    eng = LLMEngine(m, EngineConfig(block_size=32, max_num_seqs=args.seqs, max_model_len=max_len,
                                    max_num_batched_tokens=1 << 20, enforce_eager=args.eager, sync_interval=args.steps, fused_decode=not args.no_fused, fused_mlp_block=args.mlp_block,
                                    num_blocks=args.seqs * ((max_len + 31) // 32) + 8))
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(4, a.vocab_size, (args.seqs, args.ctx), generator=g).tolist()
    sp = SamplingParams(max_tokens=args.steps * 3 + 8, temperature=1.0, ignore_eos=True)
    for i, p in enumerate(prompts):
        eng.add_request(f"r{i}", p, sp)
    eng.step()  # prefill + first `steps` decode steps (also captures the graph)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    eng._run_decode(args.steps)
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / args.steps
    ctx_now = args.ctx + args.steps * 1.5
    kv_bytes = args.seqs * ctx_now * 2 * a.num_layers * m.args.num_kv_heads * a.head_dim * 2  # this rank's share
    w_bytes = (m.num_parameters()) * 2
    ideal_ms = (kv_bytes + w_bytes) / (args.hbm_gbs * 1e9) * 1e3
    if rank == 0:
        print(json.dumps({"tp": args.tp, "model": args.model, "seqs": args.seqs, "ctx": args.ctx,
                          "mode": "eager" if args.eager else "graph", "fused": not args.no_fused, "mlp_block": args.mlp_block, "ms_per_step": ms,
                          "tokens_per_s": args.seqs / ms * 1e3, "hbm_bytes_per_step_per_rank": kv_bytes + w_bytes,
                          "roofline_ms": ideal_ms, "fraction_of_measured_hbm_roofline": ideal_ms / ms}))
    if args.tp > 1:
        from skyrl_b200.ops import _lib
        from skyrl_b200.parallel import dist as pdist

        assert _lib.status_read_clear() == 0
        pdist.shutdown()


if __name__ == "__main__":
    main()
