"""Kernel micro-benchmarks with roofline fractions against the measured peaks of the machine.

    python -m skyrl_b200.benchmarks.bench_kernels --which gemm --m 4096 --n 4096 --k 4096
    python -m skyrl_b200.benchmarks.bench_kernels --which decode_attn --seqs 64 --ctx 1024
    python -m skyrl_b200.benchmarks.bench_kernels --which attn --seqs 8 --seqlen 2048
    python -m skyrl_b200.benchmarks.bench_kernels --which lmhead --tokens 4096

Peaks default to the values measured on the B200 pool (copy bandwidth 6543.4 GB/s, bf16 GEMM 1668.8 TFLOP/s burst /
1376.9 sustained) and can be overridden with --hbm-gbs / --peak-tflops.
"""

from __future__ import annotations

import argparse
import json
import math

import torch

from skyrl_b200.ops import attention, gemm, lm_head


def timeit(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    flush = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
    tot = 0.0
    for _ in range(iters):
        flush.zero_()  # evict L2 between timed iterations
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        tot += s.elapsed_time(e)
    return tot / iters


def load_reference_module(rel_path: str, name: str):
    """Import one file of the unmodified reference install under ``baseline/_ref`` by path (no package import, so
    none of the reference's heavier dependencies is pulled in)."""
    import importlib.util
    import os
    import sys

    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "baseline", "_ref", rel_path)
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path}: install the reference into baseline/_ref first")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _bench_lmhead(a) -> dict:
    """Fused LM-head log-probability, forward and forward+backward, at ``--tokens`` x ``--vocab`` x ``--hidden-lm``.

    ``--impl ours``: ``ops.lm_head.lm_head_logprobs`` (tcgen05 main loop, online-softmax epilogue, no logits).
    ``--impl reference``: the reference's own kernels on the same tensors, loaded unmodified from ``baseline/_ref``:
    its vendored Triton fused LM-head (``FusedLinearLogprobTriton``, the path ``fused_lm_head_logprob`` enables) and
    its materialised-logits path (``logits = h @ W^T`` -> ``logprobs_from_logits`` + ``chunked_entropy_from_logits``,
    the FSDP default).  ``--impl both`` runs all three back to back in one process and prints the ratios.
    """
    T, V, H = a.tokens, a.vocab, a.hidden_lm
    g = torch.Generator(device="cuda").manual_seed(0)
    h = (torch.randn(T, H, device="cuda", generator=g) * 0.5).to(torch.bfloat16).requires_grad_()
    W = (torch.randn(V, H, device="cuda", generator=g) * 0.02).to(torch.bfloat16).requires_grad_()
    tgt = torch.randint(0, V, (T,), device="cuda", generator=g)
    gout = torch.randn(T, device="cuda", generator=g)
    fl = 2.0 * T * V * H
    res = {"tokens": T, "vocab": V, "hidden": H, "impl": a.impl}

    def fwd_bwd(fn):
        def run():
            h.grad = W.grad = None
            lp = fn(h, W)
            lp.backward(gout)
        return run

    def record(tag, fn, check_against=None):
        with torch.no_grad():
            ms_f = timeit(lambda: fn(h, W), a.iters)
        ms_fb = timeit(fwd_bwd(fn), a.iters)
        row = {"fwd_ms": ms_f, "fwd_tflops": fl / ms_f / 1e9, "fwd_bwd_ms": ms_fb, "fwd_bwd_tflops": 3 * fl / ms_fb / 1e9,
               "fwd_fraction_of_measured_bf16_burst": fl / ms_f / 1e9 / a.peak_tflops}
        with torch.no_grad():
            lp = fn(h, W).float()
        if check_against is not None:
            row["max_abs_diff_vs_ours"] = (lp - check_against).abs().max().item()
        res[tag] = row
        return lp

    ours_lp = None
    if a.impl in ("ours", "both"):
        ours_lp = record("ours", lambda hh, ww: lm_head.lm_head_logprobs(hh, ww, tgt, 1.0)[0])
    if a.impl in ("reference", "both"):
        ref_fused = load_reference_module("skyrl/backends/skyrl_train/distributed/megatron/fused_linear_logprob_triton.py",
                                          "ref_fused_linear_logprob_triton")
        ref_tu = load_reference_module("skyrl/backends/skyrl_train/utils/torch_utils.py", "ref_torch_utils")
        t2 = tgt.view(1, T)

        def ref_triton(hh, ww):
            return ref_fused.FusedLinearLogprobTriton.apply(hh.view(1, T, H), ww, t2, 0, V, 1024, None, False).view(T)

        def ref_logits(hh, ww):
            logits = (hh @ ww.t()).view(1, T, V)
            lp = ref_tu.logprobs_from_logits(logits, t2, inplace_backward=True)
            return lp.view(T)

        record("reference_triton_fused", ref_triton, ours_lp)
        if T * V * 2 <= 24 << 30:  # the materialised path needs T x V bf16 logits (+ the same again in backward)
            record("reference_materialised_logits", ref_logits, ours_lp)
            with torch.no_grad():
                logits = (h @ W.t()).view(1, T, V)
                res["reference_chunked_entropy_ms"] = timeit(lambda: ref_tu.chunked_entropy_from_logits(logits), a.iters)
                del logits
        else:
            res["reference_materialised_logits"] = {"skipped": "logits would not fit the bound set for this benchmark"}
    if a.impl == "both":
        for tag in ("reference_triton_fused", "reference_materialised_logits"):
            if "fwd_ms" in res.get(tag, {}):
                res[tag]["fwd_speedup_ours"] = res[tag]["fwd_ms"] / res["ours"]["fwd_ms"]
                res[tag]["fwd_bwd_speedup_ours"] = res[tag]["fwd_bwd_ms"] / res["ours"]["fwd_bwd_ms"]
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "both"], help="lmhead: which implementation to time")
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--hidden-lm", type=int, default=1536)
    ap.add_argument("--which", default="gemm", choices=["gemm", "decode_attn", "attn", "lmhead", "tp_gather", "tp_scatter", "moe", "elementwise", "relayout",
                             "decode_block"])
    ap.add_argument("--layers", type=int, default=8, help="relayout: decoder layers of the Qwen2.5-1.5B-shaped source model")
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=768)
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--layout", default="nt", choices=["nt", "nn", "tn"])
    ap.add_argument("--seqs", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--seqlen", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--nq", type=int, default=12)
    ap.add_argument("--nkv", type=int, default=2)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--block-size", type=int, default=32, help="decode_attn: tokens per KV-cache page")
    ap.add_argument("--graph", action="store_true", help="decode_attn: time a CUDA-graph replay of several calls")
    ap.add_argument("--hbm-gbs", type=float, default=6543.4)
    ap.add_argument("--peak-tflops", type=float, default=1668.8)
    a = ap.parse_args()
    bf = dict(device="cuda", dtype=torch.bfloat16)
    out = {"which": a.which}
    if a.which == "gemm":
        if a.layout == "nt":
            x, w = torch.randn(a.m, a.k, **bf), torch.randn(a.n, a.k, **bf)
            fn = lambda: gemm.gemm_nt(x, w)  # noqa: E731
        elif a.layout == "nn":
            x, w = torch.randn(a.m, a.k, **bf), torch.randn(a.k, a.n, **bf)
            fn = lambda: gemm.gemm_nn(x, w)  # noqa: E731
        else:
            x, w = torch.randn(a.k, a.m, **bf), torch.randn(a.k, a.n, **bf)
            fn = lambda: gemm.gemm_tn(x, w)  # noqa: E731
        ms = timeit(fn, a.iters)
        fl = 2.0 * a.m * a.n * a.k
        out.update(m=a.m, n=a.n, k=a.k, layout=a.layout, ms=ms, tflops=fl / ms / 1e9,
                   fraction_of_measured_bf16_burst=fl / ms / 1e9 / a.peak_tflops)
    elif a.which == "decode_attn":
        bs, D = a.block_size, 128
        mb = (a.ctx + bs - 1) // bs
        nb = a.seqs * mb
        kc, vc = torch.randn(nb, bs, a.nkv, D, **bf), torch.randn(nb, bs, a.nkv, D, **bf)
        bt = torch.arange(nb, device="cuda", dtype=torch.int32).view(a.seqs, mb)
        cl = torch.full((a.seqs,), a.ctx, device="cuda", dtype=torch.int32)
        qkv = torch.randn(a.seqs, (a.nq + 2 * a.nkv) * D, **bf)
        if a.graph:
            # GPU time without host launch gaps: `reps` calls captured in one CUDA graph, each on its own cache copy
            # (together larger than L2) so that no call finds its K/V in cache
            reps = max(2, int(300e6 // (2 * nb * bs * a.nkv * D * 2)) + 1)
            caches = [(kc, vc)] + [(torch.randn_like(kc), torch.randn_like(vc)) for _ in range(reps - 1)]
            outb = torch.empty(a.seqs, a.nq * D, **bf)
            ws = torch.empty(attention.decode_workspace_floats(a.seqs, a.nq, D, 32), device="cuda", dtype=torch.float32)
            run = lambda: [attention.attn_decode_paged(qkv, k_, v_, bt, cl, a.nq, a.nkv, D, max_ctx=a.ctx, out=outb,  # noqa: E731
                                                       workspace=ws) for k_, v_ in caches]
            run()
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                run()
            ms = timeit(gr.replay, a.iters) / reps
        else:
            ms = timeit(lambda: attention.attn_decode_paged(qkv, kc, vc, bt, cl, a.nq, a.nkv, D, max_ctx=a.ctx), a.iters)
        by = 2.0 * a.seqs * a.ctx * a.nkv * D * 2
        out.update(seqs=a.seqs, ctx=a.ctx, ms=ms, gbs=by / ms / 1e6, fraction_of_measured_hbm=by / ms / 1e6 / a.hbm_gbs)
    elif a.which == "attn":
        D = 128
        T = a.seqs * a.seqlen
        qkv = (torch.randn(T, (a.nq + 2 * a.nkv) * D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
        cu = torch.arange(0, T + 1, a.seqlen, device="cuda", dtype=torch.int32)
        ms_f = timeit(lambda: attention.attn_varlen(qkv.detach(), cu, a.nq, a.nkv, D), a.iters)
        o = attention.attn_varlen(qkv, cu, a.nq, a.nkv, D)
        g = torch.randn_like(o)
        ms_b = timeit(lambda: torch.autograd.grad(o, qkv, g, retain_graph=True), a.iters)
        fl = 4.0 * a.seqs * a.nq * a.seqlen * a.seqlen * D / 2
        out.update(tokens=T, seqlen=a.seqlen, fwd_ms=ms_f, fwd_tflops=fl / ms_f / 1e9, bwd_ms=ms_b,
                   bwd_tflops=2.5 * fl / ms_b / 1e9, fwd_fraction_of_measured_bf16_burst=fl / ms_f / 1e9 / a.peak_tflops)
        if a.impl in ("reference", "both"):
            # anchor: the library the reference calls for this op (flash-attn varlen, model_wrapper.py:326-329), same
            # tensors (its kernels are not part of this package's hot path: timing only)
            from flash_attn import flash_attn_varlen_func

            q, k, v = (t.detach().contiguous().requires_grad_() for t in (
                qkv[:, : a.nq * D].view(T, a.nq, D), qkv[:, a.nq * D : (a.nq + a.nkv) * D].view(T, a.nkv, D),
                qkv[:, (a.nq + a.nkv) * D :].view(T, a.nkv, D)))
            fa = lambda: flash_attn_varlen_func(q, k, v, cu, cu, a.seqlen, a.seqlen, causal=True)  # noqa: E731
            ms_rf = timeit(lambda: fa().detach(), a.iters)
            ro = fa()
            err = (ro.reshape(T, -1).float() - o.float()).abs().max().item()
            ms_rb = timeit(lambda: torch.autograd.grad(ro, (q, k, v), g.view_as(ro), retain_graph=True), a.iters)
            import flash_attn

            out.update(flash_attn_version=flash_attn.__version__, ref_fwd_ms=ms_rf, ref_fwd_tflops=fl / ms_rf / 1e9,
                       ref_bwd_ms=ms_rb, ref_bwd_tflops=2.5 * fl / ms_rb / 1e9, fwd_speedup=ms_rf / ms_f,
                       bwd_speedup=ms_rb / ms_b, max_abs_diff_vs_flash_attn=err)
    elif a.which in ("tp_gather", "tp_scatter"):
        # Tensor-parallel GEMM modes with the ranks emulated by separate buffers of this GPU (the kernel code path --
        # copy warps reading "peer" shards, epilogue storing into "peer" slots -- is the one used across GPUs; only
        # the link is missing, so this measures kernel overhead, not NVLink).
        import ctypes

        from skyrl_b200.ops import _lib
        from skyrl_b200.parallel import tensor_parallel as tpm

        R = 4  # emulated ranks
        M, K, N = a.m, a.k, a.n
        rpr = M // R
        lib = tpm._k()
        w = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
        if a.which == "tp_gather":
            shards = [(torch.randn(rpr, K, device="cuda") * 0.5).to(torch.bfloat16) for _ in range(R)]
            a_full = torch.zeros(M, K, **bf)
            a_full[:rpr] = shards[0]
            outp = torch.empty(M, N, **bf)
            flags = torch.zeros(M // 128 + 2, dtype=torch.int32, device="cuda")
            peers = (ctypes.c_void_p * R)(*[t.data_ptr() for t in shards])
            fn = lambda: _lib.check(lib.sb_gemm_tp(a_full.data_ptr(), w.data_ptr(), outp.data_ptr(), None, M, N, K, K, K, N, 0, 0, 1, 0,  # noqa: E731
                                                   peers, None, R, 0, rpr, 0, flags.data_ptr(), 0, _lib.stream_ptr()), "tp")
        else:
            x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
            dests = [torch.empty(R, rpr, N, **bf) for _ in range(R)]
            outs = (ctypes.c_void_p * R)(*[t.data_ptr() for t in dests])
            fn = lambda: _lib.check(lib.sb_gemm_tp(x.data_ptr(), w.data_ptr(), None, None, M, N, K, K, K, N, 0, 0, 0, 1, None,  # noqa: E731
                                                   outs, R, 0, rpr, rpr * N, None, 0, _lib.stream_ptr()), "tp")
        ms = timeit(fn, a.iters)
        fl = 2.0 * M * N * K
        out.update(m=M, n=N, k=K, emulated_ranks=R, ms=ms, tflops=fl / ms / 1e9,
                   fraction_of_measured_bf16_burst=fl / ms / 1e9 / a.peak_tflops)
    elif a.which == "relayout":
        # weight-sync re-layout kernel on one GPU: an unsharded trainer buffer is re-sliced into the two shards of a
        # TP=2 engine (both destination buffers local, so the copies run at HBM speed: read + write of every byte)
        import dataclasses

        from skyrl_b200.models.decoder import PRESETS, flat_numel_for, param_offsets
        from skyrl_b200.models.tp_decoder import local_args
        from skyrl_b200.weight_sync import relayout as rlo

        args_full = dataclasses.replace(PRESETS["qwen2.5-1.5b"], num_layers=a.layers, tie_word_embeddings=False)
        src = torch.randn(flat_numel_for(args_full), device="cuda").to(torch.bfloat16)
        largs = local_args(args_full, 2)
        dsts = [torch.zeros(flat_numel_for(largs), **bf) for _ in range(2)]
        dests = [rlo.Destination(d.data_ptr(), param_offsets(largs), 2, r) for r, d in enumerate(dsts)]
        plan = rlo.build_plan(args_full, param_offsets(args_full), 1, 0, dests)
        push = rlo.RelayoutPush(plan, src, dests)
        ms = timeit(push.run, a.iters)
        moved = 2.0 * push.bytes_out  # read + write
        out.update(layers=a.layers, block_copies=push.n_desc, work_items=push.n_items, bytes_out=push.bytes_out, ms=ms,
                   gbs_read_plus_write=moved / ms / 1e6, fraction_of_measured_hbm=moved / ms / 1e6 / a.hbm_gbs)
    elif a.which == "decode_block":
        # persistent decode block kernel (o-proj .. down-proj of one layer, Qwen2.5-1.5B shapes): one warm launch with
        # every CTA's clock recorded at the phase boundaries; prints when the last CTA finished each phase
        from skyrl_b200.ops import _lib
        from skyrl_b200.ops import elementwise as ew

        H, Q, F, n = 1536, 1536, 8960, a.seqs
        g = torch.Generator(device="cuda").manual_seed(0)
        rnd = lambda *s, scale=1.0: (torch.randn(*s, device="cuda", generator=g) * scale).to(torch.bfloat16)  # noqa: E731
        att, x = rnd(n, Q), rnd(n, H)
        wo, wgu, wd = rnd(H, Q, scale=Q ** -0.5), rnd(2 * F, H, scale=H ** -0.5), rnd(H, F, scale=F ** -0.5)
        ln = torch.ones(H, **bf)
        ws = ew.DecodeMlpWorkspace(256, H, Q, F, "cuda")
        for _ in range(3):
            ew.decode_mlp_block(att, x.clone(), wo, ln, wgu, wd, ln, 1e-6, ws)
        torch.cuda.synchronize()
        ws.trace = torch.zeros(torch.cuda.get_device_properties(0).multi_processor_count, 16, device="cuda", dtype=torch.int64)
        ms = timeit(lambda: ew.decode_mlp_block(att, x.clone(), wo, ln, wgu, wd, ln, 1e-6, ws), a.iters)
        t = ws.trace.cpu().double()
        t0 = t[:, 0].min()
        names = ["o-proj", "barrier 1", "norm", "barrier 2", "gate/up + SwiGLU", "barrier 3", "down-proj", "barrier 4", "norm"]
        out.update(rows=n, ms_per_launch_with_clone=ms, device_status=_lib.status_read_clear(),
                   all_ctas_done_us={nm: round(float((t[:, k + 1].max() - t0) / 1e3), 2) for k, nm in enumerate(names)})
    elif a.which == "elementwise":
        # the bandwidth-bound kernels of a step: achieved bytes / s against the measured copy bandwidth
        from skyrl_b200.ops import elementwise as ew, optim, sampling

        T, H, F, V = a.tokens, 1536, 8960, 151936
        x = torch.randn(T, H, **bf)
        d = torch.randn(T, H, **bf)
        w = torch.ones(H, **bf)
        gu = torch.randn(T, 2 * F, **bf)
        rows = []

        def rec(name, nbytes, fn):
            ms = timeit(fn, a.iters)
            rows.append({"kernel": name, "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1),
                         "fraction_of_measured_hbm": round(nbytes / ms / 1e6 / a.hbm_gbs, 3)})

        with torch.no_grad():
            rec("add_rmsnorm fwd (residual add + norm)", 4 * T * H * 2, lambda: ew.add_rmsnorm(x, d, w, 1e-6))
            rec("swiglu fwd", 3 * T * F * 2, lambda: ew.swiglu(gu))
            dact = torch.randn(T, F, **bf)
            rec("swiglu bwd", 5 * T * F * 2, lambda: ew.swiglu_backward(gu, dact))
            qkv = torch.randn(T, 16 * 128, **bf)
            pos = torch.arange(T, device="cuda", dtype=torch.int32) % 2048
            table = ew.build_rope_table(4096, 128, 1e6, "cuda")
            rec("rope in place (12 q + 2 k heads)", 2 * T * 14 * 128 * 2, lambda: ew.rope_(qkv, pos, table, 14, 128))
            n = 1_543_000_000 // 8  # one rank's optimizer shard of a 1.5B model at 8 GPUs
            master, m_, v_ = (torch.zeros(n, device="cuda") for _ in range(3))
            grad = torch.randn(n, device="cuda")
            param = torch.zeros(n, **bf)
            rec("adamw_flat (fp32 master/m/v, bf16 param out)", n * (4 * 4 + 3 * 4 + 2),
                lambda: optim.adamw_flat(master, m_, v_, grad, param, 1e-5, 0.9, 0.999, 1e-8, 0.01, 1))
            logits = torch.randn(256, V, **bf)
            temp = torch.ones(256, device="cuda")
            rec("sample (gumbel + log-prob, 256 x 151936 bf16 logits)", 256 * V * 2, lambda: sampling.sample(logits, temp, 1))
        out.update(tokens=T, rows=rows)
    elif a.which == "moe":
        # one mixture-of-experts FFN layer (router, grouped gate/up GEMM, SwiGLU, grouped down GEMM, weighted combine)
        from skyrl_b200.models.moe import moe_ffn
        from skyrl_b200.ops import grouped_gemm as gg

        T, H, E, F, k = a.tokens, a.hidden, a.experts, a.ffn, a.topk
        h = (torch.randn(T, H, device="cuda") * 0.5).to(torch.bfloat16)
        rt = (torch.randn(E, H, device="cuda") * 0.5).to(torch.bfloat16)
        wgu = (torch.randn(E, 2 * F, H, device="cuda") * 0.02).to(torch.bfloat16)
        wd = (torch.randn(E, H, F, device="cuda") * 0.02).to(torch.bfloat16)
        with torch.no_grad():
            ms_layer = timeit(lambda: moe_ffn(h, rt, wgu, wd, k, True), a.iters)
            ids = torch.randint(0, E, (T * k,), device="cuda")
            plan = gg.plan_groups(ids, E)
            x = torch.zeros((plan.m_cap, H), **bf)
            ms_gu = timeit(lambda: gg.grouped_nt(x, wgu, plan), a.iters)
            act = torch.zeros((plan.m_cap, F), **bf)
            ms_dn = timeit(lambda: gg.grouped_nt(act, wd, plan), a.iters)
        fl_gu, fl_dn = 2.0 * T * k * 2 * F * H, 2.0 * T * k * F * H
        out.update(tokens=T, hidden=H, experts=E, ffn=F, topk=k, padded_rows=plan.m_cap, layer_fwd_ms=ms_layer,
                   gate_up_ms=ms_gu, gate_up_tflops=fl_gu / ms_gu / 1e9, down_ms=ms_dn, down_tflops=fl_dn / ms_dn / 1e9,
                   layer_tflops=(fl_gu + fl_dn) / ms_layer / 1e9)
    else:
        out.update(_bench_lmhead(a))
    print(json.dumps(out))


if __name__ == "__main__":
    main()
