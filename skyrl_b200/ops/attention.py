"""Attention ops: packed variable-length causal attention for training / prefill, paged-KV decode
attention for the generation engine, and the KV-cache scatter.

The packed layout is the one the reference feeds flash-attn with after ``unpad_input``
(skyrl/backends/skyrl_train/workers/model_wrapper.py:278-289,326-329): all sequences concatenated
along one token axis plus ``cu_seqlens``.  Here the kernels read Q, K and V straight out of the
fused-QKV projection output ``[T, (nq + 2 nkv) * D]`` through TMA, so no split/contiguous copy is made.
"""

from __future__ import annotations

import ctypes
import math
import os

import torch

from . import _lib

_cfg_done = False


def _k():
    global _cfg_done
    lib = _lib.kernels()
    if not _cfg_done:
        vp, ci, cf, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
        lib.sb_attn_fwd_varlen.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, cl, cf, vp]
        lib.sb_attn_bwd_varlen.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, cl, cf, vp]
        lib.sb_kv_cache_write.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, cl, ci, vp]
        lib.sb_attn_decode_paged.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, cl, cf, vp]
        lib.sb_attn_decode_paged_tc.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ci, cl, cf, vp]
        _cfg_done = True
    return lib


def _split(qkv, nq, nkv, D):
    T = qkv.shape[0]
    q = qkv[:, : nq * D].view(T, nq, D)
    k = qkv[:, nq * D : (nq + nkv) * D].view(T, nkv, D)
    v = qkv[:, (nq + nkv) * D :].view(T, nkv, D)
    return q, k, v


def attn_varlen_ref(qkv: torch.Tensor, cu_seqlens: torch.Tensor, nq: int, nkv: int, D: int, scale: float,
                    sinks: torch.Tensor | None = None):
    """fp32 PyTorch reference: returns (out [T, nq*D], lse [nq, T]).  ``sinks`` ([nq] logits): every row's softmax gets
    one more column with that logit and a zero value vector (it only enlarges the denominator)."""
    T = qkv.shape[0]
    q, k, v = _split(qkv.float(), nq, nkv, D)
    rep = nq // nkv
    out = torch.zeros(T, nq, D, dtype=torch.float32, device=qkv.device)
    lse = torch.zeros(nq, T, dtype=torch.float32, device=qkv.device)
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        if e <= s:
            continue
        qb = q[s:e].transpose(0, 1)  # [nq, L, D]
        kb = k[s:e].transpose(0, 1).repeat_interleave(rep, dim=0)
        vb = v[s:e].transpose(0, 1).repeat_interleave(rep, dim=0)
        sc = qb @ kb.transpose(1, 2) * scale
        L = e - s
        mask = torch.ones(L, L, dtype=torch.bool, device=qkv.device).tril()
        sc = sc.masked_fill(~mask, float("-inf"))
        if sinks is not None:
            sc = torch.cat([sc, sinks.float().view(nq, 1, 1).expand(nq, L, 1)], dim=-1)
            lse[:, s:e] = torch.logsumexp(sc, dim=-1)
            out[s:e] = (torch.softmax(sc, dim=-1)[..., :L] @ vb).transpose(0, 1)
            continue
        lse[:, s:e] = torch.logsumexp(sc, dim=-1)
        out[s:e] = (torch.softmax(sc, dim=-1) @ vb).transpose(0, 1)
    return out.reshape(T, nq * D).to(qkv.dtype), lse


class _AttnVarlenFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cu_seqlens, nq, nkv, D, scale, max_seqlen, sinks=None, q_begin=None):
        T = qkv.shape[0]
        B = cu_seqlens.numel() - 1
        if qkv.is_cuda:
            assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and cu_seqlens.dtype == torch.int32
            # with q_begin the kernel leaves the rows before each sequence's first query untouched: start from zeros
            alloc = torch.zeros if q_begin is not None else torch.empty
            out = alloc((T, nq * D), device=qkv.device, dtype=qkv.dtype)
            lse = alloc((nq, T), device=qkv.device, dtype=torch.float32)
            code = _k().sb_attn_fwd_varlen(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), cu_seqlens.data_ptr(),
                                           _lib.ptr(q_begin), B, T, nq, nkv, D, qkv.stride(0), scale, _lib.stream_ptr())
            _lib.check(code, "sb_attn_fwd_varlen")
            if sinks is not None:
                # A sink column only enlarges the denominator: with lse' = log(exp(lse) + exp(sink)) the output is the
                # plain one scaled by exp(lse - lse').  The backward kernels then see (out', lse') and are exact as
                # they stand, because the sink's value vector is zero.
                lse_s = torch.logaddexp(lse, sinks.float().view(nq, 1))
                gate = torch.exp(lse - lse_s).t().unsqueeze(-1)  # [T, nq, 1]
                out = (out.view(T, nq, D).float() * gate).to(qkv.dtype).view(T, nq * D)
                lse = lse_s
        else:
            out, lse = attn_varlen_ref(qkv, cu_seqlens, nq, nkv, D, scale, sinks)
        ctx.save_for_backward(qkv, out, lse, cu_seqlens, sinks, q_begin)
        ctx.meta = (nq, nkv, D, scale, max_seqlen)
        ctx.sink_main_grad = getattr(sinks, "main_grad", None) if sinks is not None else None
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, cu, sinks, q_begin = ctx.saved_tensors
        nq, nkv, D, scale, max_seqlen = ctx.meta
        T = qkv.shape[0]
        B = cu.numel() - 1

        def sink_grad(ds):
            """fp32 gradient of the sink logits: into ``main_grad`` when the parameter has one, else returned."""
            if ds is None:
                return None
            if ctx.sink_main_grad is not None:
                ctx.sink_main_grad.add_(ds.to(ctx.sink_main_grad.dtype))
                return None
            return ds.to(sinks.dtype)

        if qkv.is_cuda:
            dout = dout.contiguous()
            dqkv = torch.zeros_like(qkv) if q_begin is not None else torch.empty_like(qkv)
            delta = torch.empty(nq * T, device=qkv.device, dtype=torch.float32)
            code = _k().sb_attn_bwd_varlen(qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
                                           dqkv.data_ptr(), cu.data_ptr(), _lib.ptr(q_begin), delta.data_ptr(), B, T, nq, nkv, D,
                                           dqkv.stride(0),
                                           scale, _lib.stream_ptr())
            _lib.check(code, "sb_attn_bwd_varlen")
            ds = None
            if sinks is not None:
                # dS of the sink column = p_sink * (0 - delta), with delta = rowsum(dO * O) left in the workspace
                p_sink = torch.exp(sinks.float().view(nq, 1) - lse)
                ds = -(p_sink * delta.view(nq, T)).sum(1)
            return dqkv, None, None, None, None, None, None, sink_grad(ds), None
        with torch.enable_grad():
            x = qkv.detach().float().requires_grad_()
            sk = sinks.detach().float().requires_grad_() if sinks is not None else None
            o, _ = attn_varlen_ref(x, cu, nq, nkv, D, scale, sk)
            gs = torch.autograd.grad(o, (x,) if sk is None else (x, sk), dout.float())
        return g_cast(gs[0], qkv), None, None, None, None, None, None, sink_grad(gs[1] if sk is not None else None), None


def g_cast(g: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    return g.to(like.dtype)


def attn_varlen(qkv: torch.Tensor, cu_seqlens: torch.Tensor, nq: int, nkv: int, head_dim: int,
                scale: float | None = None, max_seqlen: int = 0, sinks: torch.Tensor | None = None,
                q_begin: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention over packed sequences. ``qkv``: ``[T, (nq+2nkv)*D]`` -> ``[T, nq*D]``.

    ``q_begin`` (``[B]`` int32): the rows of sequence ``b`` before ``q_begin[b]`` only serve as keys / values (a cached
    prefix, tokens owned by another context-parallel rank).  The CUDA kernels skip the 128-row query blocks that lie
    entirely before it, forward and backward; the output rows there are zero and must not be used.  The PyTorch
    reference path computes every row (the rows that matter are identical).

    ``sinks`` (``[nq]`` learned logits, GPT-OSS style): an extra softmax column per head that carries no value.  The
    reference gets it from a flex-attention score/mask patch compiled by inductor
    (skyrl/backends/skyrl_train/patches/gptoss/flex_attn_sink.py); here the tcgen05 kernels run unchanged and the sink
    enters through the log-sum-exp (see ``_AttnVarlenFn``)."""
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    return _AttnVarlenFn.apply(qkv, cu_seqlens, nq, nkv, head_dim, scale, max_seqlen, sinks, q_begin)


# ----------------------------------------------------------------------------- paged KV cache
def kv_cache_write(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, slots: torch.Tensor, nq: int,
                   nkv: int, D: int) -> None:
    """Scatter the K and V heads of each row of ``qkv`` into cache slot ``slots[t]`` (negative = skip).

    Caches are ``[num_blocks, block_size, nkv, D]``; a slot is ``block * block_size + offset``.
    """
    T = qkv.shape[0]
    _lib.check_index("kv_cache_write: cache slot", slots, k_cache.shape[0] * k_cache.shape[1], min_value=-(1 << 31))
    if qkv.is_cuda:
        code = _k().sb_kv_cache_write(qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), slots.data_ptr(), T, nq,
                                      nkv, D, qkv.stride(0), 0, _lib.stream_ptr())
        _lib.check(code, "sb_kv_cache_write")
        return
    _, k, v = _split(qkv, nq, nkv, D)
    kc = k_cache.view(-1, nkv, D)
    vc = v_cache.view(-1, nkv, D)
    ok = slots >= 0
    kc[slots[ok].long()] = k[ok]
    vc[slots[ok].long()] = v[ok]


def attn_decode_paged_ref(q, k_cache, v_cache, block_tables, ctx_lens, scale, sinks=None):
    n, nq, D = q.shape
    nkv = k_cache.shape[2]
    bs = k_cache.shape[1]
    rep = nq // nkv
    out = torch.zeros_like(q, dtype=torch.float32)
    for i in range(n):
        L = int(ctx_lens[i])
        if L == 0:
            continue
        nb = (L + bs - 1) // bs
        blocks = block_tables[i, :nb].long()
        kk = k_cache[blocks].reshape(-1, nkv, D)[:L].float().repeat_interleave(rep, dim=1)
        vv = v_cache[blocks].reshape(-1, nkv, D)[:L].float().repeat_interleave(rep, dim=1)
        s = torch.einsum("hd,lhd->hl", q[i].float(), kk) * scale
        if sinks is not None:
            pr = torch.softmax(torch.cat([s, sinks.float().view(nq, 1)], dim=-1), dim=-1)[:, :L]
        else:
            pr = torch.softmax(s, dim=-1)
        out[i] = torch.einsum("hl,lhd->hd", pr, vv)
    return out.to(q.dtype)


def attn_decode_paged(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                      ctx_lens: torch.Tensor, nq: int, nkv: int, D: int, scale: float | None = None,
                      out: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
                      max_ctx: int = 0, force_simt: bool = False, sinks: torch.Tensor | None = None) -> torch.Tensor:
    """One query token per sequence against its paged KV (which already contains that token).

    ``qkv``: ``[n, (nq+2nkv)*D]`` (only the q heads are read); ``block_tables``: ``[n, max_blocks]`` int32;
    ``ctx_lens``: ``[n]`` int32.  Returns ``[n, nq*D]``.  With ``sinks`` (see ``attn_varlen``) the PyTorch
    formulation runs on every device: the decode kernels do not return the log-sum-exp the sink would enter through.
    """
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    n = qkv.shape[0]
    if _lib.debug_bounds():
        bs_ = k_cache.shape[1]
        _lib.check_index("attn_decode_paged: context length", ctx_lens, block_tables.shape[1] * bs_ + 1)
        if ctx_lens.numel() and not (ctx_lens.is_cuda and torch.cuda.is_current_stream_capturing()):
            # only the table entries a sequence's context reaches are read
            used = (torch.arange(block_tables.shape[1], device=block_tables.device)[None, :] * bs_) < ctx_lens[:, None]
            _lib.check_index("attn_decode_paged: block table entry", block_tables[: ctx_lens.shape[0]][used], k_cache.shape[0])
    if not qkv.is_cuda or sinks is not None:
        q = qkv[:, : nq * D].reshape(n, nq, D)
        return attn_decode_paged_ref(q, k_cache, v_cache, block_tables, ctx_lens, scale, sinks).reshape(n, nq * D)
    if out is None:
        out = torch.empty((n, nq * D), device=qkv.device, dtype=qkv.dtype)
    bs = k_cache.shape[1]
    G = nq // nkv
    use_tc = (128 % bs == 0) and (bs % 8 == 0) and D == 128 and (G <= 8 or G in (12, 16)) and not force_simt
    mc = max_ctx if max_ctx > 0 else block_tables.shape[1] * bs
    splits = decode_num_splits_tc(n, nkv, mc) if use_tc else decode_num_splits(n, nkv, mc)
    if workspace is None and splits > 1:
        workspace = torch.empty(decode_workspace_floats(n, nq, D, splits), device=qkv.device, dtype=torch.float32)
    if use_tc:
        code = _k().sb_attn_decode_paged_tc(qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                            block_tables.data_ptr(), ctx_lens.data_ptr(), out.data_ptr(),
                                            _lib.ptr(workspace), n, nq, nkv, D, bs, k_cache.shape[0],
                                            block_tables.shape[1], splits, qkv.stride(0), scale, _lib.stream_ptr())
        _lib.check(code, "sb_attn_decode_paged_tc")
        return out
    code = _k().sb_attn_decode_paged(qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
                                     ctx_lens.data_ptr(), out.data_ptr(), _lib.ptr(workspace), n, nq, nkv, D, bs,
                                     block_tables.shape[1], splits, qkv.stride(0), scale, _lib.stream_ptr())
    _lib.check(code, "sb_attn_decode_paged")
    return out


def decode_num_splits_tc(n: int, nkv: int, max_ctx: int) -> int:
    """Context splits for the tensor-core decode kernel (one CTA per SM, 128-token tiles).

    The persistent kernel walks ``n * nkv * splits`` items round-robin over the SMs; a small cost model (measured on
    B200: about 1.8 us per tile, 1.5 us per item, 3 us for the combine pass that splits need) picks the split count
    with the least idle SM time in the last round.  ``SB_DECODE_ATTN_PERSIST=0`` selects the one-item-per-CTA kernel,
    which only splits when there are fewer items than SMs; ``SB_DECODE_ATTN_SPLITS`` forces a value (tuning)."""
    ctas = n * nkv
    forced = os.environ.get("SB_DECODE_ATTN_SPLITS")
    if forced:
        return int(max(1, min(int(forced), max(1, max_ctx // 128), 32)))
    if max_ctx <= 256:
        return 1
    if os.environ.get("SB_DECODE_ATTN_PERSIST", "1") == "0":
        if ctas >= 148:
            return 1
        want = (148 + ctas - 1) // ctas
        return int(max(1, min(want, max_ctx // 256, 32)))
    best, best_cost = 1, float("inf")
    for s in range(1, min(32, max_ctx // 256) + 1):
        tiles = (-(-max_ctx // s) + 127) // 128
        rounds = -(-ctas * s // 148)
        cost = rounds * (tiles * 1.8 + 1.5) + (3.0 if s > 1 else 0.0)
        if cost < best_cost - 0.5:  # ties go to fewer splits
            best, best_cost = s, cost
    return best


def decode_num_splits(n: int, nkv: int, max_ctx: int) -> int:
    """Split long contexts so that at least ~2 CTAs per SM are in flight."""
    ctas = n * nkv
    if ctas >= 296 or max_ctx <= 256:
        return 1
    want = (296 + ctas - 1) // ctas
    return int(max(1, min(want, max_ctx // 256, 32)))


def decode_workspace_floats(n: int, nq: int, D: int, splits: int) -> int:
    return n * nq * splits * (D + 2)
