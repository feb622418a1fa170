"""Tensor-parallel model for the generation engine: each rank holds ``1/tp`` of the attention heads (and of their
key/value cache) and ``1/tp`` of the FFN width; activations are replicated.

What the reference configures as ``generator.inference_engine.tensor_parallel_size`` and vLLM executes with worker
processes and an all-reduce after the o-proj and down-proj GEMMs
(skyrl/backends/skyrl_train/inference_servers/utils.py:89-100) is done here with the all-reduce *inside* the
row-parallel GEMM: its epilogue stores every finished tile into slot ``rank`` of a partial-sum buffer on every rank
of the group (``sb_gemm_tp`` in all-reduce layout, plain peer stores over NVLink), a device-side barrier follows, and
the consumer -- the fused residual-add + RMSNorm kernel on the decode path, a slot sum on the prefill path -- adds the
``tp`` slots in a fixed order.  Because every rank adds the same numbers in the same order, the residual stream, the
logits and therefore the sampled tokens are bit-identical on all ranks, so the ranks stay in lockstep without ever
exchanging a token: each runs its own copy of the scheduler on the same requests.

The parameter sharding is the one of ``models/tp_decoder.py`` (per-component slices of the fused QKV and gate/up
matrices), so a shard of the tensor-parallel trainer and a shard of this model are interchangeable at equal ``tp``.
Without CUDA peers (CPU tests over gloo) the same methods use ``torch.distributed.all_reduce``.
"""

from __future__ import annotations

import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..models.decoder import CausalLM, ModelArgs, _EmbeddingFn
from ..models.tp_decoder import local_args, shard_param
from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops import gemm
from ..parallel import tensor_parallel as tpm

PREFILL_CHANNELS = (4, 5)  # host-epoch barriers (eager launches)
DECODE_CHANNELS = (6, 7)   # device-epoch barriers (replayed from CUDA graphs)


class TPEngineModel(CausalLM):
    def __init__(self, full_args: ModelArgs, tp: tpm.TPGroup, device="cpu", dtype=torch.bfloat16,
                 flat_buffer: Optional[torch.Tensor] = None, seed: Optional[int] = None):
        self.full_args = full_args
        self.tp = tp
        super().__init__(local_args(full_args, tp.size), device=device, dtype=dtype, flat_buffer=flat_buffer, seed=None)
        self._slots: Dict[str, tuple] = {}
        if seed is not None:
            self.load_from_full(CausalLM(full_args, device="cpu", dtype=torch.float32, seed=seed))

    @torch.no_grad()
    def load_from_full(self, full: CausalLM) -> None:
        for name, prm in self.named_flat_views():
            prm.copy_(shard_param(name, full.p(name).detach(), self.full_args, self.tp.size, self.tp.rank).to(prm.dtype))

    # ------------------------------------------------------------------ partial-sum slots
    def slots(self, tag: str, rows: int, cols: int, dtype: torch.dtype):
        """Symmetric ``[tp, rows, cols]`` slot buffer for ``tag`` (grown collectively; every rank asks for the same
        sizes because the ranks run the same batches)."""
        cur = self._slots.get(tag)
        need = self.tp.size * rows * cols
        if cur is None or cur[0].local.numel() < need or cur[0].local.dtype != dtype:
            st = self.tp.peer.alloc(max(need, 1 << 16), dtype)
            self._slots[tag] = (st,)
            cur = self._slots[tag]
        return cur[0]

    def row_parallel_partials(self, x_local: torch.Tensor, w_shard: torch.Tensor, tag: str, dtype: torch.dtype,
                              channel: int, replayable: bool) -> torch.Tensor:
        """``x_local [T, K/tp] @ w_shard^T`` stored into slot ``rank`` of every rank's buffer; returns this rank's
        ``[tp, T, N]`` view once all ranks' partials have landed (the barrier is enqueued on the stream)."""
        T, N = x_local.shape[0], w_shard.shape[0]
        splits = 1
        if replayable and dtype == torch.float32 and T <= 256 and os.environ.get("SB_TP_DECODE_SPLITK", "0") == "1":
            # k slices would let a skinny GEMM use all SMs, but every slice's fp32 partial tile then crosses NVLink to
            # every rank: measured at 7B, 128 sequences, the step went from 6.45 ms to 8.52 ms.  Off unless asked for.
            splits = tpm.plan_scatter_splitk(T, N, x_local.shape[1])
        P = self.tp.size * splits
        st = self.slots(tag, T * splits, N, dtype)
        if splits > 1:
            tpm.gemm_all_reduce_partials(self.tp, x_local, w_shard, _View(st, P * T * N), splits)
        else:
            tpm.gemm_reduce_scatter(self.tp, x_local, w_shard, _View(st, P * T * N), T, all_ranks=True)
        if replayable:
            self.tp.peer.barrier_replayable(channel)
        else:
            self.tp.peer.barrier(channel)
        return st.local[: P * T * N].view(P, T, N)

    def row_parallel_linear(self, x_local: torch.Tensor, w_shard: torch.Tensor, tag: str, channel: int) -> torch.Tensor:
        """All-reduced ``[T, N]`` output (prefill path and CPU reference)."""
        if self.tp.fused and x_local.is_cuda:
            parts = self.row_parallel_partials(x_local.contiguous(), w_shard, tag, torch.bfloat16, channel, False)
            y = tpm.reduce_slots(parts, x_local.dtype)
            # the next writer of these slots is the same projection of the next layer; the other projection's barrier
            # lies in between on every rank, so no rank can overwrite slots that a peer is still summing
            return y
        y = gemm.gemm_nt(x_local, w_shard).float()
        if dist.is_initialized() and self.tp.size > 1:
            dist.all_reduce(y, group=self.tp.group)
        return y.to(x_local.dtype)

    # ------------------------------------------------------------------ prefill forward (replicated activations)
    def _layer(self, i: int, x, delta, pos, cu, max_seqlen, kv_sink=None, attn_fn=None):
        a = self.args
        pre = f"layers.{i}."
        x, h = ew.add_rmsnorm(x, delta, self.p(pre + "ln1"), a.rms_norm_eps)
        qkv = gemm.linear(h, self.p(pre + "wqkv"), self._p.get(pre + "bqkv"))
        if a.qk_norm:
            qkv = self._qk_norm(qkv, i)
        qkv = ew.rope(qkv, pos, self.rope_table(qkv.device), a.num_heads + a.num_kv_heads, a.head_dim)
        if kv_sink is not None:
            kv_sink(i, qkv)
        if attn_fn is not None:
            att = attn_fn(i, qkv)
        else:
            att = attn_ops.attn_varlen(qkv, cu, a.num_heads, a.num_kv_heads, a.head_dim, max_seqlen=max_seqlen)
        o = self.row_parallel_linear(att, self.p(pre + "wo"), "prefill_o", PREFILL_CHANNELS[0])
        x, h = ew.add_rmsnorm(x, o, self.p(pre + "ln2"), a.rms_norm_eps)
        act = ew.swiglu(gemm.linear(h, self.p(pre + "wgu")))
        d = self.row_parallel_linear(act, self.p(pre + "wd"), "prefill_d", PREFILL_CHANNELS[1])
        return x, d

    @torch.no_grad()
    def forward(self, input_ids, positions, cu_seqlens, max_seqlen: int = 0, kv_sink=None, attn_fn=None) -> torch.Tensor:
        x = _EmbeddingFn.apply(input_ids, self.p("embed"))
        delta = None
        for i in range(self.args.num_layers):
            x, delta = self._layer(i, x, delta, positions, cu_seqlens, max_seqlen, kv_sink, attn_fn)
        _, h = ew.add_rmsnorm(x, delta, self.p("final_norm"), self.args.rms_norm_eps)
        return h


class _View:
    """The leading ``numel`` elements of a symmetric tensor, with the peers' pointers (offset zero on all ranks)."""

    def __init__(self, st, numel: int):
        self.local = st.local[:numel]
        self.ptrs = st.ptrs
