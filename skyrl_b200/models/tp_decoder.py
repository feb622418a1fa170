"""Tensor-parallel decoder (Megatron-style TP with sequence-parallel activations) on the fused GEMM collectives.

Each rank holds ``1/tp`` of the attention heads and of the FFN width; the residual stream, norms and the LM head
work on ``1/tp`` of the packed tokens.  Per layer there are two all-gather+GEMM kernels (QKV, gate/up) and two
GEMM+reduce-scatter kernels (o-proj, down-proj); see ``parallel/tensor_parallel.py``.  This is the training-side
counterpart of what the reference configures through Megatron-Bridge
(skyrl/backends/skyrl_train/workers/megatron/megatron_worker.py:377-545, parallel sizes :468-474) and executes in
``MegatronModelWrapper.forward`` (megatron_model_wrapper.py:285-528) -- but the layer math is the same packed,
varlen code as the unsharded model, instantiated with the local head / FFN counts.

The packed token count must be a multiple of ``tp * 128`` (``pad_packed_for_tp``): the gather kernel moves whole
128-row blocks.  Parameters that every rank replicates (embedding, norms, LM head) receive the sum of the ranks'
gradients through ``reduce_replicated_grads`` before the optimizer step.
"""

from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..parallel import tensor_parallel as tpm
from .decoder import CausalLM, ModelArgs, _EmbeddingFn

REPLICATED_LEAVES = ("embed", "ln1", "ln2", "final_norm", "lm_head", "q_norm", "k_norm", "value_head")


def local_args(a: ModelArgs, tp: int, vocab_parallel_head: bool = False) -> ModelArgs:
    if vocab_parallel_head:
        if a.tie_word_embeddings or a.vocab_size % tp:
            raise ValueError("a vocabulary-parallel LM head needs untied embeddings and a vocabulary divisible by tp "
                             f"(tie_word_embeddings={a.tie_word_embeddings}, vocab_size={a.vocab_size}, tp={tp})")
        return dataclasses.replace(local_args(a, tp), lm_head_rows=a.vocab_size // tp)
    if a.num_heads % tp or a.intermediate_size % tp:
        raise ValueError(f"num_heads={a.num_heads} and intermediate_size={a.intermediate_size} must divide by tp={tp}")
    if a.num_kv_heads % tp:
        raise ValueError(f"num_kv_heads={a.num_kv_heads} must divide by tp={tp} (KV-head replication is not supported)")
    if a.num_experts:
        raise ValueError("tensor parallelism of MoE layers is expert-parallel; use the EP path")
    return dataclasses.replace(a, num_heads=a.num_heads // tp, num_kv_heads=a.num_kv_heads // tp,
                               intermediate_size=a.intermediate_size // tp)


def shard_param(name: str, full: torch.Tensor, a: ModelArgs, tp: int, r: int, vocab_parallel_head: bool = False) -> torch.Tensor:
    """Rank ``r``'s slice of a full parameter (fused QKV and gate/up are sliced per component)."""
    leaf = name.split(".")[-1]
    if leaf == "lm_head" and vocab_parallel_head:
        vs = a.vocab_size // tp
        return full[r * vs : (r + 1) * vs]
    if leaf in ("wqkv", "bqkv"):
        q, k, v = full[: a.q_dim], full[a.q_dim : a.q_dim + a.kv_dim], full[a.q_dim + a.kv_dim :]
        qs, ks = a.q_dim // tp, a.kv_dim // tp
        return torch.cat([q[r * qs : (r + 1) * qs], k[r * ks : (r + 1) * ks], v[r * ks : (r + 1) * ks]], 0)
    if leaf == "wo":
        qs = a.q_dim // tp
        return full[:, r * qs : (r + 1) * qs]
    if leaf == "wgu":
        F, fs = a.intermediate_size, a.intermediate_size // tp
        return torch.cat([full[r * fs : (r + 1) * fs], full[F + r * fs : F + (r + 1) * fs]], 0)
    if leaf == "wd":
        fs = a.intermediate_size // tp
        return full[:, r * fs : (r + 1) * fs]
    return full


def unshard_param(name: str, shards: List[torch.Tensor], a: ModelArgs) -> torch.Tensor:
    """Inverse of ``shard_param`` (used for weight sync to the generation engine and for HF export)."""
    leaf = name.split(".")[-1]
    tp = len(shards)
    if leaf in ("wqkv", "bqkv"):
        qs, ks = a.q_dim // tp, a.kv_dim // tp
        return torch.cat([s[:qs] for s in shards] + [s[qs : qs + ks] for s in shards] + [s[qs + ks :] for s in shards], 0)
    if leaf in ("wo", "wd"):
        return torch.cat(shards, 1)
    if leaf == "wgu":
        fs = a.intermediate_size // tp
        return torch.cat([s[:fs] for s in shards] + [s[fs:] for s in shards], 0)
    if leaf == "lm_head" and shards[0].shape[0] * tp == a.vocab_size and tp > 1:
        return torch.cat(shards, 0)  # vocabulary-parallel head
    return shards[0]


def pad_packed_for_tp(input_ids: torch.Tensor, positions: torch.Tensor, cu_seqlens: torch.Tensor, tp: int,
                      pad_id: int = 0) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, int]:
    """Pad the packed batch to a multiple of ``tp * 128`` tokens with one extra dummy sequence. Returns the padded
    tensors and the number of real tokens."""
    T = input_ids.numel()
    mult = tp * 128
    Tp = (T + mult - 1) // mult * mult
    if Tp == T:
        return input_ids, positions, cu_seqlens, T
    n = Tp - T
    ids = torch.cat([input_ids, torch.full((n,), pad_id, dtype=input_ids.dtype, device=input_ids.device)])
    pos = torch.cat([positions, torch.arange(n, dtype=positions.dtype, device=positions.device)])
    cu = torch.cat([cu_seqlens, torch.tensor([Tp], dtype=cu_seqlens.dtype, device=cu_seqlens.device)])
    return ids, pos, cu, T


class _GatherRowsFn(torch.autograd.Function):
    """All-gather of per-rank row shards of a small tensor (log-probs); backward keeps the local slice."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        W = dist.get_world_size(group) if dist.is_initialized() else 1
        if W == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(W)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, 0)

    @staticmethod
    def backward(ctx, g):
        W = dist.get_world_size(ctx.group) if dist.is_initialized() else 1
        if W == 1:
            return g, None
        r = dist.get_rank(ctx.group)
        n = g.shape[0] // W
        return g[r * n : (r + 1) * n].contiguous(), None


class _AllGatherRowsSumBwdFn(torch.autograd.Function):
    """All-gather of row shards whose backward *sums* the ranks' gradients and keeps the local rows (the gathered
    tensor feeds a computation that every rank continues with a different slice of the weights)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return tpm.ref_all_gather_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        return tpm.ref_reduce_scatter_rows(g.contiguous(), ctx.group), None


class _AllReduceIdentityBwdFn(torch.autograd.Function):
    """Sum (or max) over the group in forward; the gradient passes through unchanged: every rank evaluates the same
    replicated loss, so the upstream gradient is already the full one on each rank."""

    @staticmethod
    def forward(ctx, x, group, op):
        y = x.clone()
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(y, op=op, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None, None


class PeerPartials:
    """Exchange of the fused LM-head kernel's per-(row, split) softmax records between the ranks of a vocabulary-
    parallel head: each rank's records live in symmetric memory, a device barrier publishes them, and the combine
    kernel reads every peer's records through its pointer (16 bytes per token and split -- the whole cross-rank
    traffic of the log-sum-exp reduction; reference: three all-reduces, model_utils.py:46-61,95-99)."""

    CHANNEL = 2

    def __init__(self, tp: tpm.TPGroup):
        self.tp, self.sym = tp, None

    def alloc(self, T: int, splits: int) -> torch.Tensor:
        need = T * splits * 4
        if self.sym is None or self.sym.local.numel() < need:
            self.sym = self.tp.peer.alloc(max(need, 1 << 18), torch.float32)
        return self.sym.local[:need].view(T, splits, 4)

    def __call__(self, partials, splits):
        self.tp.peer.barrier(self.CHANNEL)  # every rank's records are complete
        return list(self.sym.ptrs)

    def release(self) -> None:
        self.tp.peer.barrier(self.CHANNEL)  # every rank has read them: the buffer may be overwritten


class TPCausalLM(CausalLM):
    """Local shard of a tensor-parallel model; ``full_args`` describes the unsharded architecture."""

    def __init__(self, full_args: ModelArgs, tp: tpm.TPGroup, device="cpu", dtype=torch.bfloat16, value_head: bool = False,
                 flat_buffer: Optional[torch.Tensor] = None, seed: Optional[int] = 0, vocab_parallel_head: bool = False):
        self.full_args = full_args
        if full_args.attention_sinks:
            raise NotImplementedError("attention sinks are not sharded: use data parallelism for such models")
        self.tp = tp
        # the LM head is sharded over the vocabulary only when asked for and possible (untied, divisible, no value head)
        self.vocab_parallel_head = bool(vocab_parallel_head and not value_head and tp.size > 1
                                        and not full_args.tie_word_embeddings and full_args.vocab_size % tp.size == 0)
        self.replicated_leaves = tuple(x for x in REPLICATED_LEAVES if not (x == "lm_head" and self.vocab_parallel_head))
        super().__init__(local_args(full_args, tp.size, self.vocab_parallel_head), device=device, dtype=dtype,
                         value_head=value_head, flat_buffer=flat_buffer, seed=None)
        self._partials = None
        if seed is not None:
            self.load_from_full(CausalLM(full_args, device="cpu", dtype=torch.float32, value_head=value_head, seed=seed))

    @torch.no_grad()
    def load_from_full(self, full: CausalLM) -> None:
        for name, prm in self.named_flat_views():
            prm.copy_(shard_param(name, full.p(name).detach(), self.full_args, self.tp.size, self.tp.rank,
                                  self.vocab_parallel_head).to(prm.dtype))

    @torch.no_grad()
    def init_random_on_device(self, seed: int = 0) -> None:
        """Random initialisation of large models without a host copy: every full parameter is drawn on the device from
        a generator seeded by (seed, parameter index) -- so all ranks draw the same full tensor -- and this rank keeps
        its slice.  The values differ from ``CausalLM.reset_parameters`` (a host generator); use ``load_from_full``
        when the two must match."""
        from .decoder import _param_specs

        dev = self.flat_params.device
        shapes = dict(_param_specs(self.full_args, value_head=self.has_value_head))
        for k, (name, prm) in enumerate(self.named_flat_views()):
            leaf = name.split(".")[-1]
            if leaf in ("ln1", "ln2", "final_norm", "q_norm", "k_norm"):
                prm.fill_(1.0)
            elif leaf == "bqkv":
                prm.zero_()
            else:
                g = torch.Generator(device=dev).manual_seed(seed * 1000003 + k)
                full = torch.empty(shapes[name], device=dev, dtype=prm.dtype).normal_(0.0, self.full_args.init_std, generator=g)
                prm.copy_(shard_param(name, full, self.full_args, self.tp.size, self.tp.rank, self.vocab_parallel_head))
                del full

    @torch.no_grad()
    def iter_full_state(self):
        """``(name, unsharded parameter)`` one at a time (all-gather of the shards): the caller can consume each tensor
        before the next is gathered, so the full model never exists twice."""
        for name, prm in self.named_flat_views():
            leaf = name.split(".")[-1]
            if leaf in self.replicated_leaves or self.tp.size == 1:
                yield name, prm.detach()
                continue
            parts = [torch.empty_like(prm) for _ in range(self.tp.size)]
            dist.all_gather(parts, prm.detach().contiguous(), group=self.tp.group)
            yield name, unshard_param(name, parts, self.full_args)

    @torch.no_grad()
    def gather_full_state(self) -> Dict[str, torch.Tensor]:
        """Unsharded parameters on every rank, keyed like the unsharded model."""
        return dict(self.iter_full_state())

    def reduce_replicated_grads(self) -> None:
        """Sum over the TP group of the gradients of replicated parameters (each rank saw different tokens)."""
        if self.tp.size == 1:
            return
        for name, prm in self.named_flat_views():
            if name.split(".")[-1] in self.replicated_leaves:
                g = getattr(prm, "main_grad", None)
                if g is None:
                    g = prm.grad
                if g is not None:
                    dist.all_reduce(g, group=self.tp.group)

    # ------------------------------------------------------------------ forward
    def _layer(self, i: int, x, delta, pos, cu, max_seqlen, kv_sink=None, attn_fn=None):
        a, tp = self.args, self.tp
        pre = f"layers.{i}."
        x, h = ew.add_rmsnorm(x, delta, self.p(pre + "ln1"), a.rms_norm_eps)  # [T/tp, H]
        qkv = tpm.column_parallel_linear(h, self.p(pre + "wqkv"), self._p.get(pre + "bqkv"), tp)  # [T, local heads]
        if a.qk_norm:
            qkv = self._qk_norm(qkv, i)
        qkv = ew.rope(qkv, pos, self.rope_table(qkv.device), a.num_heads + a.num_kv_heads, a.head_dim)
        att = attn_ops.attn_varlen(qkv, cu, a.num_heads, a.num_kv_heads, a.head_dim, max_seqlen=max_seqlen)
        o = tpm.row_parallel_linear(att, self.p(pre + "wo"), tp)  # [T/tp, H]
        x, h = ew.add_rmsnorm(x, o, self.p(pre + "ln2"), a.rms_norm_eps)
        gu = tpm.column_parallel_linear(h, self.p(pre + "wgu"), None, tp)  # [T, 2F/tp]
        d = tpm.row_parallel_linear(ew.swiglu(gu), self.p(pre + "wd"), tp)
        return x, d

    def forward(self, input_ids, positions, cu_seqlens, max_seqlen: int = 0, kv_sink=None) -> torch.Tensor:
        """Inputs are the full packed batch (identical on every rank of the TP group, padded with
        ``pad_packed_for_tp``); returns this rank's rows ``[T/tp, H]`` of the final hidden states."""
        tp = self.tp
        T = input_ids.numel()
        if T % (tp.size * 128) != 0 and tp.fused:
            raise ValueError(f"packed length {T} must be a multiple of tp*128 = {tp.size * 128}")
        R = T // tp.size
        x = _EmbeddingFn.apply(input_ids[tp.rank * R : (tp.rank + 1) * R], self.p("embed"))
        delta = None
        for i in range(self.args.num_layers):
            x, delta = self._layer(i, x, delta, positions, cu_seqlens, max_seqlen)
        _, h = ew.add_rmsnorm(x, delta, self.p("final_norm"), self.args.rms_norm_eps)
        return h

    def token_logprobs_full(self, hidden_shard: torch.Tensor, targets_full: torch.Tensor, temperature: float = 1.0,
                            with_entropy: bool = False):
        """Log-probs of all ``T`` targets on every rank: each rank scores its own rows, then the rows are gathered."""
        tp = self.tp
        R = hidden_shard.shape[0]
        if getattr(self, "vocab_parallel_head", False):
            return self._token_logprobs_vocab_parallel(hidden_shard, targets_full, temperature, with_entropy)
        lp, ent = self.token_logprobs(hidden_shard, targets_full[tp.rank * R : (tp.rank + 1) * R], temperature, with_entropy)
        lp = _GatherRowsFn.apply(lp, tp.group)
        if ent is not None:
            ent = _GatherRowsFn.apply(ent, tp.group)
        return lp, ent

    def _token_logprobs_vocab_parallel(self, hidden_shard, targets_full, temperature: float, with_entropy: bool):
        """Vocabulary-parallel fused LM head (reference: distributed/megatron/model_utils.py:275-428 and the TP
        epilogues of fused_linear_logprob_triton.py:478-605): every rank scores all tokens against its slice of the
        vocabulary without materialising logits; the per-split softmax records are merged across ranks by the combine
        kernel through peer pointers, so every rank obtains the full log-probabilities (and entropies)."""
        from ..ops import lm_head as lm_head_ops

        tp = self.tp
        W = self.p("lm_head")
        vs = W.shape[0]
        h_full = _AllGatherRowsSumBwdFn.apply(hidden_shard, tp.group)
        if tp.fused and h_full.is_cuda:
            if self._partials is None:
                self._partials = PeerPartials(tp)
            return lm_head_ops.lm_head_logprobs(h_full, W, targets_full, 1.0 / temperature, with_entropy,
                                                vocab_offset=tp.rank * vs, peer_exchange=self._partials)
        # host / gloo reference: the same reduction written with three all-reduces
        from ..ops import gemm

        z = gemm.linear(h_full, W).float() / temperature  # weight gradient goes to the fp32 main_grad buffer
        m = _AllReduceIdentityBwdFn.apply(z.max(-1).values.detach(), tp.group, dist.ReduceOp.MAX)
        e = torch.exp(z - m[:, None])
        s = _AllReduceIdentityBwdFn.apply(e.sum(-1), tp.group, dist.ReduceOp.SUM)
        lse = m + torch.log(s)
        t = targets_full.long() - tp.rank * vs
        own = (t >= 0) & (t < vs)
        zt = torch.where(own, z.gather(-1, t.clamp(0, vs - 1)[:, None]).squeeze(-1), torch.zeros_like(lse))
        zt = _AllReduceIdentityBwdFn.apply(zt, tp.group, dist.ReduceOp.SUM)
        lp = zt - lse
        pz = _AllReduceIdentityBwdFn.apply((e * z).sum(-1), tp.group, dist.ReduceOp.SUM) / s
        ent = lse - pz
        return lp, (ent if with_entropy else ent.detach())

    def values_full(self, hidden_shard: torch.Tensor) -> torch.Tensor:
        """Value-head outputs of all ``T`` tokens on every rank (each rank scores its rows, then the rows are gathered)."""
        return _GatherRowsFn.apply(self.values(hidden_shard), self.tp.group)


class UlyssesCausalLM(CausalLM):
    """Replicated weights, sequence-sharded activations, head-sharded attention (Ulysses sequence parallelism).

    Every rank of the ``sp`` group passes the same packed batch (padded with ``pad_packed_for_tp``); the residual
    stream, norms, MLP and LM head run on this rank's ``1/sp`` of the tokens with the full weights, attention runs on
    all tokens with ``1/sp`` of the heads.  Gradients of the (replicated) weights are partial sums over tokens, so the
    ordinary data-parallel gradient reduction over all ranks completes them.  Reference: HFModelWrapper.forward with
    ``sequence_parallel_size > 1`` (skyrl/backends/skyrl_train/workers/model_wrapper.py:296-398).
    """

    def __init__(self, args: ModelArgs, sp: tpm.TPGroup, **kw):
        if args.attention_sinks:
            raise NotImplementedError("attention sinks are not sharded: use data parallelism for such models")
        if args.num_heads % sp.size or args.num_kv_heads % sp.size:
            raise ValueError(f"sequence_parallel_size={sp.size} must divide num_heads={args.num_heads} and "
                             f"num_kv_heads={args.num_kv_heads}")
        if args.qk_norm or args.num_experts:
            raise ValueError("Ulysses sequence parallelism supports dense models without per-head q/k norms")
        self.tp = sp
        super().__init__(args, **kw)

    def _layer(self, i: int, x, delta, pos, cu, max_seqlen, kv_sink=None, attn_fn=None):
        from ..parallel import ulysses

        a, sp = self.args, self.tp
        pre = f"layers.{i}."
        x, h = ew.add_rmsnorm(x, delta, self.p(pre + "ln1"), a.rms_norm_eps)
        qkv = ulysses.qkv_proj(h, self.p(pre + "wqkv"), self._p.get(pre + "bqkv"), [a.q_dim, a.kv_dim, a.kv_dim], sp)
        nq, nkv = a.num_heads // sp.size, a.num_kv_heads // sp.size
        qkv = ew.rope(qkv, pos, self.rope_table(qkv.device), nq + nkv, a.head_dim)
        att = attn_ops.attn_varlen(qkv, cu, nq, nkv, a.head_dim, max_seqlen=max_seqlen)
        o = ulysses.o_proj(att, self.p(pre + "wo"), sp)
        x, h = ew.add_rmsnorm(x, o, self.p(pre + "ln2"), a.rms_norm_eps)
        from ..ops import gemm

        gu = gemm.linear(h, self.p(pre + "wgu"))
        d = gemm.linear(ew.swiglu(gu), self.p(pre + "wd"))
        return x, d

    def forward(self, input_ids, positions, cu_seqlens, max_seqlen: int = 0, kv_sink=None) -> torch.Tensor:
        sp = self.tp
        T = input_ids.numel()
        R = T // sp.size
        x = _EmbeddingFn.apply(input_ids[sp.rank * R : (sp.rank + 1) * R], self.p("embed"))
        delta = None
        for i in range(self.args.num_layers):
            x, delta = self._layer(i, x, delta, positions, cu_seqlens, max_seqlen)
        _, h = ew.add_rmsnorm(x, delta, self.p("final_norm"), self.args.rms_norm_eps)
        return h

    token_logprobs_full = TPCausalLM.token_logprobs_full
    values_full = TPCausalLM.values_full

    def reduce_replicated_grads(self) -> None:  # the data-parallel reduction over all ranks already sums them
        return


class ContextParallelCausalLM(UlyssesCausalLM):
    """Replicated weights, sequence-sharded activations, and attention that keeps all heads: every rank of the ``cp``
    group owns a contiguous slice of the packed token axis and all-gathers the keys and values of the tokens before it
    (context parallelism by key/value all-gather).  Unlike Ulysses, whose degree is bounded by the number of key/value
    heads, the degree here is free, at the price of gathering K and V (2 x kv_dim per token and layer; small under
    grouped-query attention).

    The attention kernel takes one packed q|k|v tensor, so a rank builds the rows from the start of the first
    sequence that reaches into its slice up to the end of its slice: K and V come from the gathered tensor, Q is zero
    for the rows it does not own, and only its own rows of the result are kept; the kernels are told where the first
    query row of each sequence is (``q_begin``) and skip the query blocks before it, forward and backward.  The
    backward pass returns the K / V gradients to their owners
    through the reduce-scatter of the gather.  Reference: Megatron ``context_parallel_size``
    (skyrl/backends/skyrl_train/distributed/megatron/megatron_utils.py:421-425,510-530) with ring attention from
    TransformerEngine; selected here with ``trainer.sequence_parallel_backend=context`` (or the Megatron strategy's
    ``context_parallel_size``).
    """

    def __init__(self, args: ModelArgs, sp: tpm.TPGroup, **kw):
        if args.attention_sinks or args.num_experts:
            raise NotImplementedError("context parallelism supports dense models without attention sinks")
        self.tp = sp
        CausalLM.__init__(self, args, **kw)

    def _layer(self, i: int, x, delta, pos, cu, max_seqlen, kv_sink=None, attn_fn=None):
        from ..ops import gemm

        a, cp = self.args, self.tp
        pre = f"layers.{i}."
        row0, row1, first, cu_loc, max_loc, q_begin = self._cp_plan
        x, h = ew.add_rmsnorm(x, delta, self.p(pre + "ln1"), a.rms_norm_eps)
        qkv = gemm.linear(h, self.p(pre + "wqkv"), self._p.get(pre + "bqkv"))
        if a.qk_norm:
            qkv = self._qk_norm(qkv, i)
        qkv = ew.rope(qkv, pos[row0:row1], self.rope_table(qkv.device), a.num_heads + a.num_kv_heads, a.head_dim)
        kv_all = _AllGatherRowsSumBwdFn.apply(qkv[:, a.q_dim:].contiguous(), cp.group)  # [T, 2 * kv_dim]
        lead = row0 - first
        q_rows = qkv[:, : a.q_dim]
        if lead > 0:
            q_rows = torch.cat([q_rows.new_zeros((lead, a.q_dim)), q_rows], 0)
        full = torch.cat([q_rows, kv_all[first:row1]], 1)
        att = attn_ops.attn_varlen(full, cu_loc, a.num_heads, a.num_kv_heads, a.head_dim, max_seqlen=max_loc,
                                   q_begin=q_begin)
        o = gemm.linear(att[lead:].contiguous(), self.p(pre + "wo"))
        x, h = ew.add_rmsnorm(x, o, self.p(pre + "ln2"), a.rms_norm_eps)
        d = gemm.linear(ew.swiglu(gemm.linear(h, self.p(pre + "wgu"))), self.p(pre + "wd"))
        return x, d

    def forward(self, input_ids, positions, cu_seqlens, max_seqlen: int = 0, kv_sink=None) -> torch.Tensor:
        cp = self.tp
        T = input_ids.numel()
        R = T // cp.size
        row0, row1 = cp.rank * R, (cp.rank + 1) * R
        # rows [first, row1): from the start of the first sequence that reaches into this rank's slice
        cu = [int(v) for v in cu_seqlens.tolist()]
        first = max(c for c in cu if c <= row0)
        bounds = [first] + [c for c in cu if first < c < row1] + [row1]
        cu_loc = torch.tensor([b - first for b in bounds], dtype=cu_seqlens.dtype, device=cu_seqlens.device)
        max_loc = max(b - a_ for a_, b in zip(bounds[:-1], bounds[1:]))
        # only the first local sequence starts with foreign rows (keys / values of earlier ranks, no queries)
        q_begin = None
        if row0 > first:
            q_begin = torch.zeros(len(bounds) - 1, dtype=torch.int32, device=cu_seqlens.device)
            q_begin[0] = row0 - first
        self._cp_plan = (row0, row1, first, cu_loc, max_loc, q_begin)
        x = _EmbeddingFn.apply(input_ids[row0:row1], self.p("embed"))
        delta = None
        for i in range(self.args.num_layers):
            x, delta = self._layer(i, x, delta, positions, cu_seqlens, max_seqlen)
        _, h = ew.add_rmsnorm(x, delta, self.p("final_norm"), self.args.rms_norm_eps)
        return h


EXPERT_LEAVES = ("experts_wgu", "experts_wd")


class EPCausalLM(CausalLM):
    """MoE model whose experts are sharded over the ``ep`` group; everything else is replicated and every rank works
    on its own tokens (data parallel).  Expert gradients are complete on the rank that owns the expert; gradients of
    the replicated parameters are partial over tokens and are summed by ``reduce_replicated_grads``."""

    def __init__(self, full_args: ModelArgs, ep: tpm.TPGroup, device="cpu", dtype=torch.bfloat16, seed: Optional[int] = 0,
                 flat_buffer: Optional[torch.Tensor] = None):
        if not full_args.num_experts or full_args.num_experts % ep.size:
            raise ValueError(f"num_experts={full_args.num_experts} must be a positive multiple of ep={ep.size}")
        self.full_args = full_args
        self.tp = ep
        super().__init__(dataclasses.replace(full_args, ep_size=ep.size), device=device, dtype=dtype, flat_buffer=flat_buffer,
                         seed=None)
        self.ep = ep
        if seed is not None:
            self.load_from_full(CausalLM(full_args, device="cpu", dtype=torch.float32, seed=seed))

    def _shard(self, name: str, full: torch.Tensor) -> torch.Tensor:
        if name.split(".")[-1] in EXPERT_LEAVES:
            el = self.full_args.num_experts // self.ep.size
            return full[self.ep.rank * el : (self.ep.rank + 1) * el]
        return full

    @torch.no_grad()
    def load_from_full(self, full: CausalLM) -> None:
        for name, prm in self.named_flat_views():
            prm.copy_(self._shard(name, full.p(name).detach()).to(prm.dtype))

    @torch.no_grad()
    def init_random_on_device(self, seed: int = 0) -> None:
        """Random initialisation without a host copy of the full model (tens of billions of parameters): replicated
        parameters are drawn from a generator seeded by (seed, parameter index), identical on every rank; each rank
        draws only its own experts, from a generator that also depends on the expert's global index."""
        dev = self.flat_params.device
        std = self.full_args.init_std
        el = self.full_args.num_experts // self.ep.size
        for k, (name, prm) in enumerate(self.named_flat_views()):
            leaf = name.split(".")[-1]
            if leaf in ("ln1", "ln2", "final_norm", "q_norm", "k_norm"):
                prm.fill_(1.0)
            elif leaf == "bqkv":
                prm.zero_()
            elif leaf in EXPERT_LEAVES:
                for e in range(el):
                    g = torch.Generator(device=dev).manual_seed((seed * 1000003 + k) * 4099 + self.ep.rank * el + e)
                    prm[e].normal_(0.0, std, generator=g)
            else:
                g = torch.Generator(device=dev).manual_seed(seed * 1000003 + k)
                prm.normal_(0.0, std, generator=g)

    @torch.no_grad()
    def iter_full_state(self):
        for name, prm in self.named_flat_views():
            if name.split(".")[-1] in EXPERT_LEAVES and self.ep.size > 1:
                parts = [torch.empty_like(prm) for _ in range(self.ep.size)]
                dist.all_gather(parts, prm.detach().contiguous(), group=self.ep.group)
                yield name, torch.cat(parts, 0)
            else:
                yield name, prm.detach()

    @torch.no_grad()
    def gather_full_state(self) -> Dict[str, torch.Tensor]:
        return dict(self.iter_full_state())

    def replicated_ranges(self) -> List[Tuple[int, int]]:
        return [(o, o + n) for name, (o, n) in self.offsets.items() if name.split(".")[-1] not in EXPERT_LEAVES]

    def reduce_replicated_grads(self) -> None:
        if self.ep.size == 1:
            return
        for name, prm in self.named_flat_views():
            if name.split(".")[-1] not in EXPERT_LEAVES:
                g = getattr(prm, "main_grad", None)
                if g is None:
                    g = prm.grad
                if g is not None:
                    dist.all_reduce(g, group=self.ep.group)
