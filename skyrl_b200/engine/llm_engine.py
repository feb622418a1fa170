"""In-process generation engine: paged KV cache, continuous batching, device-resident decode state.

What the reference gets from vLLM (skyrl/backends/skyrl_train/inference_servers/vllm_server_actor.py,
the engine behind ``/inference/v1/generate``) is rebuilt here around three ideas:

* **Admission on the host, stepping on the device.**  The C++ scheduler (``csrc/runtime``) admits
  requests, owns the block pool and the prefix cache.  Once a request is admitted its whole decode
  state (current token, position, KV slot, context length, block table, output row) lives in device
  arrays indexed by an engine *slot*; a tiny kernel advances all slots after every sampled token, so a
  decode step is a fixed launch sequence with no host input.
* **CUDA graphs per batch bucket.**  That fixed sequence is captured once per bucket size and
  replayed; the host only synchronises every ``sync_interval`` steps to harvest finished slots.
* **Shared kernels with training.**  Prefill runs the same packed-varlen model forward as the
  trainer (tcgen05 attention, fused projections) with a hook that scatters K/V into the cache, so
  rollout and training log-probabilities come from the same arithmetic.

The engine also runs on CPU tensors (PyTorch reference ops, no graphs) for the plumbing tests.
"""

from __future__ import annotations

import ctypes
import os
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from ..models.decoder import CausalLM
from ..ops import _lib
from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops import gemm, sampling


@dataclass
class SamplingParams:
    max_tokens: int = 1024
    min_tokens: int = 1
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    stop: Optional[List[str]] = None
    stop_token_ids: Optional[List[int]] = None
    ignore_eos: bool = False
    logprobs: Optional[int] = 1
    prompt_logprobs: bool = False
    include_stop_str_in_output: bool = True
    skip_special_tokens: bool = True
    seed: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Optional[dict]) -> "SamplingParams":
        d = dict(d or {})
        if "max_generate_length" in d:
            d["max_tokens"] = d.pop("max_generate_length")
        extra = d.pop("additional_kwargs", None) or {}
        d.update(extra)
        known = {f for f in cls.__dataclass_fields__}
        rp = d.pop("repetition_penalty", None)
        if rp is not None and float(rp) != 1.0:
            raise ValueError(f"repetition_penalty={rp} is not supported by this engine (only 1.0: no penalty)")
        d.pop("n", None)
        pl = d.get("prompt_logprobs")
        if pl is not None and not isinstance(pl, bool):
            d["prompt_logprobs"] = True  # engines that count alternatives use 0 for "the prompt token's own log-prob"
        elif pl is None:
            d.pop("prompt_logprobs", None)
        return cls(**{k: v for k, v in d.items() if k in known})

    @property
    def needs_mask(self) -> bool:
        return (self.top_k is not None and self.top_k > 0) or (self.top_p is not None and self.top_p < 1.0) or (
            self.min_p is not None and self.min_p > 0.0)


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: List[int]
    token_ids: List[int]
    logprobs: List[float]
    finish_reason: str  # "stop" | "length" | "abort"
    prompt_logprobs: Optional[List[float]] = None
    num_cached_tokens: int = 0
    weight_version: int = 0
    # mixture-of-experts models with ``EngineConfig.return_routed_experts``: expert ids chosen for every token that went
    # through the model, ``[prompt + generated - 1, layers, top_k]`` int16 (the last generated token is never fed back)
    routed_experts: Optional[torch.Tensor] = None


@dataclass
class _Request:
    rid: str
    sid: int  # numeric id used by the C++ scheduler
    prompt: List[int]
    params: SamplingParams
    salt: int
    slot: int = -1
    done: bool = False
    prompt_logprobs: Optional[List[float]] = None
    cached: int = 0
    # tokens generated before a pause(abort)/preemption; the request is re-admitted with prompt+partial
    partial_tokens: List[int] = field(default_factory=list)
    partial_logprobs: List[float] = field(default_factory=list)
    # routing recorded by the last prefill of this request: [prompt + partial tokens, layers, top_k] on the host
    prefill_experts: Optional[torch.Tensor] = None


@dataclass
class EngineConfig:
    block_size: int = 32
    num_blocks: int = 0  # 0 = derive from gpu_memory_utilization
    gpu_memory_utilization: float = 0.5
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 16384
    max_model_len: int = 4096
    enable_prefix_caching: bool = False
    enforce_eager: bool = False
    sync_interval: int = 16
    seed: int = 0
    graph_batch_sizes: Sequence[int] = (8, 16, 32, 64, 96, 128, 160, 192, 224, 256, 320, 384, 448, 512, 768, 1024)
    reserve_full_length: bool = True
    fused_decode: bool = True  # split-K projections with fused partial-sum consumers on the decode path
    # mixture-of-experts models: return, with every output, the experts each token was routed to (router replay in the
    # trainer).  Decode then runs without CUDA graphs and the prefix cache is bypassed (cached tokens are not routed).
    return_routed_experts: bool = False
    # speculative decoding with a draft head on the trunk's last hidden state (``set_draft_head``): every decode step
    # feeds the pending token and the head's guess for the one after it, and keeps the second row's result when the
    # token sampled from the first row equals the guess.  0 = off; depths above 1 are run as 1.
    num_speculative_tokens: int = 0
    # KV cache in a fixed-address arena (driver virtual-memory management): sleep() frees the memory, the addresses and
    # the CUDA graphs captured against them stay valid
    kv_fixed_address: bool = True
    # o-proj + norm + gate/up/SwiGLU + down-proj + norm as one persistent kernel per layer (up to 256 sequences);
    # None = follow the environment variable SB_DECODE_MLP_BLOCK (default off)
    fused_mlp_block: Optional[bool] = None
    # CUDA only: the host reads each interval's finish flags from a snapshot while the *next* interval of decode steps
    # already runs, instead of draining the stream after every interval (finished sequences are retired one interval
    # later; their rows are inactive in the meantime)
    overlap_harvest: bool = True


def _rt():
    lib = _lib.runtime()
    if getattr(lib, "_sb_cfg", False):
        return lib
    vp, ci, cl, u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_uint64
    lib.sbrt_sched_create.restype = vp
    lib.sbrt_sched_create.argtypes = [ci] * 6
    lib.sbrt_sched_destroy.argtypes = [vp]
    lib.sbrt_sched_add.argtypes = [vp, cl, vp, ci, ci, u64]
    lib.sbrt_sched_plan.argtypes = [vp, vp, vp, vp, vp, ci]
    lib.sbrt_sched_mark_prefilled.argtypes = [vp, cl]
    lib.sbrt_sched_append.argtypes = [vp, cl, ci]
    lib.sbrt_sched_finish.argtypes = [vp, cl, ci]
    lib.sbrt_sched_seq_len.argtypes = [vp, cl]
    lib.sbrt_sched_seq_cached.argtypes = [vp, cl]
    lib.sbrt_sched_seq_blocks.argtypes = [vp, cl, vp, ci]
    lib.sbrt_sched_seq_tokens.argtypes = [vp, cl, vp, ci]
    lib.sbrt_sched_set_paused.argtypes = [vp, ci]
    for f in ("num_running", "num_waiting", "num_free_blocks", "num_preemptions"):
        getattr(lib, "sbrt_sched_" + f).argtypes = [vp]
    lib.sbrt_sched_prefix_hit_rate.argtypes = [vp]
    lib.sbrt_sched_prefix_hit_rate.restype = ctypes.c_double
    lib.sbrt_sched_reset_prefix_cache.argtypes = [vp]
    lib.sbrt_sched_invalidate_all_kv.argtypes = [vp]
    lib.sbrt_sched_pop_failed.argtypes = [vp, vp, ci]
    lib.sbrt_sched_list.argtypes = [vp, ci, vp, ci]
    lib._sb_cfg = True
    return lib


class LLMEngine:
    """Generation engine bound to one device and one ``CausalLM`` (whose weights it reads in place)."""

    def __init__(self, model: CausalLM, config: Optional[EngineConfig] = None, eos_token_ids: Sequence[int] = (),
                 detokenize: Optional[Callable[[List[int]], str]] = None):
        self.model = model
        self.cfg = config or EngineConfig()
        self.device = model.flat_params.device
        self.is_cuda = self.device.type == "cuda"
        self.detokenize = detokenize
        self.eos_token_ids = list(eos_token_ids)
        a = model.args
        c = self.cfg
        self.max_blocks_per_seq = (c.max_model_len + c.block_size - 1) // c.block_size
        self.num_blocks = c.num_blocks or self._derive_num_blocks()
        self.rt = _rt()
        self.sched = self.rt.sbrt_sched_create(self.num_blocks, c.block_size, c.max_num_seqs, c.max_num_batched_tokens,
                                               int(c.enable_prefix_caching), int(c.reserve_full_length))
        self.kv_dtype = model.flat_params.dtype
        self.k_cache: List[torch.Tensor] = []
        self.v_cache: List[torch.Tensor] = []
        self._alloc_kv()
        S = c.max_num_seqs
        dev = self.device
        i32 = dict(device=dev, dtype=torch.int32)
        self.out_stride = c.max_model_len
        self.cur_tokens = torch.zeros(S, **i32)
        self.positions = torch.zeros(S, **i32)
        self.slots = torch.full((S,), -1, **i32)
        self.ctx_lens = torch.zeros(S, **i32)
        self.block_tables = torch.zeros((S, self.max_blocks_per_seq), **i32)
        self.active = torch.zeros(S, **i32)
        self.finish_reason = torch.zeros(S, **i32)
        self.gen_count = torch.zeros(S, **i32)
        self.max_new = torch.zeros(S, **i32)
        self.min_new = torch.ones(S, **i32)
        self.out_tokens = torch.zeros((S, self.out_stride), **i32)
        self.out_logprobs = torch.zeros((S, self.out_stride), device=dev, dtype=torch.float32)
        # routing capture (mixture-of-experts only): experts of generated token j of a slot, written by the decode step
        # that feeds it back, at [slot, j, layer * top_k + i]
        self._record = bool(c.return_routed_experts and a.num_experts)
        self.out_experts = (torch.zeros((S, self.out_stride, a.num_layers * a.num_experts_per_tok), device=dev,
                                        dtype=torch.int16) if self._record else None)
        # speculative decoding: the draft head's guess for the token after ``cur_tokens`` (valid where draft_valid)
        self.draft_head = None
        self.draft_tokens = torch.zeros(S, **i32)
        self.draft_valid = torch.zeros(S, **i32)
        self._spec_counts = torch.zeros(2, device=dev, dtype=torch.int64)  # rows drafted, drafts accepted
        self.eos_dev = torch.tensor(self.eos_token_ids or [-1], **i32)
        self.step_counter = torch.zeros(1, device=dev, dtype=torch.int64)
        self.temperature = torch.ones(S, device=dev, dtype=torch.float32)
        self.top_k = torch.full((S,), -1, **i32)
        self.top_p = torch.ones(S, device=dev, dtype=torch.float32)
        self.min_p = torch.zeros(S, device=dev, dtype=torch.float32)
        self.sampled = torch.zeros(S, **i32)
        self.sampled_lp = torch.zeros(S, device=dev, dtype=torch.float32)
        self._state_ptrs = None
        self._mlp_ws = None
        if self.is_cuda:
            self._mlp_block_workspace(1)  # allocate the persistent decode kernel's buffers before any graph capture
        self._graphs: Dict[int, "torch.cuda.CUDAGraph"] = {}
        self._graph_launches: Dict[int, int] = {}
        self._graph_pool = None
        self._slot_req: List[Optional[_Request]] = [None] * S
        self._free_slots = list(range(S - 1, -1, -1))
        self._reqs: Dict[int, _Request] = {}
        self._next_sid = 1
        self._mask_slots = 0  # number of occupied slots that need top-k/top-p/min-p masking
        self._cpu_gen = torch.Generator().manual_seed(c.seed)
        self.weight_version = 0
        self.paused = False
        self.asleep = False
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "decode_steps": 0, "prefill_calls": 0,
                      "graph_replays": 0, "preemptions": 0}
        self._finished: List[RequestOutput] = []
        self._snap = None  # pending (event, finish flags, generated counts, slots covered) of the last decode interval
        self._fetch_stream = torch.cuda.Stream(device=self.device) if self.is_cuda else None
        self._snap_bufs = None

    # ------------------------------------------------------------------ memory
    def _kv_block_bytes(self) -> int:
        a = self.model.args
        return 2 * a.num_layers * self.cfg.block_size * a.num_kv_heads * a.head_dim * self.model.flat_params.element_size()

    def _derive_num_blocks(self) -> int:
        c = self.cfg
        if self.is_cuda:
            free, total = torch.cuda.mem_get_info(self.device)
            budget = int(min(free * 0.9, total * c.gpu_memory_utilization))
            n = budget // self._kv_block_bytes()
        else:
            n = 4 * c.max_num_seqs * self.max_blocks_per_seq // 4
        need_all = c.max_num_seqs * self.max_blocks_per_seq
        return int(max(16, min(n, need_all + 64)))

    def _alloc_kv(self) -> None:
        a = self.model.args
        shape = (self.num_blocks, self.cfg.block_size, a.num_kv_heads, a.head_dim)
        self._kv_arena = None
        if self.is_cuda and self.cfg.kv_fixed_address:
            # one fixed-address arena for the whole cache: sleep() returns the physical memory, wake_up() maps new
            # memory at the same address, so the decode graphs captured against the cache survive a sleep
            from .vmm import VmmArena

            per = self.num_blocks * self.cfg.block_size * a.num_kv_heads * a.head_dim * torch.empty((), dtype=self.kv_dtype).element_size()
            per = (per + 255) // 256 * 256
            try:
                self._kv_arena = VmmArena(2 * a.num_layers * per, self.device)
                self._kv_arena.wake(zero=True)
                self.k_cache = [self._kv_arena.take(shape, self.kv_dtype) for _ in range(a.num_layers)]
                self.v_cache = [self._kv_arena.take(shape, self.kv_dtype) for _ in range(a.num_layers)]
                return
            except (RuntimeError, MemoryError):
                self._kv_arena = None  # no virtual-memory-management support here: plain allocations below
        self.k_cache = [torch.zeros(shape, device=self.device, dtype=self.kv_dtype) for _ in range(a.num_layers)]
        self.v_cache = [torch.zeros(shape, device=self.device, dtype=self.kv_dtype) for _ in range(a.num_layers)]

    # ------------------------------------------------------------------ requests
    def add_request(self, request_id: str, prompt_token_ids: Sequence[int], params: SamplingParams,
                    cache_salt: Optional[str] = None) -> None:
        prompt = [int(t) for t in prompt_token_ids]
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        room = self.cfg.max_model_len - len(prompt)
        if room < 1:
            self._finished.append(RequestOutput(request_id, prompt, [], [], "length", weight_version=self.weight_version))
            return
        sid = self._next_sid
        self._next_sid += 1
        salt = (hash(cache_salt) if cache_salt else 0) & ((1 << 64) - 1)
        req = _Request(request_id, sid, prompt, params, salt)
        self._reqs[sid] = req
        self._enqueue(req)

    def _enqueue(self, req: _Request) -> None:
        toks = req.prompt + req.partial_tokens
        max_new = max(1, min(req.params.max_tokens - len(req.partial_tokens), self.cfg.max_model_len - len(toks)))
        arr = np.asarray(toks, dtype=np.int32)
        self.rt.sbrt_sched_add(self.sched, req.sid, arr.ctypes.data, len(toks), int(max_new), req.salt)

    def has_unfinished(self) -> bool:
        return bool(self._reqs)

    def abort_request(self, request_id: str) -> None:
        for sid, r in list(self._reqs.items()):
            if r.rid == request_id:
                self._retire(r, "abort")

    # ------------------------------------------------------------------ forward passes
    def _layer_decode(self, i, x, delta, n, st=None):
        """One decoder layer over one token per row.  ``st`` = (positions, slots, block_tables, ctx_lens) of the rows
        when they are not simply the first ``n`` slots (speculative decoding feeds two rows per slot)."""
        m, a = self.model, self.model.args
        pre = f"layers.{i}."
        pos, slots, bt, ctx = st if st is not None else (self.positions[:n], self.slots[:n], self.block_tables[:n],
                                                         self.ctx_lens[:n])
        x, h = ew.add_rmsnorm(x, delta, m.p(pre + "ln1"), a.rms_norm_eps)
        qkv = gemm.gemm_nt(h, m.p(pre + "wqkv"), m._p.get(pre + "bqkv"))
        if a.qk_norm:
            qkv = m._qk_norm(qkv, i)
        qkv = ew.rope_(qkv, pos, m.rope_table(self.device), a.num_heads + a.num_kv_heads, a.head_dim)
        attn_ops.kv_cache_write(qkv, self.k_cache[i], self.v_cache[i], slots, a.num_heads, a.num_kv_heads,
                                a.head_dim)
        att = attn_ops.attn_decode_paged(qkv, self.k_cache[i], self.v_cache[i], bt, ctx,
                                         a.num_heads, a.num_kv_heads, a.head_dim, max_ctx=self.cfg.max_model_len,
                                         sinks=m._p.get(pre + "sinks"))
        tp = self.tp_size > 1
        o = m.row_parallel_linear(att, m.p(pre + "wo"), "prefill_o", 4) if tp else gemm.gemm_nt(att, m.p(pre + "wo"))
        x, h = ew.add_rmsnorm(x, o, m.p(pre + "ln2"), a.rms_norm_eps)
        if a.num_experts:
            from ..models.moe import moe_ffn

            d = moe_ffn(h, m.p(pre + "router"), m.p(pre + "experts_wgu"), m.p(pre + "experts_wd"),
                        a.num_experts_per_tok, a.norm_topk_prob, layer=i)
        else:
            act = ew.swiglu(gemm.gemm_nt(h, m.p(pre + "wgu")))
            d = m.row_parallel_linear(act, m.p(pre + "wd"), "prefill_d", 5) if tp else gemm.gemm_nt(act, m.p(pre + "wd"))
        return x, d

    def _splitk_linear(self, h, w, bias, n):
        """Skinny projection as fp32 split-K partials; returns (partials[P, n, N], n_written)."""
        N, K = w.shape
        splits, bn = gemm.plan_splitk(n, N, K)
        part = torch.empty((splits, n, N), device=self.device, dtype=torch.float32)
        return part, gemm.gemm_nt_splitk(h, w, bias, part, splits, bn)

    @torch.no_grad()
    def _decode_once_fused(self, n: int, masked: bool) -> None:
        """Decode step for dense models on CUDA: every projection whose tile count cannot fill the SMs runs
        split-K, and the partial sums are consumed by the next kernel (norm / RoPE + cache write)."""
        m, a = self.model, self.model.args
        x = sampling.embed(m.p("embed"), self.cur_tokens[:n])  # residual stream, updated in place
        table = m.rope_table(self.device)
        qkv = torch.empty((n, (a.num_heads + 2 * a.num_kv_heads) * a.head_dim), device=self.device, dtype=x.dtype)
        pending = None
        fused_mlp = a.intermediate_size % 128 == 0 and n >= 32 and os.environ.get("SB_DECODE_FUSED_MLP", "1") != "0"
        block_ws = self._mlp_block_workspace(n)
        h = None
        for i in range(a.num_layers):
            pre = f"layers.{i}."
            if block_ws is not None and i > 0:
                pass  # h is the previous block kernel's output, already normed with this layer's ln1
            elif pending is None:
                _, h = ew.add_rmsnorm(x, None, m.p(pre + "ln1"), a.rms_norm_eps)
            else:
                h = ew.add_rmsnorm_partials_(x, pending[0], pending[1], m.p(pre + "ln1"), a.rms_norm_eps)
            part, np_ = self._splitk_linear(h, m.p(pre + "wqkv"), m._p.get(pre + "bqkv"), n)
            ew.qkv_finalize(part, np_, self.positions[:n], table, qkv, self.k_cache[i], self.v_cache[i], self.slots[:n],
                            a.num_heads, a.num_kv_heads, a.head_dim)
            att = attn_ops.attn_decode_paged(qkv, self.k_cache[i], self.v_cache[i], self.block_tables[:n],
                                             self.ctx_lens[:n], a.num_heads, a.num_kv_heads, a.head_dim,
                                             max_ctx=self.cfg.max_model_len)
            if block_ws is not None:
                nxt = m.p(f"layers.{i + 1}.ln1") if i + 1 < a.num_layers else m.p("final_norm")
                h = ew.decode_mlp_block(att, x, m.p(pre + "wo"), m.p(pre + "ln2"), m.p(pre + "wgu"), m.p(pre + "wd"), nxt,
                                        a.rms_norm_eps, block_ws)
                continue
            part, np_ = self._splitk_linear(att, m.p(pre + "wo"), None, n)
            h = ew.add_rmsnorm_partials_(x, part, np_, m.p(pre + "ln2"), a.rms_norm_eps)
            if fused_mlp:  # SwiGLU in the epilogue of the CTA-pair gate/up GEMM
                act = gemm.gate_up_swiglu(h, m.p(pre + "wgu"), need_gu=False)[1]
            else:
                act = ew.swiglu(gemm.gemm_nt(h, m.p(pre + "wgu"), static_w=True))
            pending = self._splitk_linear(act, m.p(pre + "wd"), None, n)
        if block_ws is None:
            h = ew.add_rmsnorm_partials_(x, pending[0], pending[1], m.p("final_norm"), a.rms_norm_eps)
        logits = gemm.gemm_nt(h, m.lm_head_weight(), static_w=True)
        self._sample(logits, n, masked)
        self._advance(n)

    def _mlp_block_workspace(self, n: int):
        """Workspace of the persistent per-layer kernel when it applies to a batch of ``n`` rows, else None."""
        on = self.cfg.fused_mlp_block
        if on is None:
            on = os.environ.get("SB_DECODE_MLP_BLOCK", "0") == "1"
        a = self.model.args
        if not on or n > ew.DecodeMlpWorkspace.MAX_ROWS:
            return None
        if not ew.DecodeMlpWorkspace.supports(a.hidden_size, a.num_heads * a.head_dim, a.intermediate_size):
            return None
        if self._mlp_ws is None:
            if torch.cuda.is_current_stream_capturing():
                return None  # buffers that outlive a graph are not allocated from its pool
            self._mlp_ws = ew.DecodeMlpWorkspace(self.cfg.max_num_seqs, a.hidden_size, a.num_heads * a.head_dim,
                                                 a.intermediate_size, self.device, self.model.p("embed").dtype)
        return self._mlp_ws if n <= self._mlp_ws.max_rows else None

    @torch.no_grad()
    def _decode_once_fused_tp(self, n: int, masked: bool) -> None:
        """Decode step of a tensor-parallel engine (``engine/tp_model.py``): the QKV and gate/up projections are
        column-parallel (local heads / local FFN columns, no communication); the o-proj and down-proj GEMMs store their
        partial tiles into every rank's slot buffer from the epilogue, and after a device-side barrier the fused
        residual-add + RMSNorm kernel sums the ``tp`` slots -- the all-reduce has no kernel of its own."""
        from .tp_model import DECODE_CHANNELS

        m, a = self.model, self.model.args
        tp = m.tp.size
        x = sampling.embed(m.p("embed"), self.cur_tokens[:n])
        table = m.rope_table(self.device)
        qkv = torch.empty((n, (a.num_heads + 2 * a.num_kv_heads) * a.head_dim), device=self.device, dtype=x.dtype)
        pending = None
        fused_mlp = a.intermediate_size % 128 == 0 and n >= 32 and os.environ.get("SB_DECODE_FUSED_MLP", "1") != "0"
        for i in range(a.num_layers):
            pre = f"layers.{i}."
            if pending is None:
                _, h = ew.add_rmsnorm(x, None, m.p(pre + "ln1"), a.rms_norm_eps)
            else:
                h = ew.add_rmsnorm_partials_(x, pending, pending.shape[0], m.p(pre + "ln1"), a.rms_norm_eps)
            part, np_ = self._splitk_linear(h, m.p(pre + "wqkv"), m._p.get(pre + "bqkv"), n)
            ew.qkv_finalize(part, np_, self.positions[:n], table, qkv, self.k_cache[i], self.v_cache[i], self.slots[:n],
                            a.num_heads, a.num_kv_heads, a.head_dim)
            att = attn_ops.attn_decode_paged(qkv, self.k_cache[i], self.v_cache[i], self.block_tables[:n],
                                             self.ctx_lens[:n], a.num_heads, a.num_kv_heads, a.head_dim,
                                             max_ctx=self.cfg.max_model_len)
            parts_o = m.row_parallel_partials(att, m.p(pre + "wo"), "decode_o", torch.float32, DECODE_CHANNELS[0], True)
            h = ew.add_rmsnorm_partials_(x, parts_o, parts_o.shape[0], m.p(pre + "ln2"), a.rms_norm_eps)
            if fused_mlp:
                act = gemm.gate_up_swiglu(h, m.p(pre + "wgu"), need_gu=False)[1]
            else:
                act = ew.swiglu(gemm.gemm_nt(h, m.p(pre + "wgu"), static_w=True))
            pending = m.row_parallel_partials(act, m.p(pre + "wd"), "decode_d", torch.float32, DECODE_CHANNELS[1], True)
        h = ew.add_rmsnorm_partials_(x, pending, pending.shape[0], m.p("final_norm"), a.rms_norm_eps)
        logits = gemm.gemm_nt(h, m.lm_head_weight(), static_w=True)
        self._sample(logits, n, masked)
        self._advance(n)

    @property
    def tp_size(self) -> int:
        tp = getattr(self.model, "tp", None)
        return tp.size if (tp is not None and hasattr(self.model, "row_parallel_linear")) else 1

    @torch.no_grad()
    def _decode_once(self, n: int, masked: bool) -> None:
        m, a = self.model, self.model.args
        plain = not a.num_experts and not a.qk_norm and not a.attention_sinks
        if self.is_cuda and self.tp_size > 1 and m.tp.fused and plain:
            return self._decode_once_fused_tp(n, masked)
        if self.is_cuda and self.cfg.fused_decode and plain and self.tp_size == 1:
            return self._decode_once_fused(n, masked)
        x = sampling.embed(m.p("embed"), self.cur_tokens[:n])
        delta = None
        for i in range(a.num_layers):
            x, delta = self._layer_decode(i, x, delta, n)
        _, h = ew.add_rmsnorm(x, delta, m.p("final_norm"), a.rms_norm_eps)
        logits = gemm.gemm_nt(h, m.lm_head_weight())
        self._sample(logits, n, masked)
        self._advance(n)

    # ------------------------------------------------------------------ speculative decoding
    def set_draft_head(self, head) -> None:
        """``head(hidden [T, H]) -> [T, H]``: a module whose output, through the model's LM head, predicts the token
        *after* the one the hidden state itself predicts (``algorithms/mtp.py::DraftHead``, trained beside the policy
        with ``trainer.mtp.enabled``).  The engine keeps a reference, not a copy: a trained head drafts with its
        current weights at the next step, so there is no drafter reload after a weight sync (reference: vLLM
        ``speculative_config`` + drafter reload, inference_servers/vllm_worker.py)."""
        if self.tp_size > 1:
            raise NotImplementedError("speculative decoding is not supported by tensor-parallel engines")
        if self._record:
            raise NotImplementedError("speculative decoding cannot be combined with return_routed_experts")
        self.draft_head = head

    @property
    def _spec(self) -> bool:
        return self.draft_head is not None and self.cfg.num_speculative_tokens > 0

    @torch.no_grad()
    def _draft(self, h: torch.Tensor) -> torch.Tensor:
        """Greedy guess of the draft head on hidden states ``h`` -> int32 token ids."""
        w = self.model.lm_head_weight()
        d = self.draft_head(h).to(w.dtype).contiguous()
        return gemm.gemm_nt(d, w).float().argmax(-1).to(torch.int32)

    @torch.no_grad()
    def _decode_once_spec(self, n: int, masked: bool) -> None:
        """One decode step over two rows per slot: row A feeds the pending token, row B the draft head's guess for the
        next one.  The token sampled from row A is always kept; if it equals the guess, row B was computed on the right
        input and the token sampled from it is kept too.  Sampling is from the target model's own distributions in
        both cases, so the output distribution is exactly that of plain decoding (a greedy guess is accepted with the
        probability the target gives it, which is also what speculative sampling's accept rule yields for a
        deterministic draft).  The key/value entry row B wrote for a rejected guess is overwritten by the next step."""
        m, a = self.model, self.model.args
        bs = self.cfg.block_size
        act = self.active[:n].bool()
        posA = self.positions[:n]
        # a guess is only fed where the slot may still emit two tokens (its blocks are reserved up to that length)
        has = act & self.draft_valid[:n].bool() & ((self.gen_count[:n] + 1) < self.max_new[:n])
        posB = torch.where(has, posA + 1, posA)
        blk = self.block_tables[:n].gather(1, (posB // bs).long().unsqueeze(1)).squeeze(1)
        slotB = torch.where(has, blk * bs + posB % bs, torch.full_like(blk, -1))
        tokB = torch.where(has, self.draft_tokens[:n], self.cur_tokens[:n])
        st = (torch.cat([posA, posB]), torch.cat([self.slots[:n], slotB]),
              torch.cat([self.block_tables[:n], self.block_tables[:n]]), torch.cat([self.ctx_lens[:n], posB + 1]))
        x = sampling.embed(m.p("embed"), torch.cat([self.cur_tokens[:n], tokB]))
        delta = None
        for i in range(a.num_layers):
            x, delta = self._layer_decode(i, x, delta, 2 * n, st)
        _, h = ew.add_rmsnorm(x, delta, m.p("final_norm"), a.rms_norm_eps)
        logits = gemm.gemm_nt(h, m.lm_head_weight())
        temp = torch.cat([self.temperature[:n], self.temperature[:n]])
        if masked:
            logits = _mask_logits_rows(logits, temp, torch.cat([self.top_k[:n]] * 2), torch.cat([self.top_p[:n]] * 2),
                                       torch.cat([self.min_p[:n]] * 2))
        tok = torch.empty(2 * n, device=self.device, dtype=torch.int32)
        lp = torch.empty(2 * n, device=self.device)
        if self.is_cuda:
            sampling.sample(logits, temp.contiguous(), self.cfg.seed, self.step_counter, tok, lp)
        else:
            t_, l_ = sampling.sample(logits, temp, self.cfg.seed, generator=self._cpu_gen)
            tok.copy_(t_)
            lp.copy_(l_)
        accepted = has & (tok[:n] == self.draft_tokens[:n])
        # the next guess comes from the last hidden state that was computed on real tokens
        h_last = torch.where(accepted.unsqueeze(1), h[n:], h[:n])
        guess = self._draft(h_last)
        rows = torch.arange(n, device=self.device)
        self.sampled[:n] = tok[:n]
        self.sampled_lp[:n] = lp[:n]
        self._advance_rows(rows)
        second = rows[accepted]
        if second.numel():
            self.sampled[second] = tok[n:][accepted]
            self.sampled_lp[second] = lp[n:][accepted]
            self._advance_rows(second)  # rows that finished on their first token are inactive and stay untouched
        self.draft_tokens[:n] = guess
        self.draft_valid[:n] = self.active[:n]
        self._spec_counts[0] += has.sum()
        self._spec_counts[1] += accepted.sum()

    def _sample(self, logits: torch.Tensor, n: int, masked: bool, rows: Optional[torch.Tensor] = None) -> None:
        """Samples into ``self.sampled[:n]`` / ``self.sampled_lp[:n]`` (rows = slot index of each logits row)."""
        temp = self.temperature[:n] if rows is None else self.temperature[rows]
        if masked:
            tk = self.top_k[:n] if rows is None else self.top_k[rows]
            tp = self.top_p[:n] if rows is None else self.top_p[rows]
            mp = self.min_p[:n] if rows is None else self.min_p[rows]
            logits = _mask_logits_rows(logits, temp, tk, tp, mp)
        out_t = self.sampled[:n] if rows is None else torch.empty(logits.shape[0], device=self.device, dtype=torch.int32)
        out_l = self.sampled_lp[:n] if rows is None else torch.empty(logits.shape[0], device=self.device)
        if self.is_cuda:
            sampling.sample(logits, temp.contiguous(), self.cfg.seed, self.step_counter, out_t, out_l)
        else:
            t, l = sampling.sample(logits, temp, self.cfg.seed, generator=self._cpu_gen)
            out_t.copy_(t)
            out_l.copy_(l)
        if rows is not None:
            self.sampled[rows] = out_t
            self.sampled_lp[rows] = out_l

    def _advance(self, n: int) -> None:
        if self.is_cuda:
            if self._state_ptrs is None:
                ptrs = [self.cur_tokens, self.positions, self.slots, self.ctx_lens, self.block_tables, self.active,
                        self.finish_reason, self.gen_count, self.max_new, self.min_new, self.out_tokens,
                        self.out_logprobs, self.eos_dev, self.step_counter]
                self._state_ptrs = (ctypes.c_void_p * len(ptrs))(*[p.data_ptr() for p in ptrs])
                lib = _lib.kernels()
                lib.sb_decode_advance.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                                  ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
            code = _lib.kernels().sb_decode_advance(self._state_ptrs, self.sampled.data_ptr(), self.sampled_lp.data_ptr(),
                                                    n, self.max_blocks_per_seq, self.cfg.block_size, self.out_stride,
                                                    len(self.eos_token_ids), _lib.stream_ptr())
            _lib.check(code, "sb_decode_advance")
            return
        self._advance_rows(torch.arange(n, device=self.device))

    def _advance_rows(self, rows: torch.Tensor) -> None:
        """PyTorch mirror of ``decode_advance_kernel`` restricted to ``rows`` (CPU path, prefill install)."""
        rows = rows[self.active[rows].bool()]
        if rows.numel() == 0:
            return
        r = rows.long()
        tok, lp = self.sampled[r], self.sampled_lp[r]
        gc = self.gen_count[r].long()
        ok = gc < self.out_stride
        self.out_tokens[r[ok], gc[ok]] = tok[ok]
        self.out_logprobs[r[ok], gc[ok]] = lp[ok]
        gc = gc + 1
        self.gen_count[r] = gc.to(torch.int32)
        is_eos = torch.zeros_like(tok, dtype=torch.bool)
        for e in self.eos_token_ids:
            is_eos |= tok == e
        reason = torch.where(is_eos & (gc >= self.min_new[r]), 1, 0)
        reason = torch.where((reason == 0) & (gc >= self.max_new[r]), 2, reason).to(torch.int32)
        fin = reason != 0
        fr = r[fin]
        self.active[fr] = 0
        self.finish_reason[fr] = reason[fin]
        self.slots[fr] = -1
        self.ctx_lens[fr] = 0
        go = r[~fin]
        if go.numel():
            p = self.positions[go] + 1
            self.positions[go] = p
            self.cur_tokens[go] = tok[~fin]
            bs = self.cfg.block_size
            blk = self.block_tables[go, (p // bs).long()]
            self.slots[go] = blk * bs + p % bs
            self.ctx_lens[go] = p + 1
        if self.is_cuda:
            self.step_counter += 1

    @torch.no_grad()
    def _prefill(self, reqs: List[_Request], starts: List[int]) -> None:
        m, a = self.model, self.model.args
        bs = self.cfg.block_size
        dev = self.device
        ids, pos, slot_list, cu = [], [], [], [0]
        rows = []
        full_slots: List[int] = []  # cache slot of every token (cached prefix + new), per sequence, for the prefix path
        q_first: List[int] = []     # number of cached tokens per sequence = first row that carries a query
        new_rows_in_full: List[int] = []
        cu_full = [0]
        any_cached = False
        for req in reqs:
            toks = req.prompt + req.partial_tokens
            L = len(toks)
            bt = np.zeros(self.max_blocks_per_seq, dtype=np.int32)
            nb = self.rt.sbrt_sched_seq_blocks(self.sched, req.sid, bt.ctypes.data, self.max_blocks_per_seq)
            assert nb >= (L + bs - 1) // bs, "scheduler did not reserve enough blocks"
            req.cached = self.rt.sbrt_sched_seq_cached(self.sched, req.sid)
            # tokens whose key/value blocks are already in the cache are not recomputed (at least one token is)
            c = min(int(req.cached), L - 1) if self.cfg.enable_prefix_caching else 0
            if req.params.prompt_logprobs or self._record:
                c = 0  # prompt log-probs need every position's hidden state; routing capture every position's router
            c = (c // bs) * bs
            any_cached = any_cached or c > 0
            slot = self._free_slots.pop()
            req.slot = slot
            self._slot_req[slot] = req
            rows.append(slot)
            self.block_tables[slot].copy_(_lib.to_device(torch.from_numpy(bt), dev))
            all_slots = (bt[np.arange(L) // bs] * bs + np.arange(L) % bs).tolist()
            ids.extend(toks[c:])
            pos.extend(range(c, L))
            slot_list.extend(all_slots[c:])
            cu.append(cu[-1] + (L - c))
            new_rows_in_full.extend(range(cu_full[-1] + c, cu_full[-1] + L))
            q_first.append(c)
            full_slots.extend(all_slots)
            cu_full.append(cu_full[-1] + L)
        t_ids = _lib.to_device(torch.tensor(ids, dtype=torch.int32), dev)
        t_pos = _lib.to_device(torch.tensor(pos, dtype=torch.int32), dev)
        t_slots = _lib.to_device(torch.tensor(slot_list, dtype=torch.int32), dev)
        t_cu = _lib.to_device(torch.tensor(cu, dtype=torch.int32), dev)

        def sink(layer, qkv):
            attn_ops.kv_cache_write(qkv, self.k_cache[layer], self.v_cache[layer], t_slots, a.num_heads,
                                    a.num_kv_heads, a.head_dim)

        max_len = max(len(r.prompt) + len(r.partial_tokens) for r in reqs)
        attn_fn = None
        if any_cached:
            # Prefix path: the projections and the MLP run on the new tokens only; attention runs over rows that hold
            # the cached prefix's keys/values (gathered from the paged cache) followed by the new tokens' q, k, v.
            t_full_slots = _lib.to_device(torch.tensor(full_slots, dtype=torch.long), dev)
            t_new_rows = _lib.to_device(torch.tensor(new_rows_in_full, dtype=torch.long), dev)
            t_cu_full = _lib.to_device(torch.tensor(cu_full, dtype=torch.int32), dev)
            # the cached rows carry no query: the attention kernel skips the query blocks that lie entirely inside them
            t_q_first = _lib.to_device(torch.tensor(q_first, dtype=torch.int32), dev)
            qd, kvd = a.num_heads * a.head_dim, a.num_kv_heads * a.head_dim
            Tf = len(full_slots)

            def attn_fn(layer, qkv):  # noqa: F811 - runs after sink() has written the new keys/values
                full = torch.zeros((Tf, qd + 2 * kvd), device=dev, dtype=qkv.dtype)
                full[:, qd : qd + kvd] = self.k_cache[layer].view(-1, kvd)[t_full_slots]
                full[:, qd + kvd :] = self.v_cache[layer].view(-1, kvd)[t_full_slots]
                full[t_new_rows, :qd] = qkv[:, :qd]
                att = attn_ops.attn_varlen(full, t_cu_full, a.num_heads, a.num_kv_heads, a.head_dim, max_seqlen=max_len,
                                           sinks=m._p.get(f"layers.{layer}.sinks"), q_begin=t_q_first)
                return att[t_new_rows].contiguous()

            self.stats["prefix_cached_tokens"] = self.stats.get("prefix_cached_tokens", 0) + (Tf - len(ids))
        if self._record:
            from ..models import router_replay

            with router_replay.record_routing() as store:
                h = m(t_ids, t_pos, t_cu, max_len, kv_sink=sink, attn_fn=attn_fn)
            table = router_replay.stack_recorded(store).to(torch.int16).cpu()  # [tokens, layers, top_k]
            for k, r in enumerate(reqs):
                r.prefill_experts = table[cu[k] : cu[k + 1]].clone()
        else:
            h = m(t_ids, t_pos, t_cu, max_len, kv_sink=sink, attn_fn=attn_fn)
        last = h[(t_cu[1:] - 1).long()]
        if any(r.params.prompt_logprobs for r in reqs):
            tgt = torch.roll(t_ids, -1)
            plp, _ = m.token_logprobs(h, tgt)
            plp = plp.float().cpu()
            for k, r in enumerate(reqs):
                if r.params.prompt_logprobs:
                    r.prompt_logprobs = [None] + plp[cu[k] : cu[k + 1] - 1].tolist()
        logits = gemm.gemm_nt(last.contiguous(), m.lm_head_weight())
        rows_t = torch.tensor(rows, device=dev, dtype=torch.long)
        # per-slot sampling parameters and counters
        host = lambda f, dt: torch.tensor([f(r) for r in reqs], device=dev, dtype=dt)  # noqa: E731
        self.temperature[rows_t] = host(lambda r: r.params.temperature, torch.float32)
        self.top_k[rows_t] = host(lambda r: r.params.top_k if r.params.top_k else -1, torch.int32)
        self.top_p[rows_t] = host(lambda r: r.params.top_p, torch.float32)
        self.min_p[rows_t] = host(lambda r: r.params.min_p, torch.float32)
        self.max_new[rows_t] = host(lambda r: max(1, min(r.params.max_tokens - len(r.partial_tokens),
                                                         self.cfg.max_model_len - len(r.prompt) - len(r.partial_tokens))),
                                    torch.int32)
        self.min_new[rows_t] = host(lambda r: (1 << 30) if r.params.ignore_eos else max(0, r.params.min_tokens - len(r.partial_tokens)),
                                    torch.int32)
        self.gen_count[rows_t] = 0
        self.finish_reason[rows_t] = 0
        self.active[rows_t] = 1
        self.positions[rows_t] = host(lambda r: len(r.prompt) + len(r.partial_tokens) - 1, torch.int32)
        masked = any(r.params.needs_mask for r in reqs)
        self._mask_slots += sum(1 for r in reqs if r.params.needs_mask)
        self._sample(logits, len(reqs), masked, rows=rows_t)
        self._advance_rows(rows_t)
        if self._spec:
            self.draft_tokens[rows_t] = self._draft(last.contiguous())
            self.draft_valid[rows_t] = self.active[rows_t]
        for r in reqs:
            self.rt.sbrt_sched_mark_prefilled(self.sched, r.sid)
        self.stats["prefill_tokens"] += len(ids)
        self.stats["prefill_calls"] += 1

    # ------------------------------------------------------------------ stepping
    def _bucket(self, n: int) -> int:
        for b in self.cfg.graph_batch_sizes:
            if b >= n and b <= self.cfg.max_num_seqs:
                return b
        return self.cfg.max_num_seqs

    def _hi(self) -> int:
        hi = 0
        for s, r in enumerate(self._slot_req):
            if r is not None:
                hi = s + 1
        return hi

    def _run_decode(self, steps: int) -> None:
        hi = self._hi()
        if hi == 0:
            return
        masked = self._mask_slots > 0
        n = self._bucket(hi)
        # mixture-of-experts layers build their routing plan on the device (no host reads), so they replay from a graph
        # like dense layers -- except while the routing is being recorded or replayed (those tensors live on the host side)
        from ..models import router_replay

        use_graph = (self.is_cuda and not self.cfg.enforce_eager and not masked and not router_replay.active()
                     and not self._record and not self._spec)
        if use_graph:
            g = self._graphs.get(n)
            if g is None:
                g = self._capture(n)
            for _ in range(steps):
                g.replay()
            _lib.LAUNCH_COUNT += steps * self._graph_launches.get(n, 0)
            self.stats["graph_replays"] += steps
        elif self._spec:
            for _ in range(steps):
                self._decode_once_spec(n, masked)
        elif self._record:
            rows = torch.arange(n, device=self.device)
            for _ in range(steps):
                # the token fed by this step is generated token ``gen_count - 1`` of its slot
                at = (self.gen_count[:n].long() - 1).clamp_(0, self.out_stride - 1)
                live = self.active[:n].bool()
                with router_replay.record_routing() as store:
                    self._decode_once(n, masked)
                tab = router_replay.stack_recorded(store).reshape(n, -1).to(torch.int16)
                self.out_experts[rows, at] = torch.where(live[:, None], tab, self.out_experts[rows, at])
        else:
            for _ in range(steps):
                self._decode_once(n, masked)
        self.stats["decode_steps"] += steps

    def _capture(self, n: int):
        # warm up outside capture (lazy kernel attribute setup, tensor-map cache, workspace sizing)
        saved = [t.clone() for t in (self.cur_tokens, self.positions, self.slots, self.ctx_lens, self.active,
                                     self.finish_reason, self.gen_count, self.out_tokens, self.out_logprobs,
                                     self.step_counter)]
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            self._decode_once(n, False)
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        before = _lib.LAUNCH_COUNT
        with torch.cuda.graph(g, pool=self._graph_pool):
            self._decode_once(n, False)
        self._graph_launches[n] = _lib.LAUNCH_COUNT - before
        _lib.LAUNCH_COUNT = before  # capture does not execute; replays are counted instead
        if self._graph_pool is None:
            self._graph_pool = g.pool()
        for dst, src in zip((self.cur_tokens, self.positions, self.slots, self.ctx_lens, self.active,
                             self.finish_reason, self.gen_count, self.out_tokens, self.out_logprobs,
                             self.step_counter), saved):
            dst.copy_(src)
        self._graphs[n] = g
        return g

    def _take_snapshot(self) -> None:
        """Enqueue (behind everything issued so far) a copy of the finish flags and token counts into pinned host
        memory and an event that marks it complete; ``_process_snapshot`` consumes it later without draining the stream."""
        hi = self._hi()
        if hi == 0:
            self._snap = None
            return
        S = self.cfg.max_num_seqs
        if self._snap_bufs is None:
            self._snap_bufs = [(torch.empty(S, dtype=torch.int32, pin_memory=True), torch.empty(S, dtype=torch.int32, pin_memory=True))
                               for _ in range(2)]
            self._snap_flip = 0
        self._snap_flip ^= 1
        fr, gc = self._snap_bufs[self._snap_flip]
        fr[:hi].copy_(self.finish_reason[:hi], non_blocking=True)
        gc[:hi].copy_(self.gen_count[:hi], non_blocking=True)
        _lib.D2H_BYTES += 8 * hi
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._snap = (ev, fr, gc, hi)

    def _process_snapshot(self) -> None:
        """Retire what the pending snapshot shows as finished.  Outputs are fetched on a side stream that waits for the
        snapshot's event only, so decode steps already enqueued behind it keep running meanwhile (finished rows are
        inactive: nothing writes them)."""
        snap, self._snap = self._snap, None
        if snap is None:
            return
        ev, fr_t, gc_t, hi = snap
        ev.synchronize()
        fr, gc = fr_t[:hi].numpy(), gc_t[:hi].numpy()
        self._harvest_from(fr, gc, hi, fetch_after=ev)

    def _harvest(self) -> None:
        hi = self._hi()
        if hi == 0:
            return
        self._harvest_from(_lib.to_host(self.finish_reason[:hi]), _lib.to_host(self.gen_count[:hi]), hi)

    def _drain(self) -> None:
        """Bring the host's view up to date with the device (pending snapshot, then a synchronous harvest)."""
        if self._snap is not None:
            self._process_snapshot()
        self._harvest()

    def _harvest_from(self, fr, gc, hi: int, fetch_after=None) -> None:
        done = [s for s in range(hi) if self._slot_req[s] is not None and int(fr[s]) != 0]
        stop_str = [s for s in range(hi) if self._slot_req[s] is not None and int(fr[s]) == 0
                    and self._slot_req[s].params.stop and self.detokenize is not None]
        fetch = done + stop_str
        if not fetch:
            return
        nmax = max(1, max(int(gc[s]) for s in fetch))
        if fetch_after is not None:
            # only the copies run on the side stream; every write to the slot state below stays on the main stream
            with torch.cuda.stream(self._fetch_stream):
                self._fetch_stream.wait_event(fetch_after)
                idx = torch.tensor(fetch, device=self.device, dtype=torch.long)
                toks = _lib.to_host(self.out_tokens[idx, :nmax])
                lps = _lib.to_host(self.out_logprobs[idx, :nmax])
        else:
            idx = torch.tensor(fetch, device=self.device, dtype=torch.long)
            toks = _lib.to_host(self.out_tokens[idx, :nmax])
            lps = _lib.to_host(self.out_logprobs[idx, :nmax])
        for k, s in enumerate(fetch):
            req = self._slot_req[s]
            n = int(gc[s])
            t, l = toks[k, :n].tolist(), lps[k, :n].tolist()
            if k < len(done):
                self._retire(req, "stop" if int(fr[s]) == 1 else "length", t, l)
            else:
                cut = _find_stop(self.detokenize, t, req.params.stop)
                if cut is not None:
                    self._retire(req, "stop", t[:cut], l[:cut])

    _SLOT_STATE = ("cur_tokens", "positions", "slots", "ctx_lens", "block_tables", "active", "finish_reason", "gen_count",
                   "max_new", "min_new", "out_tokens", "out_logprobs", "temperature", "top_k", "top_p", "min_p", "sampled",
                   "sampled_lp", "out_experts", "draft_tokens", "draft_valid")

    def _compact_slots(self) -> None:
        """Move running sequences from high slots into free low slots when that lets the decode batch drop to a
        smaller bucket: the decode step is launched over slots ``[0, bucket(hi))``, so stragglers parked in high
        slots would otherwise keep every step at the full batch size while most rows are idle."""
        live = [s for s, r in enumerate(self._slot_req) if r is not None]
        if not live:
            return
        target = self._bucket(len(live))
        if target >= self._bucket(live[-1] + 1):
            return
        movers = [s for s in live if s >= len(live)]
        holes = [s for s in range(len(live)) if self._slot_req[s] is None]
        src = torch.tensor(movers, device=self.device, dtype=torch.long)
        dst = torch.tensor(holes[: len(movers)], device=self.device, dtype=torch.long)
        for name in self._SLOT_STATE:
            t = getattr(self, name)
            if t is not None:
                t[dst] = t[src]
        self.active[src] = 0
        self.finish_reason[src] = 0
        self.slots[src] = -1
        self.ctx_lens[src] = 0
        for a, b in zip(movers, holes):
            req = self._slot_req[a]
            self._slot_req[b], self._slot_req[a] = req, None
            req.slot = b
        used = {s for s, r in enumerate(self._slot_req) if r is not None}
        self._free_slots = [s for s in range(self.cfg.max_num_seqs - 1, -1, -1) if s not in used]
        self.stats["slot_compactions"] = self.stats.get("slot_compactions", 0) + 1

    def _retire(self, req: _Request, reason: str, toks: Optional[List[int]] = None,
                lps: Optional[List[float]] = None) -> None:
        routed = None
        if self._record and req.prefill_experts is not None:
            # prefill covered the prompt and the tokens generated before it; each later token but the last was fed by a
            # decode step of this slot
            a = self.model.args
            fed = max(0, len(toks or []) - 1)
            routed = req.prefill_experts
            if fed and req.slot >= 0:
                dec = self.out_experts[req.slot, :fed].cpu().view(fed, a.num_layers, a.num_experts_per_tok)
                routed = torch.cat([routed, dec], 0)
        toks = req.partial_tokens + (toks or [])
        lps = req.partial_logprobs + (lps or [])
        if req.slot >= 0:
            s = req.slot
            self.active[s] = 0
            self.finish_reason[s] = 0
            self.slots[s] = -1
            self.ctx_lens[s] = 0
            self._slot_req[s] = None
            self._free_slots.append(s)
            self._free_slots.sort(reverse=True)
            if req.params.needs_mask:
                self._mask_slots -= 1
            req.slot = -1
        # keep the scheduler's copy of the sequence in sync so that its full blocks can be published
        for t in (toks[len(req.partial_tokens):] if self.cfg.enable_prefix_caching else []):
            self.rt.sbrt_sched_append(self.sched, req.sid, int(t))
        self.rt.sbrt_sched_finish(self.sched, req.sid, int(self.cfg.enable_prefix_caching and reason != "abort"))
        self._reqs.pop(req.sid, None)
        self.stats["decode_tokens"] += len(toks)
        self._finished.append(RequestOutput(req.rid, req.prompt, toks, lps, reason, req.prompt_logprobs, req.cached,
                                            self.weight_version, routed))

    def step(self) -> List[RequestOutput]:
        """One scheduling round: admit + prefill what fits, then ``sync_interval`` decode steps, then harvest."""
        if self.is_cuda:
            # the CUDA current device is per thread; callers may step the engine from worker threads
            torch.cuda.set_device(self.device)
        if self.paused or self.asleep:
            out, self._finished = self._finished, []
            return out
        cap = self.cfg.max_num_seqs
        ids = (ctypes.c_longlong * cap)()
        starts = (ctypes.c_int * cap)()
        counts = (ctypes.c_int * cap)()
        mode = ctypes.c_int(0)
        while self._free_slots and self.rt.sbrt_sched_num_waiting(self.sched) > 0:
            n = self.rt.sbrt_sched_plan(self.sched, ctypes.byref(mode), ids, starts, counts, min(cap, len(self._free_slots)))
            if mode.value != 1 or n == 0:
                break
            self._prefill([self._reqs[ids[i]] for i in range(n)], [starts[i] for i in range(n)])
        failed = (ctypes.c_longlong * 64)()
        nf = self.rt.sbrt_sched_pop_failed(self.sched, failed, 64)
        for i in range(nf):
            req = self._reqs.pop(failed[i], None)
            if req is not None:
                self._finished.append(RequestOutput(req.rid, req.prompt, [], [], "abort", weight_version=self.weight_version))
        if self.is_cuda and self.cfg.overlap_harvest:
            # a snapshot that has already landed costs nothing to read: use it before deciding what to launch
            if self._snap is not None and self._snap[0].query():
                self._process_snapshot()
                self._compact_slots() if any(r is not None for r in self._slot_req) else None
            if any(r is not None for r in self._slot_req):
                self._run_decode(self.cfg.sync_interval)  # enqueue the next interval first ...
                self._process_snapshot()                  # ... then read the previous one while it runs
                if any(r is not None for r in self._slot_req):
                    self._compact_slots()
                self._take_snapshot()
            else:
                self._process_snapshot()
            out, self._finished = self._finished, []
            return out
        self._harvest()  # requests that finished on their very first token
        if any(r is not None for r in self._slot_req):
            self._compact_slots()
            self._run_decode(self.cfg.sync_interval)
            self._harvest()
        out, self._finished = self._finished, []
        return out

    def generate(self, prompts: Sequence[Sequence[int]], params, request_ids: Optional[Sequence[str]] = None,
                 cache_salt: Optional[str] = None) -> List[RequestOutput]:
        """Blocking convenience wrapper: run until every given prompt has finished; results in input order."""
        if isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        rids = list(request_ids) if request_ids is not None else [f"gen-{self._next_sid}-{i}" for i in range(len(prompts))]
        for rid, p, sp in zip(rids, prompts, params):
            self.add_request(rid, p, sp, cache_salt)
        want = set(rids)
        got: Dict[str, RequestOutput] = {}
        while want - set(got):
            if self.paused or self.asleep:
                raise RuntimeError("generate() called on a paused or sleeping engine")
            for o in self.step():
                got[o.request_id] = o
        return [got[r] for r in rids]

    # ------------------------------------------------------------------ control plane
    def pause(self, mode: str = "keep", clear_cache: bool = False) -> List[RequestOutput]:
        """``keep``: freeze in-flight requests with their KV; ``abort``: return partial outputs; ``wait``: drain."""
        out: List[RequestOutput] = []
        if mode == "wait":
            while self.has_unfinished():
                out.extend(self.step())
        elif mode == "abort":
            self._drain()
            hi = self._hi()
            gc = self.gen_count[:hi].cpu() if hi else []
            for s in range(hi):
                req = self._slot_req[s]
                if req is None:
                    continue
                n = int(gc[s])
                self._retire(req, "abort", self.out_tokens[s, :n].cpu().tolist(), self.out_logprobs[s, :n].cpu().tolist())
            for req in list(self._reqs.values()):
                self._retire(req, "abort")
            out, self._finished = self._finished, []
        elif mode != "keep":
            raise ValueError(f"unknown pause mode '{mode}'")
        self.paused = True
        self.rt.sbrt_sched_set_paused(self.sched, 1)
        if clear_cache:
            self.reset_prefix_cache()
        return out

    def resume(self) -> None:
        self.paused = False
        self.rt.sbrt_sched_set_paused(self.sched, 0)

    def reset_prefix_cache(self, reset_running_requests: bool = False) -> None:
        if reset_running_requests:
            self._requeue_running()
            self.rt.sbrt_sched_invalidate_all_kv(self.sched)
        else:
            self.rt.sbrt_sched_reset_prefix_cache(self.sched)

    def _requeue_running(self) -> None:
        """Move every slot's request back to the waiting queue, keeping the tokens generated so far."""
        self._drain()
        hi = self._hi()
        if hi == 0:
            return
        gc = self.gen_count[:hi].cpu()
        for s in range(hi):
            req = self._slot_req[s]
            if req is None:
                continue
            n = int(gc[s])
            if self._record and req.prefill_experts is not None and n > 1:
                a = self.model.args
                dec = self.out_experts[s, : n - 1].cpu().view(n - 1, a.num_layers, a.num_experts_per_tok)
                req.prefill_experts = torch.cat([req.prefill_experts, dec], 0)
            req.partial_tokens = req.partial_tokens + self.out_tokens[s, :n].cpu().tolist()
            req.partial_logprobs = req.partial_logprobs + self.out_logprobs[s, :n].cpu().tolist()
            self.active[s] = 0
            self.slots[s] = -1
            self.ctx_lens[s] = 0
            self._slot_req[s] = None
            self._free_slots.append(s)
            if req.params.needs_mask:
                self._mask_slots -= 1
            req.slot = -1
            self.rt.sbrt_sched_finish(self.sched, req.sid, 0)
            self._enqueue(req)
        self._free_slots.sort(reverse=True)

    def sleep(self, level: int = 1, tags: Optional[Sequence[str]] = None) -> None:
        """Release the KV cache memory (level >= 1). Weights are shared with the trainer and stay put."""
        if self.asleep:
            return
        if tags is None or "kv_cache" in tags:
            self._requeue_running()
            self.rt.sbrt_sched_invalidate_all_kv(self.sched)
            if getattr(self, "_kv_arena", None) is not None:
                self._kv_arena.sleep()  # the tensors keep their addresses; the captured graphs stay
            else:
                self.k_cache, self.v_cache = [], []
                self._graphs.clear()
                self._graph_pool = None
                if self.is_cuda:
                    torch.cuda.empty_cache()
        self.asleep = True

    def wake_up(self, tags: Optional[Sequence[str]] = None) -> None:
        if tags is None or "kv_cache" in tags:
            if getattr(self, "_kv_arena", None) is not None:
                if not self._kv_arena.mapped:
                    self._kv_arena.wake(zero=True)
            elif not self.k_cache:
                self._alloc_kv()
            self.asleep = False
        # tags == ["weights"]: nothing to map back; stay asleep until the KV cache returns

    def on_weights_updated(self, clear_kv: bool = True) -> None:
        """Called after the trainer pushed new weights into the model this engine reads."""
        self.weight_version += 1
        if clear_kv:
            self.rt.sbrt_sched_reset_prefix_cache(self.sched)

    def metrics(self) -> Dict[str, float]:
        m = dict(self.stats)
        m["num_running"] = sum(r is not None for r in self._slot_req)
        m["num_waiting"] = self.rt.sbrt_sched_num_waiting(self.sched)
        m["kv_free_blocks"] = self.rt.sbrt_sched_num_free_blocks(self.sched)
        m["kv_usage"] = 1.0 - m["kv_free_blocks"] / max(1, self.num_blocks)
        m["prefix_hit_rate"] = self.rt.sbrt_sched_prefix_hit_rate(self.sched)
        m["weight_version"] = self.weight_version
        if self._spec:
            drafted, accepted = (int(x) for x in self._spec_counts.tolist())
            m["spec_drafted"], m["spec_accepted"] = drafted, accepted
            m["spec_acceptance_rate"] = accepted / max(1, drafted)
        return m

    def __del__(self):
        try:
            if getattr(self, "sched", None):
                self.rt.sbrt_sched_destroy(self.sched)
                self.sched = None
        except Exception:
            pass


def _find_stop(detok, tokens: List[int], stops: List[str]) -> Optional[int]:
    """Smallest token count whose decoded text contains a stop string (the stop text is kept)."""
    text = detok(tokens)
    if not any(s in text for s in stops):
        return None
    lo, hi = 1, len(tokens)
    while lo < hi:
        mid = (lo + hi) // 2
        if any(s in detok(tokens[:mid]) for s in stops):
            hi = mid
        else:
            lo = mid + 1
    return lo


def _mask_logits_rows(logits, temp, top_k, top_p, min_p):
    """Per-row top-k / top-p / min-p masking (fp32 result, -inf outside the kept set)."""
    z = logits.float()
    t = torch.where(temp > 0, temp, torch.ones_like(temp))[:, None]
    zs, idx = torch.sort(z / t, dim=-1, descending=True)
    V = z.shape[-1]
    k = torch.where(top_k > 0, top_k, torch.full_like(top_k, V)).clamp(max=V).long()[:, None]
    rank = torch.arange(V, device=z.device)[None, :]
    remove = rank >= k
    probs = torch.softmax(zs, dim=-1)
    cum = probs.cumsum(-1)
    remove |= (cum - probs) >= top_p[:, None]
    remove |= probs < (min_p[:, None] * probs[:, :1])
    remove[:, 0] = False
    zs = zs.masked_fill(remove, float("-inf"))
    out = torch.full_like(z, float("-inf")).scatter(-1, idx, zs * t)
    return out
