"""Decoder-only transformer (Llama / Qwen2 / Qwen3 / Qwen3-MoE families) built on the sm_100a ops.

Differences from the HF modules the reference wraps
(skyrl/backends/skyrl_train/workers/model_wrapper.py:36-398):

* activations are always *packed*: one token axis ``[T, H]`` plus ``cu_seqlens`` -- there is no
  padded ``[B, S]`` form inside the model, so nothing is unpadded or re-padded per layer;
* Q, K and V come from one fused projection and are read in place by the attention kernels;
  gate and up are one projection feeding the SwiGLU kernel;
* every parameter is a view into one flat bf16 buffer (``flat_params``) so that the sharded
  optimizer, the trainer->engine weight push and checkpoints handle a single contiguous range;
* parameter gradients are accumulated by the backward kernels directly into a flat fp32 buffer
  (``main_grad`` views) when one is attached, and ``.grad`` stays unused.

The HF checkpoint naming is translated in ``hf_io``.
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.utils.checkpoint

from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops import gemm
from ..ops import lm_head as lm_head_ops


@dataclass
class ModelArgs:
    vocab_size: int = 1024
    hidden_size: int = 256
    num_layers: int = 2
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 64
    intermediate_size: int = 512
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    attention_bias: bool = False  # Qwen2: bias on q/k/v projections
    qk_norm: bool = False  # Qwen3: per-head RMSNorm on q and k
    attention_sinks: bool = False  # GPT-OSS: one learned sink logit per query head in every attention softmax
    # mixture of experts (0 experts = dense FFN)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    model_type: str = "qwen2"
    init_std: float = 0.02
    ep_size: int = 1  # expert parallelism: this rank stores num_experts / ep_size experts (routing stays global)
    lm_head_rows: int = 0  # vocabulary-parallel LM head: rows of the head stored on this rank (0 = the whole vocabulary)

    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    @classmethod
    def from_hf_config(cls, cfg: dict) -> "ModelArgs":
        mt = cfg.get("model_type", "llama")
        heads = cfg["num_attention_heads"]
        return cls(
            vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"], num_layers=cfg["num_hidden_layers"],
            num_heads=heads, num_kv_heads=cfg.get("num_key_value_heads", heads),
            head_dim=cfg.get("head_dim") or cfg["hidden_size"] // heads,
            intermediate_size=cfg.get("intermediate_size", 0), rms_norm_eps=cfg.get("rms_norm_eps", 1e-6),
            rope_theta=float(cfg.get("rope_theta", 10000.0)),
            max_position_embeddings=cfg.get("max_position_embeddings", 32768),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            attention_bias=bool(cfg.get("attention_bias", mt == "qwen2")), qk_norm=mt in ("qwen3", "qwen3_moe"),
            attention_sinks=bool(cfg.get("attention_sinks", False)),
            num_experts=cfg.get("num_experts", 0) or 0, num_experts_per_tok=cfg.get("num_experts_per_tok", 0) or 0,
            moe_intermediate_size=cfg.get("moe_intermediate_size", 0) or 0,
            norm_topk_prob=bool(cfg.get("norm_topk_prob", True)), model_type=mt,
        )  # fmt: skip

    def to_hf_config(self) -> dict:
        arch = {"llama": "LlamaForCausalLM", "qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM",
                "qwen3_moe": "Qwen3MoeForCausalLM"}.get(self.model_type, "LlamaForCausalLM")
        cfg = {
            "architectures": [arch], "model_type": self.model_type, "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size, "num_hidden_layers": self.num_layers,
            "num_attention_heads": self.num_heads, "num_key_value_heads": self.num_kv_heads,
            "head_dim": self.head_dim, "intermediate_size": self.intermediate_size,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings, "attention_bias": self.attention_bias,
            "hidden_act": "silu", "torch_dtype": "bfloat16",
        }  # fmt: skip
        if self.attention_sinks:
            cfg["attention_sinks"] = True
        if self.num_experts:
            cfg.update(num_experts=self.num_experts, num_experts_per_tok=self.num_experts_per_tok,
                       moe_intermediate_size=self.moe_intermediate_size, norm_topk_prob=self.norm_topk_prob)
        return cfg


# named architectures used by the benchmark configurations (random-init, no checkpoint needed)
PRESETS: Dict[str, ModelArgs] = {
    "tiny-llama": ModelArgs(vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                            intermediate_size=512, rope_theta=1e4, model_type="llama"),
    "tiny-qwen2-d128": ModelArgs(vocab_size=2048, hidden_size=256, num_layers=2, num_heads=2, num_kv_heads=1,
                                 head_dim=128, intermediate_size=512, rope_theta=1e4, attention_bias=True,
                                 tie_word_embeddings=True, model_type="qwen2"),
    "tiny-sinks": ModelArgs(vocab_size=2048, hidden_size=256, num_layers=2, num_heads=2, num_kv_heads=1, head_dim=128,
                            intermediate_size=512, rope_theta=1e4, attention_sinks=True, model_type="llama"),
    "tiny-qwen2-tp": ModelArgs(vocab_size=2048, hidden_size=512, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=128,
                               intermediate_size=1024, rope_theta=1e4, attention_bias=True, tie_word_embeddings=True,
                               model_type="qwen2"),
    "tiny-llama-d128": ModelArgs(vocab_size=2048, hidden_size=512, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=128,
                                 intermediate_size=1024, rope_theta=1e4, model_type="llama"),
    "tiny-moe": ModelArgs(vocab_size=1024, hidden_size=256, num_layers=2, num_heads=2, num_kv_heads=1, head_dim=128,
                          intermediate_size=512, rope_theta=1e4, num_experts=8, num_experts_per_tok=2,
                          moe_intermediate_size=128, model_type="qwen3_moe", qk_norm=True),
    "qwen2.5-0.5b": ModelArgs(vocab_size=151936, hidden_size=896, num_layers=24, num_heads=14, num_kv_heads=2,
                              head_dim=64, intermediate_size=4864, rope_theta=1e6, attention_bias=True,
                              tie_word_embeddings=True, model_type="qwen2"),
    "qwen2.5-1.5b": ModelArgs(vocab_size=151936, hidden_size=1536, num_layers=28, num_heads=12, num_kv_heads=2,
                              head_dim=128, intermediate_size=8960, rope_theta=1e6, attention_bias=True,
                              tie_word_embeddings=True, model_type="qwen2"),
    "qwen2.5-7b": ModelArgs(vocab_size=152064, hidden_size=3584, num_layers=28, num_heads=28, num_kv_heads=4,
                            head_dim=128, intermediate_size=18944, rope_theta=1e6, attention_bias=True,
                            tie_word_embeddings=False, model_type="qwen2"),
    "qwen3-30b-a3b": ModelArgs(vocab_size=151936, hidden_size=2048, num_layers=48, num_heads=32, num_kv_heads=4,
                               head_dim=128, intermediate_size=6144, rope_theta=1e6, qk_norm=True, num_experts=128,
                               num_experts_per_tok=8, moe_intermediate_size=768, model_type="qwen3_moe"),
}


def _param_specs(a: ModelArgs, with_lm_head: bool = True, value_head: bool = False) -> List[Tuple[str, Tuple[int, ...]]]:
    """Ordered (name, shape) list that defines the flat parameter layout."""
    specs: List[Tuple[str, Tuple[int, ...]]] = [("embed", (a.vocab_size, a.hidden_size))]
    for i in range(a.num_layers):
        p = f"layers.{i}."
        specs.append((p + "ln1", (a.hidden_size,)))
        specs.append((p + "wqkv", (a.qkv_dim, a.hidden_size)))
        if a.attention_bias:
            specs.append((p + "bqkv", (a.qkv_dim,)))
        if a.qk_norm:
            specs.append((p + "q_norm", (a.head_dim,)))
            specs.append((p + "k_norm", (a.head_dim,)))
        if a.attention_sinks:
            specs.append((p + "sinks", (a.num_heads,)))
        specs.append((p + "wo", (a.hidden_size, a.q_dim)))
        specs.append((p + "ln2", (a.hidden_size,)))
        if a.num_experts:
            specs.append((p + "router", (a.num_experts, a.hidden_size)))
            el = a.num_experts // max(1, a.ep_size)
            specs.append((p + "experts_wgu", (el, 2 * a.moe_intermediate_size, a.hidden_size)))
            specs.append((p + "experts_wd", (el, a.hidden_size, a.moe_intermediate_size)))
        else:
            specs.append((p + "wgu", (2 * a.intermediate_size, a.hidden_size)))
            specs.append((p + "wd", (a.hidden_size, a.intermediate_size)))
    specs.append(("final_norm", (a.hidden_size,)))
    if with_lm_head and not a.tie_word_embeddings and not value_head:
        specs.append(("lm_head", (a.lm_head_rows or a.vocab_size, a.hidden_size)))
    if value_head:
        specs.append(("value_head", (8, a.hidden_size)))  # row 0 is the head; 8 rows keep GEMM alignment
    return specs


def _align(n: int, a: int = 128) -> int:
    return (n + a - 1) // a * a


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        ctx.save_for_backward(ids)
        ctx.table = table
        return table[ids.long()]

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        table = ctx.table
        main_grad = getattr(table, "main_grad", None)
        if main_grad is not None:
            main_grad.index_add_(0, ids.long(), dy.float())
            return None, None
        g = torch.zeros_like(table, dtype=torch.float32)
        g.index_add_(0, ids.long(), dy.float())
        return None, g.to(table.dtype)


class CausalLM(nn.Module):
    """Packed-sequence causal LM. ``forward`` returns final-normed hidden states ``[T, H]``."""

    def __init__(self, args: ModelArgs, device="cpu", dtype=torch.bfloat16, value_head: bool = False,
                 flat_buffer: Optional[torch.Tensor] = None, seed: Optional[int] = 0):
        super().__init__()
        self.args = args
        self.has_value_head = value_head
        self.specs = _param_specs(args, value_head=value_head)
        self.offsets: Dict[str, Tuple[int, int]] = {}
        off = 0
        for name, shape in self.specs:
            n = math.prod(shape)
            self.offsets[name] = (off, n)
            off += _align(n)
        self.flat_numel = _align(off, 8192)  # divisible by 8 * world for world <= 8 with 128-element shards
        if flat_buffer is None:
            flat_buffer = torch.zeros(self.flat_numel, device=device, dtype=dtype)
        assert flat_buffer.numel() >= self.flat_numel
        self.flat_params = flat_buffer
        self._p: Dict[str, nn.Parameter] = {}
        for name, shape in self.specs:
            o, n = self.offsets[name]
            prm = nn.Parameter(flat_buffer[o : o + n].view(shape), requires_grad=True)
            self._p[name] = prm
            self.register_parameter(name.replace(".", "_"), prm)
        self.gradient_checkpointing = False
        self._rope_table: Optional[torch.Tensor] = None
        if seed is not None:
            self.reset_parameters(seed)

    # ------------------------------------------------------------------ params
    def p(self, name: str) -> nn.Parameter:
        return self._p[name]

    def named_flat_views(self):
        for name, _ in self.specs:
            yield name, self._p[name]

    @torch.no_grad()
    def reset_parameters(self, seed: int = 0) -> None:
        gen = torch.Generator(device="cpu").manual_seed(seed)
        for name, shape in self.specs:
            prm = self._p[name]
            leaf = name.split(".")[-1]
            if leaf in ("ln1", "ln2", "final_norm", "q_norm", "k_norm"):
                prm.fill_(1.0)
            elif leaf in ("bqkv", "sinks"):
                prm.zero_()
            else:
                # generate in chunks on CPU for device-independent, reproducible weights
                flat = prm.view(-1)
                step = 1 << 24
                for s in range(0, flat.numel(), step):
                    e = min(flat.numel(), s + step)
                    flat[s:e] = (torch.randn(e - s, generator=gen) * self.args.init_std).to(flat.dtype)

    def attach_main_grad(self, flat_grad: torch.Tensor) -> None:
        """Route parameter gradients into views of ``flat_grad`` (fp32, same layout as ``flat_params``)."""
        assert flat_grad.dtype == torch.float32 and flat_grad.numel() >= self.flat_numel
        self.flat_main_grad = flat_grad
        for name, shape in self.specs:
            o, n = self.offsets[name]
            self._p[name].main_grad = flat_grad[o : o + n].view(shape)

    def rope_table(self, device) -> torch.Tensor:
        if self._rope_table is None or self._rope_table.device != torch.device(device):
            self._rope_table = ew.build_rope_table(self.args.max_position_embeddings, self.args.head_dim,
                                                   self.args.rope_theta, device)
        return self._rope_table

    # ------------------------------------------------------------------ forward
    def _qk_norm(self, qkv: torch.Tensor, i: int) -> torch.Tensor:
        a = self.args
        T = qkv.shape[0]
        q = qkv[:, : a.q_dim].reshape(T * a.num_heads, a.head_dim)
        k = qkv[:, a.q_dim : a.q_dim + a.kv_dim].reshape(T * a.num_kv_heads, a.head_dim)
        q = ew.rmsnorm(q, self.p(f"layers.{i}.q_norm"), a.rms_norm_eps).reshape(T, a.q_dim)
        k = ew.rmsnorm(k, self.p(f"layers.{i}.k_norm"), a.rms_norm_eps).reshape(T, a.kv_dim)
        return torch.cat([q, k, qkv[:, a.q_dim + a.kv_dim :]], dim=-1)

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
        if attn_fn is not None:  # the caller supplies attention (e.g. over cached key/value prefixes)
            att = attn_fn(i, qkv)
        else:
            att = attn_ops.attn_varlen(qkv, cu, a.num_heads, a.num_kv_heads, a.head_dim, max_seqlen=max_seqlen,
                                       sinks=self._p.get(pre + "sinks"))
        o = gemm.linear(att, self.p(pre + "wo"))
        x, h = ew.add_rmsnorm(x, o, self.p(pre + "ln2"), a.rms_norm_eps)
        if a.num_experts and getattr(self, "ep", None) is not None:
            from ..parallel.expert_parallel import moe_ffn_ep

            d = moe_ffn_ep(h, self.p(pre + "router"), self.p(pre + "experts_wgu"), self.p(pre + "experts_wd"),
                           a.num_experts_per_tok, a.norm_topk_prob, self.ep, a.num_experts, layer=i)
        elif a.num_experts:
            from .moe import moe_ffn

            d = moe_ffn(h, self.p(pre + "router"), self.p(pre + "experts_wgu"), self.p(pre + "experts_wd"),
                        a.num_experts_per_tok, a.norm_topk_prob, layer=i, qat=getattr(self, "fake_int4_qat", None))
        else:
            d = gemm.swiglu_mlp(h, self.p(pre + "wgu"), self.p(pre + "wd"))
        return x, d

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor, cu_seqlens: torch.Tensor,
                max_seqlen: int = 0, kv_sink=None, attn_fn=None) -> torch.Tensor:
        """``input_ids`` / ``positions``: ``[T]``; ``cu_seqlens``: int32 ``[B+1]``. Returns hidden ``[T, H]``."""
        x = _EmbeddingFn.apply(input_ids, self.p("embed"))
        delta = None
        ready = getattr(self, "layer_grads_ready", None)  # callable(i): every parameter gradient of layer i is final
        for i in range(self.args.num_layers):
            if ready is not None and torch.is_grad_enabled() and x.requires_grad:
                # the gradient of a layer's input is produced by the last backward node of that layer
                x.register_hook(lambda g, i=i: ready(i))
            if self.gradient_checkpointing and torch.is_grad_enabled():
                if delta is None:
                    delta = torch.zeros_like(x)
                x, delta = torch.utils.checkpoint.checkpoint(self._layer, i, x, delta, positions, cu_seqlens,
                                                             max_seqlen, use_reentrant=False)
            else:
                x, delta = self._layer(i, x, delta, positions, cu_seqlens, max_seqlen, kv_sink, attn_fn)
        _, h = ew.add_rmsnorm(x, delta, self.p("final_norm"), self.args.rms_norm_eps)
        return h

    def lm_head_weight(self) -> torch.Tensor:
        return self.p("embed") if self.args.tie_word_embeddings else self.p("lm_head")

    def token_logprobs(self, hidden: torch.Tensor, targets: torch.Tensor, temperature: float = 1.0,
                       with_entropy: bool = False):
        """Log-probability (and optionally entropy) of ``targets[t]`` under the LM head, without logits."""
        return lm_head_ops.lm_head_logprobs(hidden, self.lm_head_weight(), targets, 1.0 / temperature, with_entropy)

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return gemm.gemm_nt(hidden, self.lm_head_weight())

    def values(self, hidden: torch.Tensor) -> torch.Tensor:
        assert self.has_value_head
        return gemm.linear(hidden, self.p("value_head"))[:, 0].float()

    def num_parameters(self) -> int:
        return sum(math.prod(s) for _, s in self.specs)


def param_offsets(args: ModelArgs, value_head: bool = False) -> Dict[str, Tuple[int, int]]:
    """name -> (element offset, numel) of the flat parameter buffer ``CausalLM`` lays out for ``args`` (no allocation)."""
    off, out = 0, {}
    for name, shape in _param_specs(args, value_head=value_head):
        n = math.prod(shape)
        out[name] = (off, n)
        off += _align(n)
    return out


def flat_numel_for(args: ModelArgs, value_head: bool = False) -> int:
    """Size (elements) of the flat parameter buffer ``CausalLM`` lays out for ``args``."""
    off = 0
    for _, shape in _param_specs(args, value_head=value_head):
        off += _align(math.prod(shape))
    return _align(off, 8192)


def resolve_model_args(name_or_path: str, model_config_kwargs: Optional[dict] = None) -> ModelArgs:
    import dataclasses

    if name_or_path in PRESETS:
        return dataclasses.replace(PRESETS[name_or_path], **(model_config_kwargs or {}))
    with open(os.path.join(name_or_path, "config.json")) as f:
        return ModelArgs.from_hf_config(json.load(f))


def build_model(name_or_path: str, device="cpu", dtype=torch.bfloat16, value_head: bool = False, seed: int = 0,
                model_config_kwargs: Optional[dict] = None, flat_buffer: Optional[torch.Tensor] = None) -> CausalLM:
    """Build from a preset name (random init) or from an HF checkpoint directory (weights loaded)."""
    if name_or_path in PRESETS:
        import dataclasses

        args = dataclasses.replace(PRESETS[name_or_path], **(model_config_kwargs or {}))
        return CausalLM(args, device=device, dtype=dtype, value_head=value_head, seed=seed, flat_buffer=flat_buffer)
    cfg_path = os.path.join(name_or_path, "config.json")
    if not os.path.exists(cfg_path):
        raise FileNotFoundError(f"'{name_or_path}' is neither a preset ({sorted(PRESETS)}) nor a checkpoint directory")
    with open(cfg_path) as f:
        args = ModelArgs.from_hf_config(json.load(f))
    model = CausalLM(args, device=device, dtype=dtype, value_head=value_head, seed=None, flat_buffer=flat_buffer)
    from . import hf_io

    hf_io.load_hf_weights(model, name_or_path)
    return model
