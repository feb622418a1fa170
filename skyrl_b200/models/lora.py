"""Low-rank adapters on the fused projection weights, trained with the same GEMM kernels and sharded optimizer.

The reference wraps the HF model with ``peft.get_peft_model`` (skyrl/backends/skyrl_train/workers/model_wrapper.py:120-170,
config ``trainer.policy.model.lora.{rank,alpha,dropout,target_modules,init_method}``) and ships adapters to the rollout
engine as files (``/skyrl/v1/load_lora_adapter``).  Here the adapter parameters live in their own flat buffer (so the
optimizer state is adapter-sized), the frozen base stays in the model's flat buffer, and the colocated engine receives
merged weights ``W + (alpha/r) B A`` computed by one small GEMM per projection.  Adapters are exported in the PEFT
layout (``adapter_config.json`` + ``adapter_model.safetensors``); a fused QKV (or gate/up) adapter exports as
per-projection adapters that share their ``lora_A``.

Ranks are padded to a multiple of 8 (GEMM row alignment); the padding rows/columns start at zero and receive zero
gradients, so they stay zero.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops import gemm
from .decoder import CausalLM, ModelArgs, _align

# module name -> (fused weight it adapts, HF projection names inside it)
TARGETS = {"qkv": ("wqkv", ("q_proj", "k_proj", "v_proj")), "o": ("wo", ("o_proj",)),
           "gate_up": ("wgu", ("gate_proj", "up_proj")), "down": ("wd", ("down_proj",))}
_HF_TO_MODULE = {"q_proj": "qkv", "k_proj": "qkv", "v_proj": "qkv", "o_proj": "o", "gate_proj": "gate_up",
                 "up_proj": "gate_up", "down_proj": "down"}


def resolve_targets(target_modules, exclude_modules=None) -> List[str]:
    """``"all-linear"`` or a list / comma string of HF projection names -> fused module names adapted here."""
    if target_modules in (None, "all-linear", "all_linear"):
        mods = list(TARGETS)
    else:
        names = target_modules.split(",") if isinstance(target_modules, str) else list(target_modules)
        mods = []
        for n in (x.strip() for x in names):
            m = _HF_TO_MODULE.get(n, n if n in TARGETS else None)
            if m is None:
                raise ValueError(f"unknown LoRA target module '{n}'")
            if m not in mods:
                mods.append(m)
    if exclude_modules:
        ex = exclude_modules.split(",") if isinstance(exclude_modules, str) else list(exclude_modules)
        drop = {_HF_TO_MODULE.get(x.strip(), x.strip()) for x in ex}
        mods = [m for m in mods if m not in drop]
    return mods


class LoRACausalLM(CausalLM):
    """``CausalLM`` with frozen base weights and trainable adapters. ``flat_params`` is the *adapter* buffer (what
    the optimizer and gradient buffers see); the base buffer is ``base_flat_params``."""

    def __init__(self, args: ModelArgs, rank: int, alpha: float = 16.0, dropout: float = 0.0, target_modules="all-linear",
                 exclude_modules=None, init_method: str = "kaiming", device="cpu", dtype=torch.bfloat16,
                 flat_buffer: Optional[torch.Tensor] = None, seed: Optional[int] = 0, lora_seed: Optional[int] = None):
        if args.num_experts:
            raise ValueError("LoRA on MoE expert weights is not supported")
        super().__init__(args, device=device, dtype=dtype, flat_buffer=flat_buffer, seed=seed)
        self.lora_rank, self.lora_alpha, self.lora_dropout = int(rank), float(alpha), float(dropout)
        self.r_pad = (self.lora_rank + 7) // 8 * 8
        self.scale = self.lora_alpha / self.lora_rank
        self.lora_modules = resolve_targets(target_modules, exclude_modules)
        self.base_flat_params = self.flat_params
        self.base_specs, self.base_offsets, self.base_flat_numel = self.specs, self.offsets, self.flat_numel
        for p in self._p.values():
            p.requires_grad_(False)
        # adapter layout
        self.lora_specs: List[Tuple[str, Tuple[int, int]]] = []
        for i in range(args.num_layers):
            for m in self.lora_modules:
                w = self._p[f"layers.{i}.{TARGETS[m][0]}"]
                self.lora_specs.append((f"layers.{i}.{m}.lora_A", (self.r_pad, w.shape[1])))
                self.lora_specs.append((f"layers.{i}.{m}.lora_B", (w.shape[0], self.r_pad)))
        off = 0
        self.lora_offsets: Dict[str, Tuple[int, int]] = {}
        for name, shape in self.lora_specs:
            n = shape[0] * shape[1]
            self.lora_offsets[name] = (off, n)
            off += _align(n)
        self.lora_flat_numel = _align(off, 8192)
        self.flat_params = torch.zeros(self.lora_flat_numel, device=device, dtype=dtype)
        self.flat_numel = self.lora_flat_numel
        self._lora: Dict[str, nn.Parameter] = {}
        for name, shape in self.lora_specs:
            o, n = self.lora_offsets[name]
            prm = nn.Parameter(self.flat_params[o : o + n].view(shape), requires_grad=True)
            self._lora[name] = prm
            self.register_parameter("lora_" + name.replace(".", "_"), prm)
        self.reset_lora(lora_seed if lora_seed is not None else (seed or 0) + 1, init_method)

    # ------------------------------------------------------------------ parameters
    @torch.no_grad()
    def reset_lora(self, seed: int = 1, init_method: str = "kaiming") -> None:
        g = torch.Generator(device="cpu").manual_seed(seed)
        r = self.lora_rank
        for name, shape in self.lora_specs:
            prm = self._lora[name]
            prm.zero_()
            if name.endswith("lora_A"):
                fan_in = shape[1]
                if init_method == "gaussian":
                    a = torch.randn(r, fan_in, generator=g) / r
                else:  # kaiming uniform with a = sqrt(5), as peft does
                    bound = 1.0 / math.sqrt(fan_in)
                    a = (torch.rand(r, fan_in, generator=g) * 2 - 1) * bound
                prm[:r].copy_(a.to(prm.dtype))

    def attach_main_grad(self, flat_grad: torch.Tensor) -> None:
        assert flat_grad.dtype == torch.float32 and flat_grad.numel() >= self.lora_flat_numel
        self.flat_main_grad = flat_grad
        for name, shape in self.lora_specs:
            o, n = self.lora_offsets[name]
            self._lora[name].main_grad = flat_grad[o : o + n].view(shape)

    def trainable_named(self) -> Iterable[Tuple[str, nn.Parameter]]:
        return self._lora.items()

    def num_trainable_parameters(self) -> int:
        return sum(s[0] * s[1] for _, s in self.lora_specs)

    # ------------------------------------------------------------------ forward
    def _lin(self, i: int, module: str, x: torch.Tensor, bias=None) -> torch.Tensor:
        w = self.p(f"layers.{i}.{TARGETS[module][0]}")
        y = gemm.linear(x, w, bias)
        if module in self.lora_modules:
            xa = x
            if self.lora_dropout > 0 and self.training and torch.is_grad_enabled():
                xa = torch.nn.functional.dropout(x, self.lora_dropout)
            z = gemm.linear(gemm.linear(xa, self._lora[f"layers.{i}.{module}.lora_A"]), self._lora[f"layers.{i}.{module}.lora_B"])
            y = y + self.scale * z
        return y

    def _layer(self, i: int, x, delta, pos, cu, max_seqlen, kv_sink=None, attn_fn=None):
        a = self.args
        pre = f"layers.{i}."
        x, h = ew.add_rmsnorm(x, delta, self.p(pre + "ln1"), a.rms_norm_eps)
        qkv = self._lin(i, "qkv", h, self._p.get(pre + "bqkv"))
        if a.qk_norm:
            qkv = self._qk_norm(qkv, i)
        qkv = ew.rope(qkv, pos, self.rope_table(qkv.device), a.num_heads + a.num_kv_heads, a.head_dim)
        if kv_sink is not None:
            kv_sink(i, qkv)
        if attn_fn is not None:
            att = attn_fn(i, qkv)
        else:
            att = attn_ops.attn_varlen(qkv, cu, a.num_heads, a.num_kv_heads, a.head_dim, max_seqlen=max_seqlen)
        o = self._lin(i, "o", att)
        x, h = ew.add_rmsnorm(x, o, self.p(pre + "ln2"), a.rms_norm_eps)
        d = self._lin(i, "down", ew.swiglu(self._lin(i, "gate_up", h)))
        return x, d

    # ------------------------------------------------------------------ merge / export
    @torch.no_grad()
    def merged_weight(self, i: int, module: str) -> torch.Tensor:
        w = self.p(f"layers.{i}.{TARGETS[module][0]}")
        if module not in self.lora_modules:
            return w
        A, B = self._lora[f"layers.{i}.{module}.lora_A"], self._lora[f"layers.{i}.{module}.lora_B"]
        delta = gemm.gemm_nn(B.contiguous(), A.contiguous()) if A.is_cuda else (B.float() @ A.float())
        return (w.float() + self.scale * delta.float()).to(w.dtype)

    @torch.no_grad()
    def merge_into(self, target: CausalLM) -> None:
        """Write ``base + scale * B A`` into ``target``'s parameters (everything else is copied unchanged)."""
        for name, prm in target.named_flat_views():
            parts = name.split(".")
            mod = next((m for m, (wn, _) in TARGETS.items() if len(parts) == 3 and parts[2] == wn), None)
            if mod is not None:
                prm.copy_(self.merged_weight(int(parts[1]), mod))
            else:
                prm.copy_(self.p(name))

    def lora_state_dict(self) -> Dict[str, torch.Tensor]:
        """PEFT key names; fused adapters are split per projection (shared ``lora_A``)."""
        a, r = self.args, self.lora_rank
        out: Dict[str, torch.Tensor] = {}
        for i in range(a.num_layers):
            for m in self.lora_modules:
                A = self._lora[f"layers.{i}.{m}.lora_A"][:r].detach()
                B = self._lora[f"layers.{i}.{m}.lora_B"][:, :r].detach()
                if m == "qkv":
                    splits = [("self_attn.q_proj", 0, a.q_dim), ("self_attn.k_proj", a.q_dim, a.q_dim + a.kv_dim),
                              ("self_attn.v_proj", a.q_dim + a.kv_dim, a.qkv_dim)]
                elif m == "o":
                    splits = [("self_attn.o_proj", 0, B.shape[0])]
                elif m == "gate_up":
                    F = a.intermediate_size
                    splits = [("mlp.gate_proj", 0, F), ("mlp.up_proj", F, 2 * F)]
                else:
                    splits = [("mlp.down_proj", 0, B.shape[0])]
                for hf, lo, hi in splits:
                    k = f"base_model.model.model.layers.{i}.{hf}"
                    out[k + ".lora_A.weight"] = A.clone().contiguous()
                    out[k + ".lora_B.weight"] = B[lo:hi].clone().contiguous()
        return out

    def save_adapter(self, path: str) -> None:
        from . import hf_io

        os.makedirs(path, exist_ok=True)
        hf_io.save_safetensors({k: v.cpu() for k, v in self.lora_state_dict().items()},
                               os.path.join(path, "adapter_model.safetensors"), {"format": "pt"})
        hf_targets = sorted({h for m in self.lora_modules for h in TARGETS[m][1]})
        with open(os.path.join(path, "adapter_config.json"), "w") as f:
            json.dump({"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": self.lora_rank, "lora_alpha": self.lora_alpha,
                       "lora_dropout": self.lora_dropout, "target_modules": hf_targets, "bias": "none",
                       "fused_shared_lora_A": True}, f, indent=1)

    @torch.no_grad()
    def load_adapter(self, path: str) -> None:
        """Inverse of ``save_adapter`` (requires the shared-``lora_A`` layout this class writes)."""
        from . import hf_io

        sd = hf_io.load_safetensors(os.path.join(path, "adapter_model.safetensors"))
        a, r = self.args, self.lora_rank
        for i in range(a.num_layers):
            for m in self.lora_modules:
                names = {"qkv": ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"], "o": ["self_attn.o_proj"],
                         "gate_up": ["mlp.gate_proj", "mlp.up_proj"], "down": ["mlp.down_proj"]}[m]
                pre = f"base_model.model.model.layers.{i}."
                A = sd[pre + names[0] + ".lora_A.weight"]
                for n in names[1:]:
                    if not torch.equal(sd[pre + n + ".lora_A.weight"], A):
                        raise ValueError(f"adapter at {path} has distinct lora_A for fused projections of layer {i}; "
                                         "only shared-A adapters can be loaded into fused weights")
                B = torch.cat([sd[pre + n + ".lora_B.weight"] for n in names], 0)
                pa, pb = self._lora[f"layers.{i}.{m}.lora_A"], self._lora[f"layers.{i}.{m}.lora_B"]
                pa.zero_()
                pb.zero_()
                pa[:r].copy_(A.to(pa.dtype))
                pb[:, :r].copy_(B.to(pb.dtype))
