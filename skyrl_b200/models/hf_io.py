"""HF checkpoint interchange: a dependency-free safetensors reader/writer and the translation
between HF parameter names (separate q/k/v and gate/up projections) and this package's fused
layout (``wqkv``, ``wgu``).  Export writes what ``save_pretrained(safe_serialization=True)`` would:
``config.json`` + ``model.safetensors`` (reference: fsdp_strategy.py:557-602 exports through HF).
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterator, List, Tuple

import numpy as np
import torch

_DT = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64, "I64": torch.int64,
       "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool}
_DT_INV = {v: k for k, v in _DT.items()}


def read_safetensors_header(path: str) -> Tuple[dict, int]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    return header, 8 + n


def load_safetensors(path: str, device="cpu") -> Dict[str, torch.Tensor]:
    header, base = read_safetensors_header(path)
    out = {}
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            s, e = meta["data_offsets"]
            dt = _DT[meta["dtype"]]
            buf = bytearray(mm[base + s : base + e])
            t = torch.frombuffer(buf, dtype=dt).reshape(meta["shape"]) if e > s else torch.empty(meta["shape"], dtype=dt)
            out[name] = t.to(device)
        mm.close()
    return out


def save_safetensors(tensors: Dict[str, torch.Tensor], path: str, metadata: Dict[str, str] | None = None) -> None:
    header = {}
    off = 0
    items = []
    for name in sorted(tensors):
        t = tensors[name].detach().contiguous().cpu()
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _DT_INV[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
        items.append(t)
    if metadata:
        header["__metadata__"] = metadata
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for t in items:
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)


# ----------------------------------------------------------------------------- name translation
def hf_names_for_layer(i: int, moe: bool) -> dict:
    p = f"model.layers.{i}."
    return {"ln1": p + "input_layernorm.weight", "ln2": p + "post_attention_layernorm.weight",
            "q": p + "self_attn.q_proj", "k": p + "self_attn.k_proj", "v": p + "self_attn.v_proj",
            "o": p + "self_attn.o_proj.weight", "q_norm": p + "self_attn.q_norm.weight",
            "k_norm": p + "self_attn.k_norm.weight", "gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
            "down": p + "mlp.down_proj.weight", "router": p + "mlp.gate.weight", "experts": p + "mlp.experts.",
            "sinks": p + "self_attn.sinks"}


def to_hf_state_dict(model) -> Dict[str, torch.Tensor]:
    """Unfuse this package's parameters into HF names (views where possible)."""
    a = model.args
    sd: Dict[str, torch.Tensor] = {"model.embed_tokens.weight": model.p("embed").detach()}
    for i in range(a.num_layers):
        n = hf_names_for_layer(i, bool(a.num_experts))
        pre = f"layers.{i}."
        sd[n["ln1"]] = model.p(pre + "ln1").detach()
        sd[n["ln2"]] = model.p(pre + "ln2").detach()
        w = model.p(pre + "wqkv").detach()
        sd[n["q"] + ".weight"], sd[n["k"] + ".weight"], sd[n["v"] + ".weight"] = (
            w[: a.q_dim], w[a.q_dim : a.q_dim + a.kv_dim], w[a.q_dim + a.kv_dim :])
        if a.attention_bias:
            b = model.p(pre + "bqkv").detach()
            sd[n["q"] + ".bias"], sd[n["k"] + ".bias"], sd[n["v"] + ".bias"] = (
                b[: a.q_dim], b[a.q_dim : a.q_dim + a.kv_dim], b[a.q_dim + a.kv_dim :])
        if a.qk_norm:
            sd[n["q_norm"]] = model.p(pre + "q_norm").detach()
            sd[n["k_norm"]] = model.p(pre + "k_norm").detach()
        if a.attention_sinks:
            sd[n["sinks"]] = model.p(pre + "sinks").detach()
        sd[n["o"]] = model.p(pre + "wo").detach()
        if a.num_experts:
            sd[n["router"]] = model.p(pre + "router").detach()
            wgu, wd = model.p(pre + "experts_wgu").detach(), model.p(pre + "experts_wd").detach()
            F = a.moe_intermediate_size
            for e in range(a.num_experts):
                sd[f"{n['experts']}{e}.gate_proj.weight"] = wgu[e, :F]
                sd[f"{n['experts']}{e}.up_proj.weight"] = wgu[e, F:]
                sd[f"{n['experts']}{e}.down_proj.weight"] = wd[e]
        else:
            wgu = model.p(pre + "wgu").detach()
            F = a.intermediate_size
            sd[n["gate"]], sd[n["up"]] = wgu[:F], wgu[F:]
            sd[n["down"]] = model.p(pre + "wd").detach()
    sd["model.norm.weight"] = model.p("final_norm").detach()
    if not a.tie_word_embeddings and "lm_head" in model._p:
        sd["lm_head.weight"] = model.p("lm_head").detach()
    if model.has_value_head:
        sd["value_head.weight"] = model.p("value_head").detach()[:1]
    return sd


@torch.no_grad()
def load_hf_state_dict(model, sd: Dict[str, torch.Tensor], strict: bool = True) -> List[str]:
    """Copy HF-named tensors into the fused parameters. Returns the names that were not consumed."""
    mine = to_hf_state_dict(model)  # HF-named *views* of our parameters: copy_ writes through
    used = set()
    for name, dst in mine.items():
        src = sd.get(name)
        if src is None and name.startswith("model."):
            src = sd.get(name[len("model."):])
        if src is None:
            if name == "value_head.weight" or not strict:
                continue
            raise KeyError(f"checkpoint is missing '{name}'")
        if tuple(src.shape) != tuple(dst.shape):
            raise ValueError(f"shape mismatch for '{name}': checkpoint {tuple(src.shape)} vs model {tuple(dst.shape)}")
        dst.copy_(src.to(dst.dtype))
        used.add(name)
    return [k for k in sd if k not in used and ("model." + k) not in used]


def iter_checkpoint_files(path: str) -> Iterator[str]:
    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        for fn in files:
            yield os.path.join(path, fn)
    else:
        single = os.path.join(path, "model.safetensors")
        if not os.path.exists(single):
            raise FileNotFoundError(f"no model.safetensors(.index.json) under {path}")
        yield single


def load_hf_weights(model, path: str, strict: bool = True) -> None:
    sd: Dict[str, torch.Tensor] = {}
    for fn in iter_checkpoint_files(path):
        sd.update(load_safetensors(fn))
    load_hf_state_dict(model, sd, strict=strict)


def save_hf_model(model, path: str, tokenizer=None, max_shard_bytes: int = 5 << 30) -> None:
    """Atomic export: write into ``path.tmp`` then rename (reference: fsdp_strategy.py:604-635)."""
    tmp = path.rstrip("/") + ".tmp"
    os.makedirs(tmp, exist_ok=True)
    sd = {k: v.contiguous() for k, v in to_hf_state_dict(model).items()}
    total = sum(v.numel() * v.element_size() for v in sd.values())
    if total <= max_shard_bytes:
        save_safetensors(sd, os.path.join(tmp, "model.safetensors"), {"format": "pt"})
    else:
        shards, cur, cur_b = [], {}, 0
        for k in sorted(sd):
            b = sd[k].numel() * sd[k].element_size()
            if cur and cur_b + b > max_shard_bytes:
                shards.append(cur)
                cur, cur_b = {}, 0
            cur[k] = sd[k]
            cur_b += b
        shards.append(cur)
        wm = {}
        for i, sh in enumerate(shards):
            fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
            save_safetensors(sh, os.path.join(tmp, fn), {"format": "pt"})
            wm.update({k: fn for k in sh})
        with open(os.path.join(tmp, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": wm}, f, indent=1)
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(model.args.to_hf_config(), f, indent=1)
    if tokenizer is not None and hasattr(tokenizer, "save_pretrained"):
        tokenizer.save_pretrained(tmp)
    if os.path.isdir(path):
        import shutil

        shutil.rmtree(path)
    os.replace(tmp, path)
