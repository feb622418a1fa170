"""Rendering of chat / Tinker model inputs into token ids, with multimodal placeholders.

References: skyrl/backends/renderer.py (Tinker ``ModelInput`` chunks -> token ids, image chunks expanded to placeholder
tokens through a render endpoint), skyrl/backends/skyrl_train/inference_servers/render_server.py:115-265 (a CPU-only
server exposing that endpoint so that tokenisation of multimodal prompts needs no GPU engine).

The image path is model-agnostic: an ``ImageProcessor`` turns image bytes into ``(pixel_values [n_patches, patch_dim],
grid_thw [1, 3])`` and tells how many placeholder tokens the prompt needs.  ``PatchImageProcessor`` is a dependency-free
processor (fixed square patches of the decoded RGB image) used by tests and by models that take raw patches; real
vision towers plug in their own processor.
"""

from __future__ import annotations

import base64
import io
import math
from typing import Any, Dict, List, NamedTuple, Optional, Sequence

import numpy as np
import torch
from ..utils.tokenizer import chat_template_ids


class RenderedModelInput(NamedTuple):
    prompt_ids: List[int]
    pixel_values: Optional[torch.Tensor] = None
    image_grid_thw: Optional[torch.Tensor] = None
    placeholder_ranges: Optional[List[tuple]] = None  # (offset, length) of every image's placeholder span


class PatchImageProcessor:
    """RGB image -> non-overlapping ``patch x patch`` patches (row-major), ``merge**2`` patches per placeholder token."""

    def __init__(self, patch: int = 14, merge: int = 2, max_side: int = 448):
        self.patch, self.merge, self.max_side = patch, merge, max_side

    def decode(self, data: bytes) -> np.ndarray:
        try:
            from PIL import Image

            img = Image.open(io.BytesIO(data)).convert("RGB")
            if max(img.size) > self.max_side:
                s = self.max_side / max(img.size)
                img = img.resize((max(1, int(img.size[0] * s)), max(1, int(img.size[1] * s))))
            return np.asarray(img, dtype=np.float32) / 255.0
        except ImportError:
            arr = np.load(io.BytesIO(data), allow_pickle=False)  # tests ship .npy payloads when PIL is absent
            return arr.astype(np.float32)

    def __call__(self, data: bytes):
        img = self.decode(data)
        unit = self.patch * self.merge
        H = max(unit, int(math.ceil(img.shape[0] / unit)) * unit)
        W = max(unit, int(math.ceil(img.shape[1] / unit)) * unit)
        canvas = np.zeros((H, W, 3), dtype=np.float32)
        canvas[: img.shape[0], : img.shape[1]] = img[:H, :W, :3]
        gh, gw = H // self.patch, W // self.patch
        patches = canvas.reshape(gh, self.patch, gw, self.patch, 3).transpose(0, 2, 1, 3, 4).reshape(gh * gw, -1)
        grid = torch.tensor([[1, gh, gw]], dtype=torch.long)
        n_tokens = (gh // self.merge) * (gw // self.merge)
        return torch.from_numpy(np.ascontiguousarray(patches)), grid, n_tokens


def _chunk_bytes(ch: Dict[str, Any]) -> bytes:
    data = ch.get("data")
    if isinstance(data, str):
        return base64.b64decode(data)
    if isinstance(data, (bytes, bytearray)):
        return bytes(data)
    loc = ch.get("location")
    if loc:
        from ..utils import io as sio

        with sio.open_file(loc, "rb") as f:
            return f.read()
    raise ValueError("image chunk carries neither data nor location")


def render_model_input(model_inputs: Sequence[Dict[str, Any]], image_token_id: Optional[int] = None,
                       processor: Optional[PatchImageProcessor] = None) -> List[RenderedModelInput]:
    """Tinker ``ModelInput`` dicts -> token ids (+ vision tensors).  Text-only inputs need no processor."""
    out = []
    for mi in model_inputs:
        ids: List[int] = []
        pvs, grids, spans = [], [], []
        for ch in mi.get("chunks", []):
            if "tokens" in ch:
                ids.extend(int(t) for t in ch["tokens"])
                continue
            if processor is None or image_token_id is None:
                raise ValueError("image chunks need an image processor and the model's image placeholder token id")
            pv, grid, n = processor(_chunk_bytes(ch))
            exp = ch.get("expected_tokens")
            if exp is not None and int(exp) != n:
                raise ValueError(f"image expands to {n} placeholder tokens but the request expected {exp}")
            spans.append((len(ids), n))
            ids.extend([image_token_id] * n)
            pvs.append(pv)
            grids.append(grid)
        out.append(RenderedModelInput(ids, torch.cat(pvs, 0) if pvs else None, torch.cat(grids, 0) if grids else None,
                                      spans or None))
    return out


def render_chat(messages: List[Dict[str, Any]], tokenizer, image_token_id: Optional[int] = None,
                processor: Optional[PatchImageProcessor] = None, add_generation_prompt: bool = True) -> RenderedModelInput:
    """OpenAI-style messages whose ``content`` may be a list of ``{"type": "text"|"image_url", ...}`` parts."""
    flat, images = [], []
    marker = "<|image_pad_marker|>"
    for m in messages:
        c = m.get("content")
        if isinstance(c, list):
            text = ""
            for part in c:
                if part.get("type") == "text":
                    text += part.get("text", "")
                elif part.get("type") in ("image_url", "image"):
                    url = part.get("image_url", {}).get("url") if part.get("type") == "image_url" else part.get("image")
                    images.append(url)
                    text += marker
            flat.append({**m, "content": text})
        else:
            flat.append(m)
    if not images:
        return RenderedModelInput(chat_template_ids(tokenizer, flat, add_generation_prompt=add_generation_prompt))
    if processor is None or image_token_id is None:
        raise ValueError("messages contain images but no image processor / placeholder token id was given")
    text = tokenizer.apply_chat_template(flat, add_generation_prompt=add_generation_prompt, tokenize=False)
    ids: List[int] = []
    pvs, grids, spans = [], [], []
    pieces = text.split(marker)
    for i, piece in enumerate(pieces):
        ids.extend(tokenizer.encode(piece, add_special_tokens=False) if piece else [])
        if i < len(images):
            url = images[i]
            data = base64.b64decode(url.split(",", 1)[1]) if isinstance(url, str) and url.startswith("data:") else _chunk_bytes({"location": url})
            pv, grid, n = processor(data)
            spans.append((len(ids), n))
            ids.extend([image_token_id] * n)
            pvs.append(pv)
            grids.append(grid)
    return RenderedModelInput(ids, torch.cat(pvs, 0), torch.cat(grids, 0), spans)


def build_render_app(tokenizer, image_token_id: Optional[int] = None, processor: Optional[PatchImageProcessor] = None):
    """CPU-only FastAPI app: ``POST /v1/chat/completions/render`` -> token ids and base64 vision tensors."""
    from fastapi import FastAPI, HTTPException, Request

    app = FastAPI(title="skyrl_b200 render server")

    async def render(request: Request):
        body = await request.json()
        try:
            r = render_chat(body["messages"], tokenizer, image_token_id, processor, body.get("add_generation_prompt", True))
        except (KeyError, ValueError) as e:
            raise HTTPException(400, str(e))
        out: Dict[str, Any] = {"prompt_token_ids": r.prompt_ids, "placeholders": r.placeholder_ranges}
        if r.pixel_values is not None:
            pv = r.pixel_values.numpy().astype(np.float16)
            out["mm_kwargs"] = {"pixel_values": {"data": base64.b64encode(pv.tobytes()).decode(), "shape": list(pv.shape),
                                                 "dtype": "float16"},
                                "image_grid_thw": r.image_grid_thw.tolist()}
        return out

    render.__annotations__["request"] = Request
    app.post("/v1/chat/completions/render")(render)

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    return app


def decode_mm_kwargs(mm: Optional[Dict[str, Any]]):
    if not mm:
        return None, None
    p = mm["pixel_values"]
    pv = torch.from_numpy(np.frombuffer(base64.b64decode(p["data"]), dtype=np.dtype(p["dtype"])).reshape(p["shape"]).copy())
    return pv, torch.tensor(mm["image_grid_thw"], dtype=torch.long)
