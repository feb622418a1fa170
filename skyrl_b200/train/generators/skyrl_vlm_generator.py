"""Multi-image, multi-turn generator: like the text generator, but prompts and observations may carry images, which
are rendered into placeholder tokens plus ``pixel_values`` / ``image_grid_thw`` rows that travel with the trajectory
(reference: skyrl/train/generators/skyrl_vlm_generator.py, 236 lines: pixel tensors accumulated per turn, handed to the
trainer as ``TensorList`` columns)."""

from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from ...inference.render import PatchImageProcessor, render_chat
from ...train.batch import TensorList
from .base import GeneratorInput, GeneratorOutput
from .skyrl_gym_generator import SkyRLGymGenerator


class SkyRLVLMGenerator(SkyRLGymGenerator):
    def __init__(self, generator_cfg, skyrl_gym_cfg, inference_engine_client, tokenizer, image_token_id: int,
                 processor: Optional[PatchImageProcessor] = None, model_name: str = "policy"):
        super().__init__(generator_cfg, skyrl_gym_cfg, inference_engine_client, tokenizer, model_name)
        self.image_token_id = image_token_id
        self.processor = processor or PatchImageProcessor()
        if self.batched:
            raise ValueError("the multimodal generator runs the per-trajectory loop; set generator.batched=false")

    def _render(self, messages: List[Dict[str, Any]], add_generation_prompt: bool = True):
        return render_chat(messages, self.tokenizer, self.image_token_id, self.processor, add_generation_prompt)

    @staticmethod
    def _has_images(messages: List[Dict[str, Any]]) -> bool:
        return any(isinstance(m.get("content"), list) and any(p.get("type") in ("image", "image_url") for p in m["content"])
                   for m in messages)

    async def generate(self, input_batch: GeneratorInput) -> GeneratorOutput:
        """Prompts are pre-rendered (so image placeholders are in the token stream), the text loop runs on the
        rendered ids, and the vision tensors of each trajectory are attached to the output."""
        prompts = input_batch["prompts"]
        pixel_rows: List[Optional[torch.Tensor]] = []
        grid_rows: List[Optional[torch.Tensor]] = []
        rendered_ids: List[List[int]] = []
        for p in prompts:
            r = self._render(p)
            rendered_ids.append(r.prompt_ids)
            pixel_rows.append(r.pixel_values)
            grid_rows.append(r.image_grid_thw)
        inp = dict(input_batch)
        inp["prompt_token_ids"] = rendered_ids
        out = await super().generate(inp)  # type: ignore[arg-type]
        n_rows, n_prompts = len(out["response_ids"]), len(prompts)
        rep = max(1, n_rows // max(1, n_prompts))
        ref = next((x for x in pixel_rows if x is not None), None)
        if ref is not None:
            empty_pv = torch.empty((0, ref.shape[1]), dtype=ref.dtype)
            empty_g = torch.empty((0, 3), dtype=torch.long)
            out["pixel_values"] = TensorList([(pixel_rows[i // rep] if pixel_rows[i // rep] is not None else empty_pv)
                                              for i in range(n_rows)])
            out["image_grid_thw"] = TensorList([(grid_rows[i // rep] if grid_rows[i // rep] is not None else empty_g)
                                                for i in range(n_rows)])
        return out
