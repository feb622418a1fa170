"""Multimodal rendering and the VLM generator (text-only engine; images travel as placeholder tokens + tensors)."""
import asyncio
import base64
import io

import numpy as np
import torch

from skyrl_b200.inference.render import (PatchImageProcessor, build_render_app, decode_mm_kwargs, render_chat,
                                         render_model_input)
from skyrl_b200.utils.tokenizer import SyntheticTokenizer


def _img_bytes(h=30, w=45):
    arr = np.random.default_rng(0).random((h, w, 3)).astype(np.float32)
    try:
        from PIL import Image

        buf = io.BytesIO()
        Image.fromarray((arr * 255).astype(np.uint8)).save(buf, format="PNG")
        return buf.getvalue()
    except ImportError:
        buf = io.BytesIO()
        np.save(buf, arr)
        return buf.getvalue()


def test_patch_processor_and_tinker_chunks():
    proc = PatchImageProcessor(patch=14, merge=2)
    pv, grid, n = proc(_img_bytes())
    gh, gw = grid[0, 1].item(), grid[0, 2].item()
    assert pv.shape == (gh * gw, 14 * 14 * 3) and n == (gh // 2) * (gw // 2) and gh % 2 == 0 and gw % 2 == 0
    mi = {"chunks": [{"tokens": [5, 6]}, {"type": "image", "data": base64.b64encode(_img_bytes()).decode(), "format": "png",
                                          "expected_tokens": n}, {"tokens": [7]}]}
    r = render_model_input([mi], image_token_id=99, processor=proc)[0]
    assert r.prompt_ids[:2] == [5, 6] and r.prompt_ids[-1] == 7 and r.prompt_ids.count(99) == n
    assert r.placeholder_ranges == [(2, n)] and r.pixel_values.shape[0] == gh * gw
    try:
        render_model_input([dict(chunks=[dict(mi["chunks"][1], expected_tokens=n + 1)])], 99, proc)
        raise AssertionError("expected a mismatch error")
    except ValueError:
        pass
    assert render_model_input([{"chunks": [{"tokens": [1, 2, 3]}]}])[0].prompt_ids == [1, 2, 3]


def test_render_chat_and_server():
    from fastapi.testclient import TestClient

    tok = SyntheticTokenizer(2048)
    proc = PatchImageProcessor()
    url = "data:image/png;base64," + base64.b64encode(_img_bytes()).decode()
    msgs = [{"role": "user", "content": [{"type": "text", "text": "what is this "}, {"type": "image_url", "image_url": {"url": url}},
                                         {"type": "text", "text": " ?"}]}]
    r = render_chat(msgs, tok, image_token_id=77, processor=proc)
    n = r.placeholder_ranges[0][1]
    assert r.prompt_ids[r.placeholder_ranges[0][0]] == 77 and r.prompt_ids.count(77) == n
    with TestClient(build_render_app(tok, 77, proc)) as c:
        out = c.post("/v1/chat/completions/render", json={"messages": msgs}).json()
        assert out["prompt_token_ids"] == r.prompt_ids
        pv, grid = decode_mm_kwargs(out["mm_kwargs"])
        assert pv.shape == r.pixel_values.shape and torch.equal(grid, r.image_grid_thw)
        assert c.post("/v1/chat/completions/render", json={}).status_code == 400


def test_vlm_generator_attaches_vision_rows():
    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_b200.inference.local_client import LocalInferenceClient
    from skyrl_b200.models.decoder import PRESETS, CausalLM
    from skyrl_b200.train.generators.skyrl_vlm_generator import SkyRLVLMGenerator
    from skyrl_b200.train.generators.utils import prepare_generator_input

    cfg = SkyRLTrainConfig.from_cli_overrides(["generator.batched=false", "generator.sampling_params.max_generate_length=6",
                                               "generator.n_samples_per_prompt=2", "trainer.max_prompt_length=512",
                                               "generator.max_input_length=600"])
    tok = SyntheticTokenizer(2048)
    m = CausalLM(PRESETS["tiny-qwen2-d128"], device="cpu", dtype=torch.float32, seed=0)
    eng = LLMEngine(m, EngineConfig(block_size=16, max_num_seqs=8, max_model_len=700, enforce_eager=True, num_blocks=256),
                    eos_token_ids=[tok.eos_token_id])
    gen = SkyRLVLMGenerator(cfg.generator, cfg.environment.skyrl_gym, LocalInferenceClient([eng], tok), tok, image_token_id=77)
    url = "data:image/png;base64," + base64.b64encode(_img_bytes()).decode()
    prompts = [{"prompt": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": url}}, {"type": "text", "text": "hi"}]}],
                "uid": "a", "env_extras": {"p": 0.5, "seed": 1}},
               {"prompt": [{"role": "user", "content": "plain text"}], "uid": "b", "env_extras": {"p": 0.5, "seed": 2}}]
    gi, uids = prepare_generator_input(prompts, 2, None, "synthetic_bernoulli", "train", 0)
    out = asyncio.run(gen.generate(gi))
    assert len(out["response_ids"]) == 4 and len(out["pixel_values"]) == 4
    assert out["pixel_values"][0].shape[0] > 0 and out["pixel_values"][3].shape[0] == 0  # text-only rows get empty tensors
    assert out["prompt_token_ids"][0].count(77) > 0 and out["prompt_token_ids"][2].count(77) == 0
