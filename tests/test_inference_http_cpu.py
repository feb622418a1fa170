"""HTTP data/control plane on CPU: real uvicorn servers around tiny engines, router affinity, client retries."""
import asyncio

import pytest
import torch

from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine
from skyrl_b200.inference.local_client import LocalInferenceClient
from skyrl_b200.inference.remote_client import RemoteInferenceClient
from skyrl_b200.inference.router import SessionRouter, build_router_app
from skyrl_b200.inference.server import ServerThread, build_app, clamp_logprobs
from skyrl_b200.models.decoder import CausalLM, ModelArgs
from skyrl_b200.utils.tokenizer import SyntheticTokenizer


def _server():
    args = ModelArgs(vocab_size=97, hidden_size=32, num_layers=1, num_heads=2, num_kv_heads=1, head_dim=16,
                     intermediate_size=48, tie_word_embeddings=True, max_position_embeddings=128)
    m = CausalLM(args, dtype=torch.float32, seed=1)
    eng = LLMEngine(m, EngineConfig(block_size=4, max_num_seqs=4, max_model_len=64, sync_interval=2, enforce_eager=True))
    client = LocalInferenceClient([eng], SyntheticTokenizer(97))
    return ServerThread(build_app(client)).start(), eng


def test_generate_over_http_matches_in_process_and_control_plane():
    srv, eng = _server()
    try:
        rc = RemoteInferenceClient([srv.url], tokenizer=SyntheticTokenizer(97))

        async def run():
            out = await rc.generate({"prompt_token_ids": [[5, 6, 7], [8, 9]], "session_ids": ["a", "b"],
                                     "sampling_params": {"max_generate_length": 6, "temperature": 0.0}})
            assert await rc.health()
            await rc.pause("keep")
            assert eng.paused
            await rc.resume()
            assert not eng.paused
            await rc.reset_prefix_cache()
            await rc.sleep(1)
            assert eng.asleep
            await rc.wake_up()
            assert not eng.asleep
            await rc.teardown()
            return out

        out = asyncio.run(run())
        ref = eng.generate([[5, 6, 7], [8, 9]], __import__("skyrl_b200.engine.llm_engine", fromlist=["SamplingParams"])
                           .SamplingParams(max_tokens=6, temperature=0.0))
        assert out["response_ids"] == [r.token_ids for r in ref]
        assert out["stop_reasons"] == ["length", "length"]
        assert all(len(l) == 6 for l in out["response_logprobs"])
    finally:
        srv.stop()


def test_router_is_session_affine_and_ejects_dead_servers():
    r = SessionRouter(["http://a", "http://b", "http://c"])
    picks = {sid: r.pick(sid) for sid in (f"s{i}" for i in range(50))}
    assert all(r.pick(sid) == u for sid, u in picks.items())
    assert len(set(picks.values())) == 3
    dead = picks["s0"]
    r.mark(dead, False)
    assert r.pick("s0") != dead and r.pick("s0") == r.pick("s0")
    moved = sum(1 for sid, u in picks.items() if u != dead and r.pick(sid) != u)
    assert moved == 0  # sessions on live servers keep their server


def test_router_proxies_to_servers():
    s1, _ = _server()
    s2, _ = _server()
    router = SessionRouter([s1.url, s2.url])
    rs = ServerThread(build_router_app(router)).start()
    try:
        rc = RemoteInferenceClient([s1.url, s2.url], router_url=rs.url)

        async def run():
            outs = await asyncio.gather(*[rc.generate({"prompt_token_ids": [[3, 4, 5]], "session_ids": [f"sess{i}"],
                                                       "sampling_params": {"max_generate_length": 3, "temperature": 0.0}})
                                          for i in range(8)])
            await rc.teardown()
            return outs

        outs = asyncio.run(run())
        assert len({tuple(o["response_ids"][0]) for o in outs}) == 1
        assert sum(router.stats.values()) >= 8 and all(v > 0 for v in router.stats.values())
    finally:
        rs.stop()
        s1.stop()
        s2.stop()


def test_logprob_clamping():
    assert clamp_logprobs([-1.0, None, float("nan"), float("-inf")]) == [-1.0, -9999.0, -9999.0, -9999.0]
