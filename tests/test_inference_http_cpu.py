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


@pytest.mark.parametrize("transport", ["delta", "path"])
def test_trainer_syncs_weights_to_stand_alone_server(tmp_path, transport):
    """Disaggregated set-up in one test process: the rollout engine lives behind HTTP with its *own* weights; after an
    RL step the server has loaded the trainer's new weights (delta replay or safetensors export) and kept serving."""
    import torch

    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_b200.inference.local_client import LocalInferenceClient
    from skyrl_b200.inference.remote_client import RemoteInferenceClient
    from skyrl_b200.inference.server import ServerThread, build_app
    from skyrl_b200.models.decoder import PRESETS, CausalLM
    from skyrl_b200.parallel.dist import get_env
    from skyrl_b200.train.trainer import PPOTrainer
    from skyrl_b200.utils.tokenizer import SyntheticTokenizer
    from skyrl_b200.weight_sync.remote import make_weight_loader

    tok = SyntheticTokenizer(2048)
    server_model = CausalLM(PRESETS["tiny-qwen2-d128"], device="cpu", dtype=torch.float32, seed=123)  # not the trainer's
    eng = LLMEngine(server_model, EngineConfig(block_size=16, max_num_seqs=8, max_model_len=64, enforce_eager=True, num_blocks=64),
                    eos_token_ids=[tok.eos_token_id])
    local = LocalInferenceClient([eng], tok)
    srv = ServerThread(build_app(local, weight_loader=make_weight_loader(server_model, eng, local_dir=str(tmp_path / "local")))).start()
    try:
        cfg = SkyRLTrainConfig.from_cli_overrides([
            "trainer.policy.model.path=tiny-qwen2-d128", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
            "generator.n_samples_per_prompt=4", "trainer.max_prompt_length=16", "generator.sampling_params.max_generate_length=8",
            "environment.env_class=synthetic_bernoulli", "trainer.bf16=false", "trainer.policy.optimizer_config.lr=1e-3",
            "trainer.policy.optimizer_config.num_warmup_steps=0", "trainer.resume_mode=none", "trainer.algorithm.use_kl_loss=false",
            "trainer.placement.colocate_all=false", "generator.inference_engine.external_server_urls=['" + srv.url + "']",
            f"generator.inference_engine.weight_sync_backend={'delta' if transport == 'delta' else 'broadcast'}",
            f"generator.inference_engine.delta_weight_sync.sync_dir={tmp_path}/sync", "trainer.logger=console"])
        client = RemoteInferenceClient([srv.url], tokenizer=tok)
        tr = PPOTrainer(cfg, tokenizer=tok, inference_engine_client=client, env=get_env())
        tr.build_models()
        assert tr.engine is None
        prompts = [{"prompt": [{"role": "user", "content": f"q{i}"}], "uid": f"u{i}", "env_extras": {"p": 0.5, "seed": i}}
                   for i in range(2)]
        for _ in range(2):  # first sync publishes the base, the second one a delta
            tr.train_step(prompts)
            assert torch.equal(server_model.flat_params[: tr.policy.model.flat_numel], tr.policy.model.flat_params[: tr.policy.model.flat_numel])
        assert eng.weight_version >= 2 and not eng.paused
    finally:
        srv.stop()


def test_sample_tokenize_render_and_context_manager_over_http():
    srv, eng = _server()
    try:
        async def run():
            async with RemoteInferenceClient([srv.url], tokenizer=SyntheticTokenizer(97)) as rc:
                res = await rc.sample({"json": {"prompt": {"chunks": [{"tokens": [5, 6]}, {"tokens": [7]}]}, "num_samples": 3,
                                                "sampling_params": {"max_tokens": 4, "temperature": 0.0},
                                                "include_prompt_logprobs": True, "topk_prompt_logprobs": 2},
                                       "session_id": "s"})
                tok = await rc.tokenize({"json": {"prompt": "5 6 7"}})
                detok = await rc.detokenize({"json": {"tokens": [5, 6, 7]}})
                rendered = await rc.render_chat_completion({"json": {"messages": [{"role": "user", "content": "5 6"}]}})
                await rc.pause_generation()
                paused = eng.paused
                await rc.resume_generation()
                return res, tok, detok, rendered, paused, eng.paused

        res, tok, detok, rendered, paused, resumed = asyncio.run(run())
        assert res["type"] == "sample" and len(res["sequences"]) == 3 and res["topk_prompt_logprobs"] is None
        from skyrl_b200.engine.llm_engine import SamplingParams

        ref = eng.generate([[5, 6, 7]], SamplingParams(max_tokens=4, temperature=0.0, prompt_logprobs=True))[0]
        for s in res["sequences"]:
            assert s["tokens"] == ref.token_ids and s["stop_reason"] == "length" and len(s["logprobs"]) == 4
        # the first prompt token has no predecessor, the others carry the model's log-prob of the token itself
        plp = res["prompt_logprobs"]
        assert plp[0] is None and plp[1:] == pytest.approx(ref.prompt_logprobs[1:], abs=1e-5)
        assert tok == {"tokens": [5, 6, 7], "count": 3} and detok["prompt"] == "5 6 7"
        assert rendered["token_ids"] == [2, 5, 6, 1, 3] and rendered["count"] == 5
        assert paused and not resumed
        # vLLM-style "0 alternatives" still asks for the prompt tokens' own log-probs
        assert SamplingParams.from_dict({"prompt_logprobs": 0}).prompt_logprobs is True
        assert SamplingParams.from_dict({"prompt_logprobs": None}).prompt_logprobs is False
    finally:
        srv.stop()


def test_sticky_least_loaded_balances_new_sessions_and_frees_finished_ones():
    r = SessionRouter(["http://a", "http://b", "http://c"], policy="sticky_least_loaded")
    first = [r.pick(f"s{i}") for i in range(3)]
    assert sorted(first) == ["http://a", "http://b", "http://c"]        # one new session per replica
    assert [r.pick(f"s{i}") for i in range(3)] == first and r.open_sessions == [1, 1, 1]   # sticky, not recounted
    home0 = r.pick("s0")
    assert r.finish("s0") == home0 and r.finish("s0") is None
    assert r.pick("s3") == home0                                        # the freed replica is the least loaded one
    assert r.pick("s4") in ("http://a", "http://b", "http://c") and sum(r.open_sessions) == 4
    # a session whose server disappears moves to the least loaded live one and stays there
    victim = r.pick("s1")
    r.mark(victim, False)
    moved = r.pick("s1")
    assert moved != victim and r.pick("s1") == moved and r.open_sessions[r.urls.index(victim)] >= 0
    assert r.pick(None) != victim                                      # session-less requests avoid it too
    with pytest.raises(ValueError):
        SessionRouter(["http://a"], policy="nope")


def test_router_app_releases_sessions_on_finish():
    srv1, eng1 = _server()
    srv2, eng2 = _server()
    router = SessionRouter([srv1.url, srv2.url], policy="sticky_least_loaded")
    rt = ServerThread(build_router_app(router)).start()
    try:
        rc = RemoteInferenceClient([srv1.url, srv2.url], router_url=rt.url, tokenizer=SyntheticTokenizer(97))

        async def run():
            sp = {"max_generate_length": 3, "temperature": 0.0}
            await rc.generate({"prompt_token_ids": [[5, 6], [7, 8]], "session_ids": ["x", "y"], "sampling_params": sp})
            open_before = list(router.open_sessions)
            await rc.generate({"prompt_token_ids": [[5, 6, 9]], "session_ids": ["x"], "sampling_params": sp})
            still = list(router.open_sessions)
            await rc.finish_session("x")
            await rc.finish_session("y")
            await rc.teardown()
            return open_before, still

        open_before, still = asyncio.run(run())
        assert open_before == [1, 1] and still == [1, 1] and router.open_sessions == [0, 0]
        assert eng1.stats["prefill_calls"] >= 1 and eng2.stats["prefill_calls"] >= 1
    finally:
        rt.stop()
        srv1.stop()
        srv2.stop()
