"""Rollout router replay end to end on CPU: the engine returns the experts it routed every token to, the generator and
the trainer carry them to the worker, and the worker's forward passes run through those experts."""
import pytest
import torch

from skyrl_b200.config.config import SkyRLTrainConfig
from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams
from skyrl_b200.models import router_replay
from skyrl_b200.models.decoder import CausalLM, PRESETS
from skyrl_b200.parallel import dist as pdist
from skyrl_b200.train.trainer import PPOTrainer
from skyrl_b200.train.utils import validate_cfg
from skyrl_b200.utils.tokenizer import SyntheticTokenizer


def _engine(**kw):
    torch.manual_seed(0)
    m = CausalLM(PRESETS["tiny-moe"], dtype=torch.float32, device="cpu")
    cfg = EngineConfig(block_size=16, max_num_seqs=4, max_model_len=96, num_blocks=64, max_num_batched_tokens=256,
                       enforce_eager=True, sync_interval=3, **kw)
    return m, LLMEngine(m, cfg, eos_token_ids=[])


def _routing_of(model, tokens):
    ids = torch.tensor(tokens, dtype=torch.int32)
    pos = torch.arange(len(tokens), dtype=torch.int32)
    cu = torch.tensor([0, len(tokens)], dtype=torch.int32)
    with torch.no_grad(), router_replay.record_routing() as store:
        model(ids, pos, cu, len(tokens))
    return router_replay.stack_recorded(store)


def test_engine_returns_the_experts_of_every_fed_token():
    m, eng = _engine(return_routed_experts=True)
    a = m.args
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(4, 1000, (n,), generator=g).tolist() for n in (9, 20, 33)]
    sp = [SamplingParams(max_tokens=n, temperature=1.0, ignore_eos=True) for n in (1, 7, 12)]
    outs = eng.generate(prompts, sp)
    for p, o in zip(prompts, outs):
        r = o.routed_experts
        assert r is not None and r.dtype == torch.int16
        assert tuple(r.shape) == (len(p) + len(o.token_ids) - 1, a.num_layers, a.num_experts_per_tok)
        want = _routing_of(m, p + o.token_ids[:-1])
        # a full forward over the same tokens makes the same choices (sets of experts: top-k order may differ on ties)
        assert torch.equal(r.long().sort(-1).values, want.sort(-1).values)
    # the slots are reused: a second batch gets its own tables, not the previous occupants'
    outs2 = eng.generate(prompts[::-1], sp)
    for p, o in zip(prompts[::-1], outs2):
        want = _routing_of(m, p + o.token_ids[:-1])
        assert torch.equal(o.routed_experts.long().sort(-1).values, want.sort(-1).values)


def test_engine_without_the_flag_returns_none():
    _, eng = _engine()
    out = eng.generate([[5, 6, 7, 8]], SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True))[0]
    assert out.routed_experts is None and eng.out_experts is None


def test_pad_routes_lays_tables_under_left_padded_sequences():
    t0 = torch.arange(3 * 2 * 2).view(3, 2, 2)
    t1 = torch.arange(5 * 2 * 2).view(5, 2, 2) + 100
    out = router_replay.pad_routes([t0.numpy(), t1], [4, 5], 6)
    assert tuple(out.shape) == (2, 6, 2, 2) and out.dtype == torch.int16
    assert (out[0, :2] == router_replay.PAD).all() and torch.equal(out[0, 2:5].long(), t0)
    assert (out[0, 5] == router_replay.PAD).all()  # the token that was never fed keeps the model's own choice
    assert (out[1, 0] == router_replay.PAD).all() and torch.equal(out[1, 1:].long(), t1)
    with pytest.raises(ValueError):
        router_replay.pad_routes([t0, t1[:, :1]], [4, 5], 6)
    # a padded row leaves the layer's own routing in place
    idx = torch.tensor([[1, 2], [3, 4]])
    router_replay.set_replay(torch.tensor([[[5, 0]], [[-1, -1]]], dtype=torch.int16))
    try:
        got = router_replay.on_route(0, idx)
    finally:
        router_replay.set_replay(None)
    assert got.tolist() == [[5, 0], [3, 4]] and router_replay.on_route(0, idx) is None


def _cfg(tmp, extra=()):
    return SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model.path=tiny-moe", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4",
        "trainer.micro_train_batch_size_per_gpu=4", "trainer.micro_forward_batch_size_per_gpu=8",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=12",
        "generator.sampling_params.temperature=1.0", "trainer.max_prompt_length=32",
        "trainer.algorithm.use_kl_loss=false", "trainer.policy.optimizer_config.lr=1e-5",
        "environment.env_class=synthetic_even", "generator.batched=true", "trainer.bf16=false",
        "generator.inference_engine.max_num_seqs=16", "generator.inference_engine.enforce_eager=true", "trainer.seed=0",
        f"trainer.ckpt_path={tmp}/ckpt", f"trainer.export_path={tmp}/export", "trainer.resume_mode=none", *extra])


def _prompts(n=4, L=24, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for i in range(n):
        ids = torch.randint(4, 1024, (L,), generator=g).tolist()
        out.append({"prompt": [{"role": "user", "content": ids}], "prompt_token_ids": ids, "uid": f"p{i}"})
    return out


@pytest.mark.parametrize("ckpt", [False, True])
def test_trainer_replays_rollout_routing_in_the_policy_passes(tmp_path, ckpt):
    pdist.reset_env_for_tests()
    cfg = _cfg(tmp_path, ["generator.inference_engine.enable_return_routed_experts=true",
                          "trainer.policy.megatron_config.moe_enable_routing_replay=true",
                          f"trainer.gradient_checkpointing={'true' if ckpt else 'false'}"])
    validate_cfg(cfg)
    tr = PPOTrainer(cfg, tokenizer=SyntheticTokenizer(1024))
    tr.build_models()
    assert tr.engine.cfg.return_routed_experts

    seen = {"tables": 0, "forced_rows": 0}
    real = router_replay.set_replay

    def spy(ind):
        if ind is not None:
            seen["tables"] += 1
            seen["forced_rows"] += int((ind[:, 0, 0] >= 0).sum())
        return real(ind)

    router_replay.set_replay = spy
    try:
        m = tr.train_step(_prompts())
    finally:
        router_replay.set_replay = real
    assert seen["tables"] >= 2 and seen["forced_rows"] > 0  # the no-grad forward and the training pass both replayed
    assert not router_replay.active()                  # and nothing is left set for the next rollout
    assert m["policy/grad_norm"] > 0
    assert m["policy/rollout_train_logprobs_abs_diff_mean"] < 1e-4
    m2 = tr.train_step(_prompts(seed=1))
    assert m2["trainer/global_step"] == 2.0


def test_replay_without_returned_routes_is_rejected(tmp_path):
    cfg = _cfg(tmp_path, ["trainer.policy.megatron_config.moe_enable_routing_replay=true"])
    with pytest.raises(ValueError, match="enable_return_routed_experts"):
        validate_cfg(cfg)


def test_routed_experts_cross_the_http_wire():
    import asyncio

    from skyrl_b200.inference.local_client import LocalInferenceClient
    from skyrl_b200.inference.remote_client import RemoteInferenceClient
    from skyrl_b200.inference.server import ServerThread, build_app

    m, eng = _engine(return_routed_experts=True)
    srv = ServerThread(build_app(LocalInferenceClient([eng], SyntheticTokenizer(1024)))).start()
    try:
        rc = RemoteInferenceClient([srv.url], tokenizer=SyntheticTokenizer(1024))
        prompts = [[5, 6, 7, 8, 9], [11, 12, 13]]

        async def run():
            out = await rc.generate({"prompt_token_ids": prompts, "session_ids": ["a", "b"],
                                     "sampling_params": {"max_generate_length": 5, "temperature": 0.0}})
            await rc.teardown()
            return out

        out = asyncio.run(run())
        routes = out["rollout_expert_indices"]
        assert routes is not None and len(routes) == 2
        for p, ids, r in zip(prompts, out["response_ids"], routes):
            want = _routing_of(m, p + ids[:-1])
            assert torch.equal(torch.from_numpy(r.astype("int64")).sort(-1).values, want.sort(-1).values)
        padded = router_replay.pad_routes(routes, [len(p) + len(i) for p, i in zip(prompts, out["response_ids"])], 12)
        assert padded.shape[:2] == (2, 12) and (padded[0, -1] == router_replay.PAD).all()
    finally:
        srv.stop()


def test_persistent_replay_is_seen_by_other_threads():
    """On CUDA the backward pass (and with it the recomputation of checkpointed layers) runs in the autograd engine's
    thread: the table set for a micro-batch must reach it, while record / replay blocks stay private to their thread."""
    import threading

    idx = torch.tensor([[1, 2], [3, 4]])
    table = torch.tensor([[[5, 0]], [[7, 6]]], dtype=torch.int16)
    got = {}

    def other():
        got["persistent"] = router_replay.on_route(0, idx)
        got["active"] = router_replay.active()

    router_replay.set_replay(table)
    try:
        t = threading.Thread(target=other)
        t.start()
        t.join()
    finally:
        router_replay.set_replay(None)
    assert got["active"] and got["persistent"].tolist() == [[5, 0], [7, 6]]
    with router_replay.replay_routing(table):
        t = threading.Thread(target=other)
        t.start()
        t.join()
    assert not got["active"] and got["persistent"] is None


def test_freeze_moe_router_keeps_the_routers_and_trains_the_rest(tmp_path):
    pdist.reset_env_for_tests()
    cfg = _cfg(tmp_path, ["trainer.policy.megatron_config.freeze_moe_router=true",
                          "trainer.policy.optimizer_config.weight_decay=0.1", "trainer.policy.optimizer_config.lr=1e-3"])
    tr = PPOTrainer(cfg, tokenizer=SyntheticTokenizer(1024))
    tr.build_models()
    m = tr.policy.model
    routers = {n: m.p(n).detach().clone() for n in m.offsets if n.endswith(".router")}
    experts = m.p("layers.0.experts_wgu").detach().clone()
    assert routers
    out = tr.train_step(_prompts())
    assert out["policy/grad_norm"] > 0
    for n, w in routers.items():
        assert torch.equal(m.p(n), w), n                          # not even weight decay touched them
    assert not torch.equal(m.p("layers.0.experts_wgu"), experts)  # everything else trains
    lo, n_ = m.offsets["layers.0.router"]
    assert torch.equal(tr.policy.optimizer.master[lo : lo + n_], routers["layers.0.router"].float().reshape(-1))
