"""Generation engine on CPU: paged decode must reproduce full-recompute greedy decoding and log-probs."""
import torch

from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams
from skyrl_b200.models.decoder import CausalLM, ModelArgs


def _model():
    args = ModelArgs(vocab_size=97, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
                     intermediate_size=96, tie_word_embeddings=True, attention_bias=True, max_position_embeddings=256)
    return CausalLM(args, dtype=torch.float32, seed=11)


def _naive_greedy(m, prompt, n):
    toks = list(prompt)
    lps = []
    for _ in range(n):
        ids = torch.tensor(toks)
        pos = torch.arange(len(toks), dtype=torch.int32)
        cu = torch.tensor([0, len(toks)], dtype=torch.int32)
        with torch.no_grad():
            z = m.logits(m(ids, pos, cu, len(toks)))[-1].float()
        t = int(z.argmax())
        lps.append(float(torch.log_softmax(z, -1)[t]))
        toks.append(t)
    return toks[len(prompt):], lps


def test_greedy_matches_full_recompute_and_slots_recycle():
    m = _model()
    eng = LLMEngine(m, EngineConfig(block_size=4, max_num_seqs=3, max_model_len=64, max_num_batched_tokens=64,
                                    sync_interval=3, enforce_eager=True))
    prompts = [[5, 6, 7, 8, 9], [10, 11], [3] * 9, [20, 21, 22], [40]]
    outs = eng.generate(prompts, SamplingParams(max_tokens=7, temperature=0.0))
    for p, o in zip(prompts, outs):
        ref_t, ref_l = _naive_greedy(m, p, 7)
        assert o.token_ids == ref_t, (p, o.token_ids, ref_t)
        assert torch.allclose(torch.tensor(o.logprobs), torch.tensor(ref_l), atol=1e-4)
        assert o.finish_reason == "length"
    assert not eng.has_unfinished()
    assert eng.metrics()["kv_free_blocks"] == eng.num_blocks


def test_eos_stops_and_per_request_lengths():
    m = _model()
    ref_t, _ = _naive_greedy(m, [1, 2, 3], 6)
    eos = ref_t[3]
    eng = LLMEngine(m, EngineConfig(block_size=4, max_num_seqs=4, max_model_len=64, sync_interval=2, enforce_eager=True),
                    eos_token_ids=[eos])
    o1, o2 = eng.generate([[1, 2, 3], [1, 2, 3]], [SamplingParams(max_tokens=6, temperature=0.0),
                                                    SamplingParams(max_tokens=2, temperature=0.0)])
    first = ref_t.index(eos)
    assert o1.token_ids == ref_t[: first + 1] and o1.finish_reason == "stop"
    assert o2.token_ids == ref_t[: min(2, first + 1)]
    assert o2.finish_reason == ("stop" if first < 2 else "length")


def test_sampling_is_seeded_and_logprobs_are_consistent():
    m = _model()
    cfg = EngineConfig(block_size=8, max_num_seqs=8, max_model_len=64, enforce_eager=True, seed=3)
    a = LLMEngine(m, cfg).generate([[4, 5, 6]] * 4, SamplingParams(max_tokens=5, temperature=1.0))
    b = LLMEngine(m, cfg).generate([[4, 5, 6]] * 4, SamplingParams(max_tokens=5, temperature=1.0))
    assert [o.token_ids for o in a] == [o.token_ids for o in b]
    assert len({tuple(o.token_ids) for o in a}) > 1
    for o in a:  # the reported logprob is the model's logprob of the sampled token
        toks = [4, 5, 6] + o.token_ids
        ids = torch.tensor(toks)
        with torch.no_grad():
            z = m.logits(m(ids, torch.arange(len(toks), dtype=torch.int32), torch.tensor([0, len(toks)], dtype=torch.int32),
                           len(toks))).float()
        lp = torch.log_softmax(z, -1)
        want = [float(lp[2 + i, t]) for i, t in enumerate(o.token_ids)]
        assert torch.allclose(torch.tensor(o.logprobs), torch.tensor(want), atol=1e-4)


def test_pause_keep_resume_and_abort():
    m = _model()
    eng = LLMEngine(m, EngineConfig(block_size=4, max_num_seqs=2, max_model_len=64, sync_interval=2, enforce_eager=True))
    ref_t, _ = _naive_greedy(m, [9, 8, 7], 10)
    eng.add_request("a", [9, 8, 7], SamplingParams(max_tokens=10, temperature=0.0))
    eng.step()
    eng.pause("keep")
    assert eng.step() == [] and eng.has_unfinished()
    eng.resume()
    outs = []
    while eng.has_unfinished():
        outs += eng.step()
    assert outs[0].token_ids == ref_t
    eng.add_request("b", [9, 8, 7], SamplingParams(max_tokens=10, temperature=0.0))
    eng.step()
    part = eng.pause("abort")
    assert part[0].finish_reason == "abort" and part[0].token_ids == ref_t[: len(part[0].token_ids)]
    assert 0 < len(part[0].token_ids) < 10


def test_top_k_one_equals_greedy_and_requeue_after_kv_reset():
    m = _model()
    eng = LLMEngine(m, EngineConfig(block_size=4, max_num_seqs=2, max_model_len=64, sync_interval=2, enforce_eager=True))
    ref_t, _ = _naive_greedy(m, [2, 4, 6, 8], 8)
    (o,) = eng.generate([[2, 4, 6, 8]], SamplingParams(max_tokens=8, temperature=1.0, top_k=1))
    assert o.token_ids == ref_t
    eng.add_request("x", [2, 4, 6, 8], SamplingParams(max_tokens=8, temperature=0.0))
    eng.step()
    eng.reset_prefix_cache(reset_running_requests=True)  # weights changed mid-flight: KV dropped, tokens kept
    outs = []
    while eng.has_unfinished():
        outs += eng.step()
    assert outs[0].token_ids == ref_t and len(outs[0].logprobs) == 8


def test_prefix_cached_prefill_skips_cached_tokens_and_matches_full_prefill():
    """A second request that shares a prompt prefix reuses the cached key/value blocks: only the new tokens go through
    the projections, and the continuation is identical to a full prefill."""
    import torch

    from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams
    from skyrl_b200.models.decoder import PRESETS, CausalLM

    m = CausalLM(PRESETS["tiny-llama"], device="cpu", dtype=torch.float32, seed=3)
    g = torch.Generator().manual_seed(0)
    shared = torch.randint(4, 1024, (70,), generator=g).tolist()
    p1 = shared + torch.randint(4, 1024, (9,), generator=g).tolist()
    p2 = shared + torch.randint(4, 1024, (13,), generator=g).tolist()
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    outs = {}
    for caching in (False, True):
        eng = LLMEngine(m, EngineConfig(block_size=16, max_num_seqs=4, max_model_len=128, enforce_eager=True, num_blocks=64,
                                        enable_prefix_caching=caching))
        a = eng.generate([p1], sp)[0]
        b = eng.generate([p2], sp)[0]
        c = eng.generate([p1], sp)[0]
        outs[caching] = (a.token_ids, b.token_ids, c.token_ids, eng.stats.get("prefix_cached_tokens", 0),
                         eng.stats["prefill_tokens"])
    assert outs[True][:3] == outs[False][:3]
    assert outs[False][3] == 0
    assert outs[True][3] >= 64 + 64  # p2 reuses 4 shared blocks, the repeat of p1 reuses 4 (79 tokens -> 64 cached)
    assert outs[True][4] == outs[False][4] - outs[True][3]


def test_slot_compaction_keeps_outputs_and_shrinks_the_decode_batch():
    """Sequences of very different lengths: stragglers are moved to low slots, results are unchanged."""
    import torch

    from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams
    from skyrl_b200.models.decoder import PRESETS, CausalLM

    m = CausalLM(PRESETS["tiny-llama"], device="cpu", dtype=torch.float32, seed=1)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(4, 1024, (10 + i,), generator=g).tolist() for i in range(24)]
    lens = [3] * 20 + [40, 44, 48, 52]  # the long ones sit in the highest slots
    params = [SamplingParams(max_tokens=n, temperature=0.0, ignore_eos=True) for n in lens]
    cfgs = dict(block_size=16, max_model_len=128, enforce_eager=True, num_blocks=256, sync_interval=4)
    eng = LLMEngine(m, EngineConfig(max_num_seqs=32, graph_batch_sizes=(8, 16, 32), **cfgs))
    out = eng.generate(prompts, params)
    assert eng.stats.get("slot_compactions", 0) >= 1
    assert [len(o.token_ids) for o in out] == lens
    ref_eng = LLMEngine(m, EngineConfig(max_num_seqs=32, graph_batch_sizes=(32,), **cfgs))  # one bucket: never compacts
    ref = ref_eng.generate(prompts, params)
    assert ref_eng.stats.get("slot_compactions", 0) == 0
    for a, b in zip(out, ref):
        assert a.token_ids == b.token_ids
    assert eng.metrics()["kv_free_blocks"] == 256 and sorted(eng._free_slots) == list(range(32))


def test_same_prompt_sampled_n_times_is_prefilled_once():
    """GRPO sends every prompt n times in one call.  With the prefix cache on, the scheduler admits one copy, lets it
    publish its blocks, and the other copies share them: only their last block is computed again."""
    m = _model()
    torch.manual_seed(3)
    p1, p2 = torch.randint(4, 97, (40,)).tolist(), torch.randint(4, 97, (37,)).tolist()
    prompts = [p1] * 4 + [p2] * 3
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    res = {}
    for caching in (False, True):
        eng = LLMEngine(m, EngineConfig(block_size=8, max_num_seqs=8, max_model_len=64, num_blocks=128,
                                        enable_prefix_caching=caching))
        outs = eng.generate(prompts, sp)
        res[caching] = ([o.token_ids for o in outs], eng.stats.get("prefix_cached_tokens", 0),
                        eng.stats.get("prefill_tokens", None))
        assert eng.metrics()["kv_free_blocks"] == 128
    assert res[True][0] == res[False][0]
    assert all(t == res[True][0][0] for t in res[True][0][:4])  # greedy copies agree
    # p1: 39 matchable tokens -> 4 full blocks (32 tokens) shared by 3 copies; p2: 36 -> 4 blocks shared by 2 copies
    assert res[False][1] == 0 and res[True][1] == 3 * 32 + 2 * 32


class _OracleHead(torch.nn.Module):
    """A draft head that cannot be trained but is always right or always wrong: it ignores the hidden state and its
    output, through the LM head, selects a fixed token."""

    def __init__(self, model, token):
        super().__init__()
        w = model.lm_head_weight().float()
        self.vec = w[token] / w[token].norm() ** 2 * 1e4  # the LM head scores `token` far above everything else

    def forward(self, h):
        return self.vec.to(h.dtype).expand(h.shape[0], -1)


def _spec_engine(head_factory, **kw):
    from skyrl_b200.algorithms.mtp import DraftHead  # noqa: F401
    from skyrl_b200.models.decoder import PRESETS

    torch.manual_seed(0)
    m = CausalLM(PRESETS["tiny-llama"], dtype=torch.float32, device="cpu", seed=3)
    eng = LLMEngine(m, EngineConfig(block_size=16, max_num_seqs=4, max_model_len=128, num_blocks=64, enforce_eager=True,
                                    sync_interval=3, **kw), eos_token_ids=[])
    if head_factory is not None:
        eng.set_draft_head(head_factory(m))
    return m, eng


def test_speculative_decoding_keeps_the_greedy_output_and_counts_acceptances():
    from skyrl_b200.algorithms.mtp import DraftHead

    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(4, 1000, (n,), generator=g).tolist() for n in (7, 19, 33)]
    sp = [SamplingParams(max_tokens=n, temperature=0.0, ignore_eos=True) for n in (1, 6, 11)]
    _, plain = _spec_engine(None)
    want = plain.generate(prompts, sp)

    # an untrained head (identity: it guesses that the next token repeats) must not change a single token or log-prob
    m, eng = _spec_engine(lambda m: DraftHead(m.args.hidden_size), num_speculative_tokens=1)
    got = eng.generate(prompts, sp)
    for a, b in zip(want, got):
        assert a.token_ids == b.token_ids and a.finish_reason == b.finish_reason
        assert torch.allclose(torch.tensor(a.logprobs), torch.tensor(b.logprobs), atol=1e-5)
    mt = eng.metrics()
    assert mt["spec_drafted"] > 0 and 0.0 <= mt["spec_acceptance_rate"] <= 1.0

    # a head that always guesses a token the model never produces: nothing is accepted, the output is unchanged
    never = max(set(range(4, 1000)) - {t for o in want for t in o.token_ids})
    m, eng = _spec_engine(lambda m: _OracleHead(m, never), num_speculative_tokens=1)
    got = eng.generate(prompts, sp)
    assert [o.token_ids for o in got] == [o.token_ids for o in want] and eng.metrics()["spec_accepted"] == 0

    # the same engine, second batch: slots are reused and still match
    got2 = eng.generate(prompts[::-1], sp[::-1])
    assert [o.token_ids for o in got2] == [o.token_ids for o in want][::-1]


def test_speculative_decoding_accepts_correct_guesses_and_takes_two_tokens_per_step():
    """A model whose final norm is zeroed gives uniform logits, so greedy decoding always emits token 0; a head that
    always guesses 0 is always right: every step yields two tokens, limits are respected exactly, log-probs match."""
    import math

    import pytest

    def zeroed(m):
        m.p("final_norm").data.zero_()
        return m

    m0, plain = _spec_engine(None)
    zeroed(m0)
    prompts = [[5, 6, 7, 8], [9, 10, 11], [12, 13]]
    sp = [SamplingParams(max_tokens=n, temperature=0.0, ignore_eos=True) for n in (9, 4, 1)]
    want = plain.generate(prompts, sp)
    assert all(set(o.token_ids) == {0} for o in want)
    m, eng = _spec_engine(lambda m: _OracleHead(zeroed(m), 0), num_speculative_tokens=1)
    got = eng.generate(prompts, sp)
    for a, b in zip(want, got):
        assert a.token_ids == b.token_ids and a.finish_reason == b.finish_reason == "length"
        assert b.logprobs == pytest.approx([-math.log(m.args.vocab_size)] * len(b.token_ids), abs=1e-4)
    mt = eng.metrics()
    assert mt["spec_drafted"] > 0 and mt["spec_accepted"] == mt["spec_drafted"]
    # 9 tokens: 1 from prefill, then 4 steps of two; plain decoding needs 8 steps
    assert eng.stats["decode_steps"] < plain.stats["decode_steps"]
    # sampled (temperature 1) outputs stay inside the vocabulary and respect the limits too
    out = eng.generate(prompts, [SamplingParams(max_tokens=n, temperature=1.0, ignore_eos=True) for n in (9, 4, 1)])
    assert [len(o.token_ids) for o in out] == [9, 4, 1]


def test_unsupported_sampling_knobs_are_rejected_not_ignored():
    import pytest

    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.train.utils import validate_cfg

    assert SamplingParams.from_dict({"repetition_penalty": 1.0, "max_generate_length": 5}).max_tokens == 5
    with pytest.raises(ValueError, match="repetition_penalty"):
        SamplingParams.from_dict({"repetition_penalty": 1.2})
    with pytest.raises(ValueError, match="repetition_penalty"):
        validate_cfg(SkyRLTrainConfig.from_cli_overrides(["trainer.policy.model.path=tiny-llama",
                                                          "generator.sampling_params.repetition_penalty=1.1"]))
