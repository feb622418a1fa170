"""Speculative decoding next to the engine's other machinery: prefix sharing, slot compaction, pausing and requeueing."""
import torch

from skyrl_b200.algorithms.mtp import DraftHead
from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams
from skyrl_b200.models.decoder import PRESETS, CausalLM


def _engines(**kw):
    m = CausalLM(PRESETS["tiny-llama"], dtype=torch.float32, device="cpu", seed=11)
    base = dict(block_size=8, max_num_seqs=8, max_model_len=160, num_blocks=256, enforce_eager=True, sync_interval=2)
    base.update(kw)
    plain = LLMEngine(m, EngineConfig(**base), eos_token_ids=[])
    spec = LLMEngine(m, EngineConfig(num_speculative_tokens=1, **base), eos_token_ids=[])
    torch.manual_seed(0)
    head = DraftHead(m.args.hidden_size)
    with torch.no_grad():  # a head that is neither the identity nor trained: guesses are sometimes right
        head.down.weight.normal_(0, 0.05)
    spec.set_draft_head(head)
    return plain, spec


def _same(a, b):
    assert [o.token_ids for o in a] == [o.token_ids for o in b]
    for x, y in zip(a, b):
        assert torch.allclose(torch.tensor(x.logprobs), torch.tensor(y.logprobs), atol=1e-5)
        assert x.finish_reason == y.finish_reason


def test_greedy_outputs_match_with_shared_prefixes_and_more_requests_than_slots():
    plain, spec = _engines(enable_prefix_caching=True, max_num_seqs=4)
    g = torch.Generator().manual_seed(2)
    stem = torch.randint(4, 1000, (24,), generator=g).tolist()
    prompts = [stem + torch.randint(4, 1000, (k,), generator=g).tolist() for k in (1, 5, 9, 2, 7, 3, 8, 4, 6, 10)]
    prompts += [prompts[0], prompts[0]]  # the same prompt sampled again: its blocks are shared
    sp = [SamplingParams(max_tokens=3 + (i % 7), temperature=0.0, ignore_eos=True) for i in range(len(prompts))]
    want, got = plain.generate(prompts, sp), spec.generate(prompts, sp)
    _same(want, got)
    assert spec.metrics()["spec_drafted"] > 0
    # eos handling: treat the most common generated token as the end-of-sequence token
    from collections import Counter

    eos = Counter(t for o in want for t in o.token_ids).most_common(1)[0][0]
    plain2, spec2 = _engines()
    plain2.eos_token_ids, spec2.eos_token_ids = [eos], [eos]
    for e in (plain2, spec2):
        e.eos_dev = torch.tensor([eos], dtype=torch.int32)
    sp2 = [SamplingParams(max_tokens=12, temperature=0.0) for _ in prompts]
    w2, g2 = plain2.generate(prompts, sp2), spec2.generate(prompts, sp2)
    _same(w2, g2)
    assert any(o.finish_reason == "stop" for o in w2)


def test_requeue_in_the_middle_of_generation_keeps_the_output():
    plain, spec = _engines()
    prompts = [[5, 6, 7, 8, 9], [10, 11, 12]]
    sp = SamplingParams(max_tokens=14, temperature=0.0, ignore_eos=True)
    want = plain.generate(prompts, sp)
    for i, p in enumerate(prompts):
        spec.add_request(f"r{i}", p, sp)
    got = {}
    for o in spec.step():
        got[o.request_id] = o
    spec.sleep(1)       # running requests go back to the queue with what they have generated so far
    spec.wake_up()
    while len(got) < 2:
        for o in spec.step():
            got[o.request_id] = o
    _same(want, [got["r0"], got["r1"]])
