"""Attention sinks (one learned logit per query head that joins every softmax and carries no value): the PyTorch
formulation against a hand-written softmax, gradients of the autograd function, and a tiny model that trains and
generates with them."""
import math

import torch

from skyrl_b200.models.decoder import PRESETS, CausalLM
from skyrl_b200.ops import attention as A


def _manual(qkv, cu, nq, nkv, D, scale, sinks):
    T = qkv.shape[0]
    q, k, v = A._split(qkv.double(), nq, nkv, D)
    out = torch.zeros(T, nq, D, dtype=torch.float64)
    for b in range(len(cu) - 1):
        for t in range(cu[b], cu[b + 1]):
            for h in range(nq):
                g = h // (nq // nkv)
                sc = (k[cu[b]: t + 1, g] @ q[t, h]) * scale
                w = torch.softmax(torch.cat([sc, sinks[h].double().view(1)]), 0)[:-1]
                out[t, h] = w @ v[cu[b]: t + 1, g]
    return out.reshape(T, nq * D)


def test_reference_matches_manual_softmax_with_sink_column():
    torch.manual_seed(0)
    nq, nkv, D = 4, 2, 16
    cu = [0, 5, 12]
    qkv = torch.randn(12, (nq + 2 * nkv) * D)
    sinks = torch.tensor([0.5, -1.0, 2.0, 0.0])
    out, lse = A.attn_varlen_ref(qkv, torch.tensor(cu, dtype=torch.int32), nq, nkv, D, 0.25, sinks)
    assert (out.double() - _manual(qkv, cu, nq, nkv, D, 0.25, sinks)).abs().max() < 1e-5
    # without sinks the rows sum to one; with a sink the mass exp(sink - lse) is missing
    plain, lse0 = A.attn_varlen_ref(qkv, torch.tensor(cu, dtype=torch.int32), nq, nkv, D, 0.25)
    assert torch.allclose(lse, torch.logaddexp(lse0, sinks.view(nq, 1)), atol=1e-5)
    assert torch.allclose(out.view(12, nq, D), plain.view(12, nq, D) * torch.exp(lse0 - lse).t().unsqueeze(-1), atol=1e-5)


def test_autograd_function_gradients_match_reference_autograd():
    torch.manual_seed(1)
    nq, nkv, D = 2, 1, 16
    cu = torch.tensor([0, 7, 10], dtype=torch.int32)
    qkv = torch.randn(10, (nq + 2 * nkv) * D, requires_grad=True)
    sinks = torch.tensor([0.3, -0.7], requires_grad=True)
    dy = torch.randn(10, nq * D)
    out = A.attn_varlen(qkv, cu, nq, nkv, D, sinks=sinks)
    out.backward(dy)
    q2 = qkv.detach().clone().requires_grad_()
    s2 = sinks.detach().clone().requires_grad_()
    ref, _ = A.attn_varlen_ref(q2, cu, nq, nkv, D, 1 / math.sqrt(D), s2)
    ref.backward(dy)
    assert torch.allclose(out, ref, atol=1e-5)
    assert torch.allclose(qkv.grad, q2.grad, atol=1e-5)
    assert torch.allclose(sinks.grad, s2.grad, atol=1e-5) and sinks.grad.abs().max() > 1e-3


def test_tiny_model_with_sinks_trains_and_generates():
    from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams
    from skyrl_b200.models import hf_io

    a = PRESETS["tiny-sinks"]
    m = CausalLM(a, device="cpu", dtype=torch.float32, seed=3)
    for i in range(a.num_layers):
        m.p(f"layers.{i}.sinks").data.copy_(torch.tensor([1.5, -0.5]))
    grad = torch.zeros_like(m.flat_params, dtype=torch.float32)
    m.attach_main_grad(grad)
    ids = torch.randint(4, a.vocab_size, (24,), dtype=torch.int32)
    pos = torch.cat([torch.arange(10), torch.arange(14)]).int()
    cu = torch.tensor([0, 10, 24], dtype=torch.int32)
    h = m(ids, pos, cu, 14)
    lp, _ = m.token_logprobs(h, torch.roll(ids, -1))
    (-lp.mean()).backward()
    for i in range(a.num_layers):
        assert m.p(f"layers.{i}.sinks").main_grad.abs().max() > 0

    # a sink changes the output, and the engine's paged decode agrees with the packed forward
    plain = CausalLM(a, device="cpu", dtype=torch.float32, seed=3)
    assert (plain(ids, pos, cu, 14) - h.detach()).abs().max() > 1e-4
    eng = LLMEngine(m, EngineConfig(block_size=16, max_num_seqs=4, max_model_len=64, num_blocks=32))
    prompt = ids[:10].tolist()
    out = eng.generate([prompt], SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True, logprobs=1))[0]
    toks = torch.tensor(prompt + out.token_ids, dtype=torch.int32)
    with torch.no_grad():
        hh = m(toks, torch.arange(len(toks), dtype=torch.int32), torch.tensor([0, len(toks)], dtype=torch.int32), len(toks))
        want, _ = m.token_logprobs(hh[len(prompt) - 1: -1], toks[len(prompt):])
    assert (want - torch.tensor(out.logprobs)).abs().max() < 1e-4

    # HF-named state dict carries the sinks and loads back
    sd = {k: v.clone() for k, v in hf_io.to_hf_state_dict(m).items()}
    assert "model.layers.0.self_attn.sinks" in sd
    m2 = CausalLM(a, device="cpu", dtype=torch.float32, seed=9)
    hf_io.load_hf_state_dict(m2, sd)
    assert torch.equal(m2.p("layers.1.sinks"), m.p("layers.1.sinks"))
