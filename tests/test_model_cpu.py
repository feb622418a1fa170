"""Model parity on CPU: our fused-layout decoder against HF transformers on a tiny random Qwen2."""
import math

import pytest
import torch

from skyrl_b200.models import hf_io
from skyrl_b200.models.decoder import CausalLM, ModelArgs


def _hf_tiny():
    from transformers import Qwen2Config, Qwen2ForCausalLM

    cfg = Qwen2Config(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256, rope_theta=1e4,
                      rms_norm_eps=1e-6, tie_word_embeddings=False, attention_dropout=0.0)
    torch.manual_seed(0)
    return Qwen2ForCausalLM(cfg).float().eval(), cfg


def test_forward_matches_hf_and_packing_is_exact():
    hf, cfg = _hf_tiny()
    args = ModelArgs.from_hf_config(cfg.to_dict())
    args.max_position_embeddings = 256
    m = CausalLM(args, dtype=torch.float32, seed=None)
    hf_io.load_hf_state_dict(m, hf.state_dict())
    lens = [7, 13, 1]
    ids = [torch.randint(0, 512, (n,)) for n in lens]
    packed = torch.cat(ids)
    pos = torch.cat([torch.arange(n) for n in lens]).to(torch.int32)
    cu = torch.tensor([0, 7, 20, 21], dtype=torch.int32)
    with torch.no_grad():
        h = m(packed, pos, cu, max(lens))
        logits = m.logits(h).float()
        for i, x in enumerate(ids):
            ref = hf(x[None]).logits[0]
            got = logits[cu[i]:cu[i + 1]]
            assert torch.allclose(got, ref, atol=2e-4, rtol=2e-4), (i, (got - ref).abs().max())


def test_logprob_head_and_backward_match_autograd():
    torch.manual_seed(1)
    args = ModelArgs(vocab_size=300, hidden_size=64, num_layers=1, num_heads=2, num_kv_heads=1, head_dim=32,
                     intermediate_size=128, tie_word_embeddings=True)
    m = CausalLM(args, dtype=torch.float32, seed=3)
    ids = torch.randint(0, 300, (12,))
    pos = torch.arange(12, dtype=torch.int32)
    cu = torch.tensor([0, 12], dtype=torch.int32)
    h = m(ids, pos, cu, 12)
    tgt = torch.randint(0, 300, (12,))
    lp, ent = m.token_logprobs(h, tgt, temperature=0.7, with_entropy=True)
    z = m.logits(h.detach()).float() / 0.7
    assert torch.allclose(lp, torch.log_softmax(z, -1).gather(-1, tgt[:, None]).squeeze(-1), atol=1e-5)
    p = torch.softmax(z, -1)
    assert torch.allclose(ent, -(p * torch.log_softmax(z, -1)).sum(-1), atol=1e-5)
    (lp.sum() + 0.1 * ent.sum()).backward()
    g = m.p("embed").grad.clone()
    m.zero_grad()
    # same through plain autograd on materialised logits
    h2 = m(ids, pos, cu, 12)
    z2 = (h2 @ m.p("embed").t()) / 0.7
    lp2 = torch.log_softmax(z2, -1)
    (lp2.gather(-1, tgt[:, None]).sum() + 0.1 * -(lp2.exp() * lp2).sum()).backward()
    assert torch.allclose(g, m.p("embed").grad, atol=1e-5)


def test_main_grad_accumulation_equals_grad():
    args = ModelArgs(vocab_size=128, hidden_size=64, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=32,
                     intermediate_size=96, attention_bias=True)
    m = CausalLM(args, dtype=torch.float32, seed=5)
    ids = torch.randint(0, 128, (9,))
    pos = torch.arange(9, dtype=torch.int32)
    cu = torch.tensor([0, 4, 9], dtype=torch.int32)
    pos = torch.tensor([0, 1, 2, 3, 0, 1, 2, 3, 4], dtype=torch.int32)
    tgt = torch.randint(0, 128, (9,))
    lp, _ = m.token_logprobs(m(ids, pos, cu, 5), tgt)
    lp.sum().backward()
    ref = {n: p.grad.clone() for n, p in m.named_flat_views()}
    m.zero_grad()
    flat = torch.zeros(m.flat_numel, dtype=torch.float32)
    m.attach_main_grad(flat)
    for _ in range(2):  # accumulates across micro-batches
        lp, _ = m.token_logprobs(m(ids, pos, cu, 5), tgt)
        lp.sum().backward()
    for n, p in m.named_flat_views():
        assert p.grad is None
        assert torch.allclose(p.main_grad, 2 * ref[n], atol=1e-5), n


def test_hf_export_roundtrip(tmp_path):
    args = ModelArgs(vocab_size=64, hidden_size=32, num_layers=1, num_heads=2, num_kv_heads=1, head_dim=16,
                     intermediate_size=48, attention_bias=True, tie_word_embeddings=True)
    m = CausalLM(args, dtype=torch.bfloat16, seed=7)
    hf_io.save_hf_model(m, str(tmp_path / "export"))
    from skyrl_b200.models.decoder import build_model

    m2 = build_model(str(tmp_path / "export"))
    assert torch.equal(m.flat_params, m2.flat_params)


def test_gradient_checkpointing_accumulates_into_main_grad():
    """Recomputation must route weight gradients into the fp32 flat buffer exactly like the plain backward."""
    import torch

    from skyrl_b200.models.decoder import PRESETS, CausalLM

    a = PRESETS["tiny-llama"]
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(4, a.vocab_size, (33,), generator=g).int()
    pos = torch.cat([torch.arange(13), torch.arange(20)]).int()
    cu = torch.tensor([0, 13, 33]).int()
    grads = []
    for ck in (False, True):
        m = CausalLM(a, device="cpu", dtype=torch.float32, seed=0)
        fg = torch.zeros(m.flat_params.numel())
        m.attach_main_grad(fg)
        m.gradient_checkpointing = ck
        lp, _ = m.token_logprobs(m(ids, pos, cu, 32), torch.roll(ids.long(), -1))
        lp.sum().backward()
        assert all(p.grad is None for p in m.parameters())
        grads.append(fg)
    assert torch.allclose(grads[0], grads[1], atol=1e-5, rtol=1e-4)
    assert grads[0].abs().sum() > 0
