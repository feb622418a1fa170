"""GPU integration: fused LM-head, bf16 model vs fp32 reference, graph decode vs eager, one GRPO step."""
import math

import pytest
import torch

from skyrl_b200.ops import _lib, lm_head

pytestmark = pytest.mark.gpu


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("T,V,H", [(300, 5000, 256), (1000, 151936, 1536), (129, 777 * 8, 512)])
def test_lm_head_fused_forward_backward(T, V, H):
    torch.manual_seed(0)
    h = (torch.randn(T, H, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    W = (torch.randn(V, H, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    tgt = torch.randint(0, V, (T,), device="cuda")
    lp, ent = lm_head.lm_head_logprobs(h, W, tgt, 1 / 0.8, with_entropy=True)
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    hr, Wr = h.detach().float().requires_grad_(), W.detach().float().requires_grad_()
    z = (hr @ Wr.t()) / 0.8
    lpr = torch.log_softmax(z, -1)
    ref_lp = lpr.gather(-1, tgt[:, None]).squeeze(-1)
    ref_ent = -(lpr.exp() * lpr).sum(-1)
    assert (lp - ref_lp).abs().max() < 3e-2 and (ent - ref_ent).abs().max() < 3e-2
    g1, g2 = torch.randn(T, device="cuda"), 0.1 * torch.randn(T, device="cuda")
    ((lp * g1).sum() + (ent * g2).sum()).backward()
    ((ref_lp * g1).sum() + (ref_ent * g2).sum()).backward()
    assert rel(h.grad, hr.grad) < 3e-2 and rel(W.grad, Wr.grad) < 3e-2


def test_model_bf16_cuda_matches_fp32_cpu():
    from skyrl_b200.models.decoder import PRESETS, CausalLM

    args = PRESETS["tiny-qwen2-d128"]
    ref = CausalLM(args, device="cpu", dtype=torch.float32, seed=3)
    m = CausalLM(args, device="cuda", dtype=torch.bfloat16, seed=None)
    m.flat_params.copy_(ref.flat_params)
    ref.flat_params.copy_(m.flat_params.float().cpu())  # identical (bf16-rounded) weights on both sides
    lens = [200, 37, 129]
    ids = torch.randint(0, args.vocab_size, (sum(lens),))
    pos = torch.cat([torch.arange(n) for n in lens]).to(torch.int32)
    cu = torch.tensor([0, 200, 237, 366], dtype=torch.int32)
    tgt = torch.randint(0, args.vocab_size, (sum(lens),))
    for mod, dev in ((ref, "cpu"), (m, "cuda")):
        h = mod(ids.to(dev), pos.to(dev), cu.to(dev), max(lens))
        lp, _ = mod.token_logprobs(h, tgt.to(dev))
        lp.sum().backward()
    hr = ref(ids, pos, cu, 200)
    hm = m(ids.cuda(), pos.cuda(), cu.cuda(), 200)
    assert rel(hm.cpu(), hr) < 3e-2
    for n, p in m.named_flat_views():
        gr = ref.p(n).grad
        if gr.abs().max() > 0:
            assert rel(p.grad.cpu(), gr) < 8e-2, n
    assert _lib.status_read_clear() == 0


def test_engine_graph_decode_matches_eager_and_naive():
    from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams
    from skyrl_b200.models.decoder import PRESETS, CausalLM

    m = CausalLM(PRESETS["tiny-qwen2-d128"], device="cuda", dtype=torch.bfloat16, seed=5)
    prompts = [torch.randint(4, 2048, (n,)).tolist() for n in (40, 7, 130, 64, 1)]
    sp = SamplingParams(max_tokens=20, temperature=0.0, ignore_eos=True)
    outs = {}
    for eager in (True, False):
        eng = LLMEngine(m, EngineConfig(block_size=16, max_num_seqs=8, max_model_len=256, sync_interval=4,
                                        enforce_eager=eager, num_blocks=256))
        outs[eager] = eng.generate(prompts, sp)
        assert eng.metrics()["kv_free_blocks"] == 256
    for a, b in zip(outs[True], outs[False]):
        assert a.token_ids == b.token_ids
        assert torch.allclose(torch.tensor(a.logprobs), torch.tensor(b.logprobs), atol=1e-3)
    # paged decode log-probs agree with a full packed forward over prompt + response
    for p, o in zip(prompts, outs[False]):
        toks = p + o.token_ids
        ids = torch.tensor(toks, device="cuda", dtype=torch.int32)
        with torch.no_grad():
            h = m(ids, torch.arange(len(toks), device="cuda", dtype=torch.int32),
                  torch.tensor([0, len(toks)], device="cuda", dtype=torch.int32), len(toks))
            lp, _ = m.token_logprobs(h[len(p) - 1 : -1], ids[len(p):])
        assert (lp.cpu() - torch.tensor(o.logprobs)).abs().max() < 5e-2
    assert _lib.status_read_clear() == 0


def test_engine_fused_decode_matches_unfused():
    from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams
    from skyrl_b200.models.decoder import PRESETS, CausalLM

    m = CausalLM(PRESETS["tiny-qwen2-d128"], device="cuda", dtype=torch.bfloat16, seed=7)
    prompts = [torch.randint(4, 2048, (n,)).tolist() for n in (33, 5, 90, 64)]
    sp = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
    outs = {}
    for fused in (False, True):
        eng = LLMEngine(m, EngineConfig(block_size=16, max_num_seqs=8, max_model_len=256, sync_interval=4,
                                        enforce_eager=True, num_blocks=256, fused_decode=fused))
        outs[fused] = eng.generate(prompts, sp)
    same = total = 0
    for a, b in zip(outs[False], outs[True]):
        # greedy decoding may fork on a near-tie; compare the common prefix
        k = 0
        while k < len(a.token_ids) and a.token_ids[k] == b.token_ids[k]:
            k += 1
        same += k
        total += len(a.token_ids)
        assert k >= 1
        assert (torch.tensor(a.logprobs[:k]) - torch.tensor(b.logprobs[:k])).abs().max() < 5e-2
    assert same >= 0.7 * total
    assert _lib.status_read_clear() == 0


def test_grpo_step_on_gpu():
    import __graft_entry__ as ge

    ge.smoke()


def test_moe_grpo_step_with_router_replay_on_gpu(tmp_path):
    """One GRPO step of a mixture-of-experts policy whose training passes replay the rollout's expert choices."""
    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.models import router_replay
    from skyrl_b200.parallel import dist as pdist
    from skyrl_b200.train.trainer import PPOTrainer
    from skyrl_b200.utils.tokenizer import SyntheticTokenizer

    pdist.reset_env_for_tests()
    cfg = SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model.path=tiny-moe", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4",
        "trainer.micro_train_batch_size_per_gpu=4", "trainer.micro_forward_batch_size_per_gpu=8",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=24",
        "trainer.max_prompt_length=48", "trainer.algorithm.use_kl_loss=false", "environment.env_class=synthetic_even",
        "generator.batched=true", "generator.inference_engine.max_num_seqs=16", "trainer.seed=0",
        "generator.inference_engine.enable_return_routed_experts=true",
        "trainer.policy.megatron_config.moe_enable_routing_replay=true",
        f"trainer.ckpt_path={tmp_path}/ckpt", f"trainer.export_path={tmp_path}/export", "trainer.resume_mode=none"])
    tr = PPOTrainer(cfg, tokenizer=SyntheticTokenizer(1024))
    tr.build_models()
    g = torch.Generator().manual_seed(0)
    prompts = []
    for i in range(4):
        ids = torch.randint(4, 1024, (40,), generator=g).tolist()
        prompts.append({"prompt": [{"role": "user", "content": ids}], "prompt_token_ids": ids, "uid": f"p{i}"})
    m = tr.train_step(prompts)
    assert math.isfinite(m["policy/final_loss"]) and m["policy/grad_norm"] > 0
    # the training pass ran through the rollout's experts: its log-probs agree with the engine's to bf16 accuracy
    assert m["policy/rollout_train_logprobs_abs_diff_mean"] < 5e-2
    assert not router_replay.active()
    assert _lib.status_read_clear() == 0


def test_engine_moe_graph_decode_matches_eager():
    """Mixture-of-experts decode replays from a CUDA graph (device-side routing plan) with the eager path's tokens."""
    from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams
    from skyrl_b200.models.decoder import PRESETS, CausalLM

    m = CausalLM(PRESETS["tiny-moe"], device="cuda", dtype=torch.bfloat16, seed=9)
    prompts = [torch.randint(4, 1024, (n,)).tolist() for n in (33, 5, 70, 18)]
    sp = SamplingParams(max_tokens=16, temperature=0.0, ignore_eos=True)
    outs = {}
    for eager in (True, False):
        eng = LLMEngine(m, EngineConfig(block_size=16, max_num_seqs=8, max_model_len=256, sync_interval=4,
                                        enforce_eager=eager, num_blocks=128))
        outs[eager] = eng.generate(prompts, sp)
        if not eager:
            assert eng.stats["graph_replays"] > 0
    for a, b in zip(outs[True], outs[False]):
        assert a.token_ids == b.token_ids
        assert torch.allclose(torch.tensor(a.logprobs), torch.tensor(b.logprobs), atol=1e-3)
    assert _lib.status_read_clear() == 0


def test_engine_returns_routed_experts_on_gpu_and_replay_reproduces_the_forward():
    """Routing capture on the device path: tables have one row per fed token, agree with a full forward over the same
    tokens (bf16 near-ties aside), and replaying them through the model gives that forward's hidden states."""
    from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams
    from skyrl_b200.models import router_replay
    from skyrl_b200.models.decoder import PRESETS, CausalLM

    m = CausalLM(PRESETS["tiny-moe"], device="cuda", dtype=torch.bfloat16, seed=9)
    a = m.args
    eng = LLMEngine(m, EngineConfig(block_size=16, max_num_seqs=8, max_model_len=256, sync_interval=4, num_blocks=128,
                                    return_routed_experts=True))
    gen = torch.Generator().manual_seed(3)
    prompts = [torch.randint(4, 1024, (n,), generator=gen).tolist() for n in (33, 5, 70)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
    assert eng.stats["graph_replays"] == 0  # recording runs the decode steps eagerly
    agree, total = 0, 0
    for p, o in zip(prompts, outs):
        toks = p + o.token_ids[:-1]
        r = o.routed_experts
        assert tuple(r.shape) == (len(toks), a.num_layers, a.num_experts_per_tok) and r.dtype == torch.int16
        assert int(r.min()) >= 0 and int(r.max()) < a.num_experts
        ids = torch.tensor(toks, dtype=torch.int32, device="cuda")
        pos = torch.arange(len(toks), dtype=torch.int32, device="cuda")
        cu = torch.tensor([0, len(toks)], dtype=torch.int32, device="cuda")
        with torch.no_grad(), router_replay.record_routing() as store:
            h_free = m(ids, pos, cu, len(toks))
        want = router_replay.stack_recorded(store).cpu()
        same = (r.long().sort(-1).values == want.sort(-1).values).all(-1)
        agree += int(same.sum())
        total += same.numel()
        with torch.no_grad(), router_replay.replay_routing(want.to(torch.int16).cuda()):
            h_replay = m(ids, pos, cu, len(toks))
        assert rel(h_replay, h_free) < 5e-3  # gate weights: fused router kernel vs softmax + gather, in bf16
    assert agree / total > 0.9, (agree, total)
    assert _lib.status_read_clear() == 0


def test_attention_sinks_kernels_match_reference():
    """Sink attention = the tcgen05 kernels unchanged + the sink folded into the log-sum-exp: forward and all three
    gradients (qkv, sinks) against the fp32 PyTorch formulation with an explicit sink column."""
    import math

    from skyrl_b200.ops import attention as A

    torch.manual_seed(0)
    nq, nkv, D = 4, 2, 128
    lens = [150, 37, 260]
    cu = torch.tensor([0, 150, 187, 447], device="cuda", dtype=torch.int32)
    T = sum(lens)
    qkv = (torch.randn(T, (nq + 2 * nkv) * D, device="cuda") * 0.5).bfloat16().requires_grad_()
    sinks = torch.tensor([1.0, -2.0, 3.0, 0.0], device="cuda", requires_grad=True)
    dy = (torch.randn(T, nq * D, device="cuda") * 0.1).bfloat16()
    out = A.attn_varlen(qkv, cu, nq, nkv, D, max_seqlen=max(lens), sinks=sinks)
    out.backward(dy)
    q2 = qkv.detach().float().requires_grad_()
    s2 = sinks.detach().clone().requires_grad_()
    ref, _ = A.attn_varlen_ref(q2, cu, nq, nkv, D, 1 / math.sqrt(D), s2)
    ref.backward(dy.float())
    assert (out.float() - ref).abs().max() < 2e-2
    assert (qkv.grad.float() - q2.grad).abs().max() < 2e-2
    assert (sinks.grad - s2.grad).abs().max() < 5e-2 * max(1.0, s2.grad.abs().max().item())
    assert s2.grad.abs().max() > 1e-2
    assert _lib.status_read_clear() == 0


def test_vmm_arena_keeps_addresses_across_sleep():
    from skyrl_b200.engine.vmm import VmmArena

    free0 = torch.cuda.mem_get_info()[0]
    ar = VmmArena(512 << 20, "cuda")
    a = ar.take((1024, 1024), torch.bfloat16)
    b = ar.take((7, 3), torch.float32)
    assert a.data_ptr() == ar.ptr and b.data_ptr() % 256 == 0 and b.data_ptr() >= a.data_ptr() + a.numel() * 2
    a.fill_(1.5)
    b.fill_(2.0)
    assert float(a.float().sum()) == 1.5 * 1024 * 1024 and float(b.sum()) == 42.0
    assert free0 - torch.cuda.mem_get_info()[0] >= 500 << 20
    ar.sleep()
    assert not ar.mapped and free0 - torch.cuda.mem_get_info()[0] < 64 << 20  # physical memory returned
    ar.wake()
    assert ar.mapped and a.data_ptr() == ar.ptr
    assert float(a.float().abs().sum()) == 0.0  # fresh memory, zeroed by wake()
    a.fill_(0.5)
    assert float(a.float().sum()) == 0.5 * 1024 * 1024
    ar.close()
    assert free0 - torch.cuda.mem_get_info()[0] < 64 << 20


def test_engine_sleep_wake_keeps_graphs_with_fixed_address_cache():
    from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams
    from skyrl_b200.models.decoder import PRESETS, CausalLM

    m = CausalLM(PRESETS["tiny-qwen2-d128"], device="cuda", dtype=torch.bfloat16, seed=5)
    prompts = [torch.randint(4, 2048, (n,)).tolist() for n in (40, 7, 64)]
    sp = SamplingParams(max_tokens=16, temperature=0.0, ignore_eos=True)
    eng = LLMEngine(m, EngineConfig(block_size=16, max_num_seqs=8, max_model_len=256, sync_interval=4, num_blocks=4096))
    assert eng._kv_arena is not None
    first = eng.generate(prompts, sp)
    graphs = dict(eng._graphs)
    assert graphs, "decode should have been captured"
    ptr = eng.k_cache[0].data_ptr()
    torch.cuda.synchronize()
    used = torch.cuda.mem_get_info()[0]
    eng.sleep()
    assert torch.cuda.mem_get_info()[0] - used >= eng._kv_arena.nbytes - (32 << 20)
    eng.wake_up()
    assert eng.k_cache[0].data_ptr() == ptr and dict(eng._graphs) == graphs  # nothing re-captured
    again = eng.generate(prompts, sp)
    for a, b in zip(first, again):
        assert a.token_ids == b.token_ids
    assert _lib.status_read_clear() == 0
