"""LoRA adapters: zero-initialised delta, gradients only on adapters, merge equals adapter forward, PEFT export
round trip, and an RL step that trains only the adapter buffer."""
import os

import torch

from skyrl_b200.models.decoder import PRESETS, CausalLM
from skyrl_b200.models.lora import LoRACausalLM, resolve_targets


def _inputs(a):
    lens = [13, 20]
    ids = torch.randint(4, a.vocab_size, (sum(lens),), generator=torch.Generator().manual_seed(0)).int()
    pos = torch.cat([torch.arange(n) for n in lens]).int()
    cu = torch.tensor([0, 13, 33]).int()
    return ids, pos, cu


def test_targets():
    assert resolve_targets("all-linear") == ["qkv", "o", "gate_up", "down"]
    assert resolve_targets("q_proj,v_proj,down_proj") == ["qkv", "down"]
    assert resolve_targets("all-linear", "o_proj") == ["qkv", "gate_up", "down"]


def test_lora_forward_backward_merge_and_export(tmp_path):
    a = PRESETS["tiny-llama"]
    base = CausalLM(a, device="cpu", dtype=torch.float32, seed=0)
    m = LoRACausalLM(a, rank=4, alpha=8, device="cpu", dtype=torch.float32, seed=0)
    ids, pos, cu = _inputs(a)
    h0 = base(ids, pos, cu, 32)
    assert torch.allclose(m(ids, pos, cu, 32), h0, atol=1e-6)  # B starts at zero
    assert m.num_trainable_parameters() < 0.1 * base.num_parameters()
    with torch.no_grad():
        for n, p in m.trainable_named():
            if n.endswith("lora_B"):
                p[:, :4].normal_(0, 0.05)
    h = m(ids, pos, cu, 32)
    assert (h - h0).abs().max() > 1e-3
    h.square().sum().backward()
    assert all(p.grad is None for p in m._p.values())  # the base is frozen
    for n, p in m.trainable_named():
        assert p.grad is not None and torch.isfinite(p.grad).all()
        if n.endswith("lora_A"):
            assert p.grad[4:].abs().max() == 0  # rank padding stays untouched
    merged = CausalLM(a, device="cpu", dtype=torch.float32, seed=None)
    m.merge_into(merged)
    assert torch.allclose(merged(ids, pos, cu, 32), h.detach(), atol=2e-4)
    m.save_adapter(str(tmp_path))
    assert os.path.exists(tmp_path / "adapter_config.json")
    m2 = LoRACausalLM(a, rank=4, alpha=8, device="cpu", dtype=torch.float32, seed=0)
    m2.load_adapter(str(tmp_path))
    assert torch.allclose(m2(ids, pos, cu, 32), h.detach(), atol=1e-6)


def test_rl_step_with_lora_updates_only_adapters():
    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.parallel.dist import get_env
    from skyrl_b200.train.trainer import PPOTrainer
    from skyrl_b200.utils.tokenizer import SyntheticTokenizer

    cfg = SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model.path=tiny-qwen2-d128", "trainer.policy.model.lora.rank=8", "trainer.train_batch_size=2",
        "trainer.policy_mini_batch_size=2", "generator.n_samples_per_prompt=4", "trainer.max_prompt_length=16",
        "generator.sampling_params.max_generate_length=8", "environment.env_class=synthetic_bernoulli", "trainer.bf16=false",
        "trainer.policy.optimizer_config.lr=1e-2", "trainer.policy.optimizer_config.num_warmup_steps=0",
        "generator.inference_engine.max_num_seqs=8", "generator.inference_engine.enforce_eager=true",
        "generator.inference_engine.engine_init_kwargs={num_blocks: 64}", "trainer.resume_mode=none",
        "trainer.algorithm.use_kl_loss=false", "trainer.logger=console"])
    tok = SyntheticTokenizer(2048)
    tr = PPOTrainer(cfg, tokenizer=tok, env=get_env())
    tr.build_models()
    m = tr.policy.model
    assert isinstance(m, LoRACausalLM) and tr.engine.model is not m
    base_before = m.base_flat_params.clone()
    eng_before = tr.engine.model.flat_params.clone()
    prompts = [{"prompt": [{"role": "user", "content": f"q{i}"}], "uid": f"u{i}", "env_extras": {"p": 0.5, "seed": i}}
               for i in range(2)]
    moved = False
    for _ in range(3):
        tr.train_step(prompts)
        moved = moved or not torch.equal(tr.engine.model.flat_params, eng_before)
    assert torch.equal(m.base_flat_params, base_before)
    assert moved  # merged weights reached the engine once the adapters moved
