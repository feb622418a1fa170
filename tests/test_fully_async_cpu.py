"""Fully-async trainer: admission rule, invariants, an end-to-end run with in-flight weight sync, resume state."""
import asyncio

import pytest
import torch

from skyrl_b200.config.config import SkyRLTrainConfig
from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine
from skyrl_b200.inference.local_client import LocalInferenceClient
from skyrl_b200.models.decoder import build_model
from skyrl_b200.parallel import dist as pdist
from skyrl_b200.train.dataset import PromptDataset
from skyrl_b200.train.fully_async_trainer import AsyncDataloader, AsyncStalenessManager, FullyAsyncPPOTrainer
from skyrl_b200.utils.tokenizer import SyntheticTokenizer


def test_capacity_rule_and_invariant():
    async def run():
        m = AsyncStalenessManager(max_workers=6, max_staleness_steps=1, mini_batch_size=4)
        assert m.capacity() == min(6, (1 + 1) * 4)
        for _ in range(6):
            await m.acquire_submission_slot()
        assert m.capacity() == 0 and m.running == 6
        for _ in range(4):
            await m.on_rollout_accepted()
        m.check_invariant()
        # step 1 budget: (S + 1) * B = 8 rollouts may exist; 4 accepted + 2 running -> 2 more
        assert m.capacity() == min(6 - 2, 8 - 6) == 2
        blocked = asyncio.create_task(asyncio.wait_for(_take(m, 3), 0.05))
        with pytest.raises(asyncio.TimeoutError):
            await blocked
        await m.on_rollout_cancelled()  # the timed-out acquire may have taken slots; restore for the check below
        await m.notify_capacity_change(2)
        assert m.capacity() > 0
        await m.on_rollout_filtered()
        m.check_invariant()

    async def _take(m, n):
        for _ in range(n):
            await m.acquire_submission_slot()

    asyncio.run(run())


def test_dataloader_skips_consumed_and_rolls_epochs():
    ds = PromptDataset([{"prompt": [{"role": "user", "content": "1 2"}], "uid": f"u{i}"} for i in range(5)])

    async def run():
        dl = AsyncDataloader(ds, seed=0, epochs=2, consumed_uids={"0:u1", "0:u3"})
        seen = []
        while True:
            it = await dl.next()
            if it is None:
                break
            seen.append(it["_consumed_key"])
        return seen

    seen = asyncio.run(run())
    assert len(seen) == 3 + 5 and "0:u1" not in seen and "1:u1" in seen


def test_fully_async_end_to_end(tmp_path):
    pdist.reset_env_for_tests()
    cfg = SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model.path=tiny-llama", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=8",
        "trainer.max_prompt_length=16", "trainer.algorithm.use_kl_loss=false", "trainer.algorithm.policy_loss_type=rollout_is",
        "trainer.placement.colocate_all=false", "trainer.fully_async.enabled=true",
        "trainer.fully_async.max_staleness_steps=1", "trainer.fully_async.num_parallel_generation_workers=3",
        "trainer.micro_train_batch_size_per_gpu=4", "trainer.micro_forward_batch_size_per_gpu=4",
        "environment.env_class=synthetic_even", "trainer.bf16=false", "trainer.gradient_checkpointing=false",
        "trainer.max_training_steps=3", "trainer.ckpt_interval=2", f"trainer.ckpt_path={tmp_path}/ckpt",
        "trainer.resume_mode=none", "trainer.policy.optimizer_config.lr=1e-4"])
    tok = SyntheticTokenizer(1024)
    engine_model = build_model("tiny-llama", dtype=torch.float32, seed=cfg.trainer.seed)
    eng = LLMEngine(engine_model, EngineConfig(block_size=8, max_num_seqs=8, max_model_len=64, sync_interval=2,
                                               enforce_eager=True), eos_token_ids=[1])
    client = LocalInferenceClient([eng], tok)
    items = [{"prompt": [{"role": "user", "content": " ".join(str(4 + (7 * i + j) % 900) for j in range(8))}],
              "uid": f"u{i}"} for i in range(12)]
    tr = FullyAsyncPPOTrainer(cfg, tokenizer=tok, train_dataset=PromptDataset(items), inference_engine_client=client)
    tr.build_models()
    syncs = []

    def transfer():
        engine_model.flat_params.copy_(tr.policy.model.flat_params)
        syncs.append(eng.paused)

    tr.weight_transfer = transfer
    asyncio.run(tr.train_async())
    assert tr.global_step == 3 and syncs == [True, True, True] and not eng.paused
    assert torch.equal(engine_model.flat_params, tr.policy.model.flat_params)
    assert eng.weight_version == 3 and len(tr.consumed_uids) == 6
    tr.staleness.check_invariant()
    st = torch.load(f"{tmp_path}/ckpt/global_step_2/fully_async_state.pt", weights_only=False)
    assert len(st["consumed_uids"]) == 4


def test_one_step_off_trainer_overlaps_generation_and_training(tmp_path):
    """Batch k+1 is generated from the weights of step k-1 while step k trains; the engine has its own weight copy."""
    import torch

    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.parallel.dist import get_env
    from skyrl_b200.train.async_trainer import OneStepOffPPOTrainer
    from skyrl_b200.train.dataset import PromptDataset
    from skyrl_b200.utils.tokenizer import SyntheticTokenizer

    cfg = SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model.path=tiny-qwen2-d128", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
        "generator.n_samples_per_prompt=4", "trainer.max_prompt_length=32", "generator.sampling_params.max_generate_length=8",
        "environment.env_class=synthetic_bernoulli", "trainer.bf16=false", "trainer.policy.optimizer_config.lr=1e-3",
        "generator.inference_engine.max_num_seqs=8", "generator.inference_engine.enforce_eager=true",
        "generator.inference_engine.engine_init_kwargs={num_blocks: 64}", "trainer.resume_mode=none", "trainer.ckpt_interval=-1",
        "trainer.algorithm.use_kl_loss=false", "trainer.logger=console", "trainer.eval_interval=-1", "trainer.epochs=1",
        f"trainer.ckpt_path={tmp_path}"])
    tok = SyntheticTokenizer(2048)
    rows = [{"prompt": [{"role": "user", "content": f"q{i}"}], "env_class": "synthetic_bernoulli",
             "env_extras": {"p": 0.5, "seed": i}} for i in range(6)]
    ds = PromptDataset(rows, tok, 32)
    tr = OneStepOffPPOTrainer(cfg, tokenizer=tok, train_dataset=ds, env=get_env())
    tr.build_models()
    assert tr.engine.model is not tr.policy.model
    before = tr.policy.model.flat_params.clone()
    tr.train()
    assert tr.global_step == 3
    assert not torch.equal(tr.policy.model.flat_params, before)
    assert torch.equal(tr.engine.model.flat_params, tr.policy.model.flat_params)  # last sync published the weights


def test_zero_variance_group_filter_ignores_masked_trajectories():
    from types import SimpleNamespace

    def zv(tol, rewards, masks):
        fake = SimpleNamespace(cfg=SimpleNamespace(trainer=SimpleNamespace(algorithm=SimpleNamespace(zero_variance_filter_tol=tol))))
        return FullyAsyncPPOTrainer._zero_variance(fake, {"rewards": rewards, "loss_masks": masks})

    assert zv(0.0, [1.0, 1.0], [[1], [1]]) is True          # nothing to learn from: dropped
    assert zv(0.0, [1.0, 0.0], [[1], [1]]) is False
    assert zv(0.0, [1.0], [[1]]) is False                    # a single trajectory is kept
    assert zv(0.0, [1.0, 1.0, 0.0], [[1], [1], [0]]) is True  # the masked one does not count
    assert zv(1e-6, [0.6667, 0.66670001], [[1], [1]]) is True
    assert zv(0.0, [[0.0, 1.0], [1.0, 0.0]], [[1, 1], [1, 1]]) is True   # token-level rewards: compared by their sums
    assert zv(0.0, [[0.0, 1.0], [0.0, 0.0]], [[1, 1], [1, 1]]) is False
