"""Dynamic sampling (DAPO filter / POLARIS replace): unit behaviour and the trainer loop that keeps sampling."""
import pytest
import torch

from skyrl_b200.train.dynamic_sampling import DynamicSampler, group_informative, select_rows
from skyrl_b200.train.generators.base import GeneratorOutput, TrajectoryID


def _out(rewards, n=2):
    B = len(rewards)
    return GeneratorOutput(prompt_token_ids=[[1, 2, i] for i in range(B)], response_ids=[[5, 6 + i] for i in range(B)],
                           rewards=list(rewards), loss_masks=[[1, 1]] * B, stop_reasons=["stop"] * B,
                           rollout_logprobs=[[-0.1, -0.2]] * B, rollout_metrics={},
                           trajectory_ids=[TrajectoryID(f"u{i // n}", i % n) for i in range(B)])


def _uids(B, n=2, tag="u"):
    return [f"{tag}{i // n}" for i in range(B)]


def test_group_informative_and_select_rows():
    out = _out([1.0, 0.0, 1.0, 1.0, [0.0, 1.0], [0.5, 0.5]])
    good = group_informative(out, _uids(6), 2)
    assert good == {"u0": True, "u1": False, "u2": False}  # token-level rewards are summed per trajectory
    assert group_informative(out, _uids(6), 1) == {"u0": True, "u1": True, "u2": True}
    sub = select_rows(out, [3, 0, 0])
    assert sub["response_ids"] == [[5, 9], [5, 6], [5, 6]] and sub["rewards"][0] == 1.0
    assert sub["rollout_metrics"]["generate/avg_num_tokens"] == 2.0


def test_filter_accumulates_until_target_then_truncates():
    s = DynamicSampler("filter", target_prompts=3, n_samples_per_prompt=2, max_sample_batches=5)
    out1 = _out([1, 0, 1, 1, 0, 0, 0, 1])  # groups: good, bad, bad, good
    res, uids, keep = s.handle(out1, _uids(8, tag="a"))
    assert keep and s.collected_prompts == 2
    out2 = _out([0, 1, 1, 0, 1, 1, 1, 0])  # good, good, bad, good -> three more, one too many
    res, uids, keep = s.handle(out2, _uids(8, tag="b"))
    assert not keep
    assert uids == ["a0", "a0", "a3", "a3", "b0", "b0"]
    assert res["rewards"] == [1, 0, 0, 1, 0, 1] and len(res["response_ids"]) == 6
    assert s.rounds == 0 and s.collected is None  # reset for the next RL step
    assert s.metrics()["dynamic_sampling/sample_batches"] == 2.0


def test_filter_gives_up_after_max_sample_batches():
    s = DynamicSampler("filter", target_prompts=2, n_samples_per_prompt=2, max_sample_batches=2)
    flat = _out([1, 1, 0, 0])
    assert s.handle(flat, _uids(4))[2] is True
    with pytest.raises(RuntimeError, match="max_sample_batches"):
        s.handle(flat, _uids(4))


def test_replace_overwrites_flat_groups_and_keeps_batch_size():
    s = DynamicSampler("replace", target_prompts=4, n_samples_per_prompt=2, min_replace_ratio=0.3, seed=1)
    out = _out([1, 0, 1, 1, 0, 0, 0, 1])
    res, uids, keep = s.handle(out, _uids(8))
    assert not keep and len(uids) == 8 and len(res["rewards"]) == 8
    assert uids[:2] == ["u0", "u0"] and uids[6:] == ["u3", "u3"]
    for lo in (2, 4):  # the two flat groups now hold copies of informative groups, under their own group ids
        assert res["rewards"][lo : lo + 2] in ([1, 0], [0, 1]) and uids[lo] == uids[lo + 1] and "#r" in uids[lo]
    # too few informative groups: ask for another batch
    s2 = DynamicSampler("replace", target_prompts=4, n_samples_per_prompt=2, min_replace_ratio=0.5)
    assert s2.handle(_out([1, 0, 1, 1, 0, 0, 1, 1]), _uids(8))[2] is True
    with pytest.raises(ValueError):
        DynamicSampler("nope", 1, 1)


def test_trainer_keeps_sampling_until_the_batch_is_informative(tmp_path):
    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.parallel import dist as pdist
    from skyrl_b200.train.trainer import PPOTrainer
    from skyrl_b200.utils.tokenizer import SyntheticTokenizer

    pdist.reset_env_for_tests()
    cfg = SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model.path=tiny-llama", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4",
        "trainer.micro_train_batch_size_per_gpu=4", "trainer.micro_forward_batch_size_per_gpu=4",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=8",
        "trainer.max_prompt_length=16", "trainer.algorithm.use_kl_loss=false", "environment.env_class=synthetic_bernoulli",
        "generator.batched=true", "trainer.bf16=false", "trainer.gradient_checkpointing=false",
        "generator.inference_engine.max_num_seqs=16", "generator.inference_engine.enforce_eager=true",
        "trainer.resume_mode=none", "trainer.algorithm.dynamic_sampling.type=filter",
        "trainer.algorithm.dynamic_sampling.max_sample_batches=50", f"trainer.ckpt_path={tmp_path}/c",
        f"trainer.export_path={tmp_path}/e"])
    tr = PPOTrainer(cfg, tokenizer=SyntheticTokenizer(1024))
    tr.build_models()
    g = torch.Generator().manual_seed(0)
    rounds, m = 0, {"trainer/keep_sampling": 1.0}
    while m.get("trainer/keep_sampling"):
        items = []
        for i in range(4):
            ids = torch.randint(4, 1024, (16,), generator=g).tolist()
            items.append({"prompt": [{"role": "user", "content": ids}], "prompt_token_ids": ids, "uid": f"r{rounds}p{i}",
                          "env_extras": {"p": 0.0 if rounds == 0 else 0.5, "seed": 17 * rounds + i}})
        m = tr.train_step(items)
        rounds += 1
        assert rounds < 50
    # the first round's rewards are all zero (nothing informative); Bernoulli(0.5) pairs are informative half of the time
    assert rounds >= 2 and tr.global_step == 1 and m["dynamic_sampling/sample_batches"] == float(rounds)
    assert m["trainer/num_generated_tokens"] == 4 * 2 * 8
    assert m["reward/avg_raw_reward"] == 0.5  # every kept group holds one success and one failure
