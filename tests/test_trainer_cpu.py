"""CPU plumbing GRPO: tiny Llama-style model, synthetic prompts, in-process engine, one policy update per step."""
import os

import pytest
import torch

from skyrl_b200.config.config import SkyRLTrainConfig
from skyrl_b200.models.decoder import PRESETS
from skyrl_b200.parallel import dist as pdist
from skyrl_b200.train.trainer import PPOTrainer
from skyrl_b200.utils.tokenizer import SyntheticTokenizer


def _cfg(tmp, extra=()):
    return SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model.path=tiny-llama", "trainer.train_batch_size=8", "trainer.policy_mini_batch_size=8",
        "trainer.micro_train_batch_size_per_gpu=4", "trainer.micro_forward_batch_size_per_gpu=8",
        "generator.n_samples_per_prompt=4", "generator.sampling_params.max_generate_length=32",
        "generator.sampling_params.temperature=1.0", "trainer.max_prompt_length=64",
        "trainer.algorithm.kl_loss_coef=0.001", "trainer.algorithm.use_kl_loss=true",
        "trainer.policy.optimizer_config.lr=1e-5", "trainer.policy.optimizer_config.adam_betas=[0.9,0.999]",
        "environment.env_class=synthetic_even", "generator.batched=true", "trainer.bf16=false",
        "trainer.gradient_checkpointing=false", "generator.inference_engine.max_num_seqs=32",
        "generator.inference_engine.enforce_eager=true", "trainer.seed=0", f"trainer.ckpt_path={tmp}/ckpt",
        f"trainer.export_path={tmp}/export", "trainer.resume_mode=none", *extra])


def _prompts(n=8, L=64, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for i in range(n):
        ids = torch.randint(4, 1024, (L,), generator=g).tolist()
        out.append({"prompt": [{"role": "user", "content": ids}], "prompt_token_ids": ids, "uid": f"p{i}"})
    return out


def test_grpo_step_runs_and_updates_weights(tmp_path):
    pdist.reset_env_for_tests()
    cfg = _cfg(tmp_path)
    tr = PPOTrainer(cfg, tokenizer=SyntheticTokenizer(1024))
    tr.build_models()
    w0 = tr.policy.model.flat_params.clone()
    m = tr.train_step(_prompts())
    assert torch.isfinite(torch.tensor(m["policy/final_loss"]))
    assert m["policy/grad_norm"] > 0
    assert not torch.equal(w0, tr.policy.model.flat_params)
    assert 8 * 4 * 16 < m["trainer/num_generated_tokens"] <= 8 * 4 * 32  # a few samples may hit EOS early
    # rollout and trainer log-probs come from the same weights and the same arithmetic
    assert m["policy/rollout_train_logprobs_abs_diff_mean"] < 1e-4
    assert tr.engine.weight_version == 1
    # on-policy first update: ratio == 1 so nothing is clipped
    assert m["policy/loss_metrics/clip_ratio"] == 0.0
    m2 = tr.train_step(_prompts(seed=1))
    assert m2["trainer/global_step"] == 2.0


def test_checkpoint_resume_roundtrip(tmp_path):
    pdist.reset_env_for_tests()
    cfg = _cfg(tmp_path)
    tr = PPOTrainer(cfg, tokenizer=SyntheticTokenizer(1024))
    tr.build_models()
    tr.train_step(_prompts())
    tr.save_checkpoints()
    ref_params = tr.policy.model.flat_params.clone()
    ref_m = tr.policy.optimizer.exp_avg.clone()
    assert open(os.path.join(cfg.trainer.ckpt_path, "latest_ckpt_global_step.txt")).read() == "1"
    cfg2 = _cfg(tmp_path, ["trainer.resume_mode=latest"])
    tr2 = PPOTrainer(cfg2, tokenizer=SyntheticTokenizer(1024))
    tr2.build_models()
    assert tr2.load_checkpoints() == 1
    assert torch.equal(tr2.policy.model.flat_params, ref_params)
    assert torch.equal(tr2.policy.optimizer.exp_avg, ref_m)


def test_ppo_with_critic_gae(tmp_path):
    pdist.reset_env_for_tests()
    cfg = _cfg(tmp_path, ["trainer.algorithm.advantage_estimator=gae", "trainer.critic.model.path=tiny-llama",
                          "trainer.critic_mini_batch_size=8", "trainer.algorithm.use_kl_loss=false",
                          "trainer.algorithm.lambd=0.95"])
    tr = PPOTrainer(cfg, tokenizer=SyntheticTokenizer(1024))
    tr.build_models()
    m = tr.train_step(_prompts())
    assert "critic/critic_loss" in m and m["critic/grad_norm"] > 0 and m["policy/grad_norm"] > 0


def test_two_minibatches_recompute_old_logprobs_with_train_packing(tmp_path):
    """train_batch 8 / mini-batch 4: two optimizer steps; the old log-probs are computed mini-batch by mini-batch with
    the training micro-batch size, so the first update of the step sees ratio == 1 exactly (nothing clipped)."""
    pdist.reset_env_for_tests()
    cfg = _cfg(tmp_path, ["trainer.policy_mini_batch_size=4", "trainer.micro_train_batch_size_per_gpu=2",
                          "trainer.micro_forward_batch_size_per_gpu=16", "trainer.recompute_old_logprobs_per_minibatch=true",
                          "trainer.algorithm.use_kl_loss=false"])
    tr = PPOTrainer(cfg, tokenizer=SyntheticTokenizer(1024))
    tr.build_models()
    seen = []
    orig = tr.policy.forward_backward

    def spy(mini, **kw):
        st = orig(mini, **kw)
        seen.append((mini.batch_size, st["loss_metrics/clip_ratio"]))
        return st

    tr.policy.forward_backward = spy
    tr.train_step(_prompts())
    assert tr.policy.optimizer.step_count == 2 and [b for b, _ in seen] == [16, 16]
    assert seen[0][1] == 0.0
    # same values as one full-batch forward (fp32 on CPU: packing changes nothing beyond rounding)
    b = tr._last_batch
    full = tr.policy.forward(b)["output"]
    per_mb = tr._forward_old(tr.policy, "policy", b)
    assert torch.allclose(full, per_mb, atol=1e-5)


def test_example_logging_trajectory_samples_and_batch_dump(tmp_path, caplog):
    import glob
    import json
    import logging

    from skyrl_b200.train.batch import TrainingInputBatch

    pdist.reset_env_for_tests()
    cfg = _cfg(tmp_path, ["trainer.print_example_interval=1", "trainer.num_logger_train_samples=3",
                          "trainer.dump_data_batch=true", f"trainer.log_path={tmp_path}/logs"])
    tr = PPOTrainer(cfg, tokenizer=SyntheticTokenizer(1024))
    tr.build_models()
    with caplog.at_level(logging.INFO, logger="skyrl_b200.train.trainer"):
        tr.train_step(_prompts())
    assert any("--- response ---" in r.getMessage() for r in caplog.records)
    rows = [json.loads(l) for l in open(glob.glob(f"{tmp_path}/logs/trajectories/train_trajectories_step_0.jsonl")[0])]
    assert len(rows) == 3 and all(r["response_length"] > 0 for r in rows)
    dumped = glob.glob(f"{tmp_path}/export/dumped_data/global_step_0_training_input.bin")
    assert len(dumped) == 1
    back = TrainingInputBatch.from_bytes(open(dumped[0], "rb").read())
    assert back["sequences"].shape[0] == 32 and "advantages" in back
    # the old name of the interval still works
    old = _cfg(tmp_path, ["trainer.log_example_interval=7"])
    assert old.trainer.print_example_interval == 7
    # decode-graph sizes reach the engine
    sized = _cfg(tmp_path, ["trainer.b200.decode_graph_batch_sizes=[4,16,8]"])
    tr2 = PPOTrainer(sized, tokenizer=SyntheticTokenizer(1024))
    tr2.build_models()
    assert tuple(tr2.engine.cfg.graph_batch_sizes) == (4, 8, 16)


def test_postprocess_rewards_metrics_superset_and_step_wise_merge(tmp_path):
    from skyrl_b200.train.generators.base import TrajectoryID

    pdist.reset_env_for_tests()
    tr = PPOTrainer(_cfg(tmp_path, ["generator.n_samples_per_prompt=1"]), tokenizer=SyntheticTokenizer(1024))
    go = {"prompt_token_ids": [[1, 2], [3, 4]], "response_ids": [[5, 6], [7, 8, 9]], "rewards": [1.0, 0.5],
          "loss_masks": [[1, 1], [1, 1, 1]], "stop_reasons": ["stop", "stop"], "rollout_metrics": None}
    out, uids = tr.postprocess_generator_output(go, ["u1", "u2"])
    assert uids == ["u1", "u2"] and out["rewards"] == [[0.0, 1.0], [0.0, 0.0, 0.5]]
    tok = {"prompt_token_ids": [[1, 2]], "response_ids": [[3, 4, 5]], "rewards": [[0.1, 0.2, 0.3]],
           "loss_masks": [[1, 1, 1]], "stop_reasons": ["stop"], "rollout_metrics": None}
    assert tr.postprocess_generator_output(tok, ["u1"])[0]["rewards"] == [[0.1, 0.2, 0.3]]
    # reward metrics over a superset of the trained rows (groups the fully-async trainer dropped)
    kept = {"prompt_token_ids": [[1]], "response_ids": [[3, 4]], "rewards": [1.0], "loss_masks": [[1, 1]],
            "stop_reasons": ["stop"], "rollout_metrics": None}
    union = {"prompt_token_ids": [[1]] * 3, "response_ids": [[3, 4], [5], [6]], "rewards": [1.0, 0.0, 0.0],
             "loss_masks": [[1, 1], [1], [1]], "stop_reasons": ["stop"] * 3, "rollout_metrics": None}
    tr.all_metrics = {}
    out, _ = tr.postprocess_generator_output(kept, ["u1"], metrics_generator_output=union, metrics_uids=["u1", "u2", "u3"])
    assert out["rewards"] == [[0.0, 1.0]]
    assert tr.all_metrics["reward/avg_raw_reward"] == pytest.approx(1 / 3)
    assert tr.all_metrics["reward/avg_pass_at_1"] == pytest.approx(1 / 3)

    # step-wise rows: metrics from the last step of each trajectory; merging folds steps whose prompt extends the
    # previous step's tokens and shortens the uid list with them
    pdist.reset_env_for_tests()
    sw = PPOTrainer(_cfg(tmp_path, ["generator.n_samples_per_prompt=1", "generator.batched=false",
                                    "generator.step_wise_trajectories=true", "generator.merge_stepwise_output=true"]),
                    tokenizer=SyntheticTokenizer(1024))
    t = [TrajectoryID("a", 0), TrajectoryID("a", 0), TrajectoryID("b", 0)]
    steps = {"prompt_token_ids": [[1, 2], [1, 2, 5, 6, 40], [3]], "response_ids": [[5, 6], [7], [9, 9]],
             "rewards": [[0.0, 0.25], [1.0], [0.0, 0.0]], "loss_masks": [[1, 1], [1], [1, 1]],
             "stop_reasons": ["stop"] * 3, "rollout_metrics": None, "rollout_logprobs": None, "trajectory_ids": t,
             "is_last_step": [False, True, True]}
    sw.all_metrics = {}
    out, uids = sw.postprocess_generator_output(steps, ["a", "a", "b"])
    assert uids == ["a", "b"] and out["response_ids"] == [[5, 6, 40, 7], [9, 9]]
    assert out["loss_masks"] == [[1, 1, 0, 1], [1, 1]] and out["rewards"] == [[0.0, 0.25, 0.0, 1.0], [0.0, 0.0]]
    assert sw.all_metrics["generate/num_seq_before_merge"] == 3 and sw.all_metrics["generate/num_seq_after_merge"] == 2
    assert sw.all_metrics["reward/avg_raw_reward"] == pytest.approx(0.5)  # last steps only: (1.0 + 0.0) / 2


def test_step_wise_advantages_follow_each_steps_own_mask(tmp_path):
    """Intermediate and last steps have different response lengths, so their masks end at different columns: each
    step gets its trajectory's advantage on its *own* mask (the reference's regression test for its issue 1492)."""
    from skyrl_b200.train.batch import TrainingInputBatch

    pdist.reset_env_for_tests()
    tr = PPOTrainer(_cfg(tmp_path, ["generator.step_wise_trajectories=true", "generator.batched=false",
                                    "trainer.algorithm.grpo_norm_by_std=false"]), tokenizer=SyntheticTokenizer(1024))
    rm = torch.tensor([[0, 0, 1, 1, 1, 1], [0, 0, 0, 0, 0, 1], [0, 0, 0, 1, 1, 1], [0, 0, 0, 0, 1, 1]])
    rew = torch.zeros(4, 6)
    rew[1, -1] = 2.0
    d = TrainingInputBatch({"sequences": torch.zeros(4, 6, dtype=torch.long), "attention_mask": torch.ones(4, 6, dtype=torch.long),
                            "loss_mask": rm.float(), "response_mask": rm, "rewards": rew})
    d.metadata = {"uids": ["g"] * 4, "response_length": 6, "is_last_step": [False, True, False, True]}
    tr.all_metrics = {}
    out = tr.compute_advantages_and_returns(d)
    want = torch.tensor([[0, 0, 1, 1, 1, 1], [0, 0, 0, 0, 0, 1], [0, 0, 0, -1, -1, -1], [0, 0, 0, 0, -1, -1]], dtype=torch.float32)
    assert torch.allclose(out["advantages"], want) and torch.allclose(out["returns"], want)


def test_mtp_enabled_trainer_drafts_with_the_head_it_trains(tmp_path):
    """trainer.mtp.enabled: the colocated engine speculates with the policy worker's own draft head (no copy, so no
    reload after an update); the rollout log-probs still agree with the training pass."""
    pdist.reset_env_for_tests()
    tr = PPOTrainer(_cfg(tmp_path, ["trainer.mtp.enabled=true"]), tokenizer=SyntheticTokenizer(1024))
    tr.build_models()
    assert tr.engine.draft_head is tr.policy.mtp_head and tr.engine.cfg.num_speculative_tokens == 1
    m = tr.train_step(_prompts())
    em = tr.engine.metrics()
    assert em["spec_drafted"] > 0 and 0.0 <= em["spec_acceptance_rate"] <= 1.0
    assert m["policy/rollout_train_logprobs_abs_diff_mean"] < 1e-4 and m["policy/grad_norm"] > 0
    assert 8 * 4 * 16 < m["trainer/num_generated_tokens"] <= 8 * 4 * 32
    # switched off: the head is still trained, the engine decodes plainly
    pdist.reset_env_for_tests()
    tr2 = PPOTrainer(_cfg(tmp_path, ["trainer.mtp.enabled=true", "trainer.b200.speculative_decode=false"]),
                     tokenizer=SyntheticTokenizer(1024))
    tr2.build_models()
    assert tr2.engine.draft_head is None and tr2.policy.mtp_head is not None


class _Recorder:
    """Records every event with the fields that were set, and asks for a save + stop after the second step."""

    def __init__(self):
        from skyrl_b200.train.callbacks import EVENTS

        self.events = []
        for name in EVENTS:
            setattr(self, name, self._make(name))

    def _make(self, name):
        def handler(trainer, ci, control):
            self.events.append((name, ci.global_step, ci.epoch, sorted(k for k in ("batch", "metrics", "logs", "ckpt_path")
                                                                         if getattr(ci, k) is not None)))
            if name == "on_log":
                ci.logs["custom/from_callback"] = 1.0
            if name == "on_step_end" and ci.global_step == 2:
                control.should_save = True
                control.should_stop = True

        return handler


def test_rl_training_loop_fires_callbacks_in_order_and_honours_control(tmp_path):
    import pandas as pd

    from skyrl_b200.train.dataset import PromptDataset

    pdist.reset_env_for_tests()
    rows = [{"prompt": [{"role": "user", "content": f"{10 + i} {20 + i}"}], "env_class": "synthetic_even", "uid": f"q{i}"}
            for i in range(16)]
    path = str(tmp_path / "train.parquet")
    pd.DataFrame(rows).to_parquet(path)
    cfg = _cfg(tmp_path, ["trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4", "generator.n_samples_per_prompt=2",
                          "trainer.epochs=3", "trainer.eval_interval=0", "trainer.eval_before_train=false",
                          "trainer.ckpt_interval=0", "trainer.hf_save_interval=0", "generator.sampling_params.max_generate_length=8"])
    tok = SyntheticTokenizer(1024)
    logged = []

    class Tracker:
        def log(self, metrics, step):
            logged.append((step, dict(metrics)))

        def finish(self):
            pass

    tr = PPOTrainer(cfg, tracker=Tracker(), tokenizer=tok, train_dataset=PromptDataset([path], tok, 64))
    rec = _Recorder()
    tr.callbacks.add(rec)
    tr.build_models()
    tr.train()
    names = [e[0] for e in rec.events]
    assert names == ["on_train_start", "on_epoch_start",
                     "on_step_start", "on_step_end", "on_log",
                     "on_step_start", "on_step_end", "on_log", "on_save",   # the callback asked for a checkpoint and a stop
                     "on_epoch_end", "on_train_end"]
    by = {(n, s): f for n, s, _, f in rec.events}
    assert by[("on_step_start", 0)] == ["batch"] and by[("on_step_end", 1)] == ["batch", "metrics"]
    assert by[("on_log", 2)] == ["logs"] and by[("on_save", 2)] == ["ckpt_path"]
    assert tr.global_step == 2 and os.path.isdir(os.path.join(cfg.trainer.ckpt_path, "global_step_2"))
    assert [s for s, _ in logged] == [1, 2] and all(m["custom/from_callback"] == 1.0 for _, m in logged)
    assert tr.total_steps == 12 and tr.steps_per_epoch == 4


def test_dispatch_facade_offers_the_reference_worker_verbs(tmp_path):
    import asyncio

    pdist.reset_env_for_tests()
    tr = PPOTrainer(_cfg(tmp_path), tokenizer=SyntheticTokenizer(1024))
    tr.build_models()
    d = tr.dispatch
    assert d.has("policy") and d.has("ref") and not d.has("critic") and d.dp_size("policy") == 1 and d.get_lcm_dp_size() == 1
    tr.train_step(_prompts())
    batch = tr._last_batch
    lp = d.forward("policy", batch)["output"]
    assert lp.shape == batch["response_mask"].shape
    w0 = tr.policy.model.flat_params.clone()
    d.set_lr("policy", 1e-4)
    assert tr.policy.get_lr() == 1e-4
    st = d.forward_backward("policy", batch, loss_fn="regular", loss_fn_config={"eps_clip_low": 0.1})
    assert "final_loss" in st and d.optim_step("policy") is not None and not torch.equal(w0, tr.policy.model.flat_params)
    v = tr.engine.weight_version
    tr.init_weight_sync_state()
    asyncio.run(d.save_weights_for_sampler())
    assert tr.engine.weight_version == v + 1
    d.set_algorithm_config("policy", eps_clip_high=0.3)
    assert tr.policy.cfg.algorithm.eps_clip_high == 0.3
    d.save_checkpoint("policy", str(tmp_path / "p"))
    d.load_checkpoint("policy", str(tmp_path / "p"))
    with pytest.raises(ValueError, match="no 'critic' worker"):
        d.forward("critic", batch)
    with pytest.raises(ValueError, match="unknown model role"):
        d.optim_step("reward")
