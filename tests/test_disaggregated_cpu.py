"""Disaggregated placement inside one launch: training ranks and rollout-only ranks split from the same process set
(``trainer.placement.colocate_all=false``), requests over HTTP, weights published to the servers after every update."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _data(d):
    import pandas as pd

    os.makedirs(d, exist_ok=True)
    rows = [{"prompt": [{"role": "user", "content": f"what is {i} plus {i} ?"}], "env_class": "synthetic_bernoulli",
             "uid": f"q{i}"} for i in range(32)]
    pd.DataFrame(rows).to_parquet(os.path.join(d, "train.parquet"))
    return os.path.join(d, "train.parquet")


def _launch(tmp, nproc, port, extra):
    path = _data(str(tmp / "data"))
    args = ["trainer.policy.model.path=tiny-llama", f'data.train_data=["{path}"]', "environment.env_class=synthetic_bernoulli",
            "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4", "generator.n_samples_per_prompt=2",
            "trainer.max_prompt_length=64", "generator.sampling_params.max_generate_length=8", "trainer.bf16=false",
            "trainer.gradient_checkpointing=false", "trainer.max_training_steps=2", "trainer.epochs=1",
            "trainer.eval_interval=0", "trainer.ckpt_interval=0", "trainer.hf_save_interval=0",
            "generator.inference_engine.enforce_eager=true", "generator.inference_engine.max_num_seqs=16",
            "trainer.resume_mode=none", "trainer.logger=console", "trainer.algorithm.use_kl_loss=false",
            "trainer.placement.colocate_all=false", f"trainer.ckpt_path={tmp}/ckpt", f"trainer.export_path={tmp}/export",
            *extra]
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "skyrl_b200.launch", "--nproc-per-node", str(nproc), "--master-port", str(port), "-m",
           "skyrl_b200.entrypoints.main_base", *args]
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)


def test_one_training_rank_and_one_rollout_rank(tmp_path):
    p = _launch(tmp_path, 2, 29881, ["trainer.placement.policy_num_gpus_per_node=1", "generator.inference_engine.num_engines=1"])
    out = p.stdout + p.stderr
    assert p.returncode == 0, out[-3000:]
    assert "[step 2]" in out and '"server_url"' in out
    # the rollout server generated with the weights the trainer published: log-probs agree with the trainer's own
    assert "policy/rollout_train_logprobs_abs_diff_mean=" in out


def test_two_training_ranks_and_two_rollout_ranks_fully_async(tmp_path):
    p = _launch(tmp_path, 4, 29885, ["trainer.placement.policy_num_gpus_per_node=2", "generator.inference_engine.num_engines=2",
                                     "trainer.fully_async.enabled=true", "trainer.fully_async.max_staleness_steps=1",
                                     "trainer.fully_async.num_parallel_generation_workers=4",
                                     "trainer.algorithm.policy_loss_type=rollout_is"])
    out = p.stdout + p.stderr
    assert p.returncode == 0, out[-3000:]
    assert "trainer/global_step=2" in out and "async/staleness_max" in out


def test_placement_must_add_up(tmp_path):
    p = _launch(tmp_path, 2, 29889, ["trainer.placement.policy_num_gpus_per_node=2", "generator.inference_engine.num_engines=1"])
    assert p.returncode != 0 and "== world size" in (p.stdout + p.stderr)
