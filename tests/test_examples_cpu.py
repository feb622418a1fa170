"""Every example launch script must only use configuration keys that exist."""
import glob
import os
import re

from skyrl_b200.config.config import SkyRLTrainConfig
from skyrl_b200.config.sft_config import SFTConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _overrides(path):
    out = []
    for line in open(path):
        line = line.strip().rstrip("\\").strip()
        if re.match(r"^[a-z_][a-z0-9_.]*=", line):
            line = re.sub(r"\$\{[A-Z_]+:-([^}]*)\}", r"\1", line)
            line = line.replace("$MODEL", "tiny-llama").replace("$DATA", "/tmp/d").replace("$HOME", "/tmp").replace("$NGPU", "1")
            out.append(line)
    return out


def test_example_scripts_parse():
    scripts = sorted(glob.glob(os.path.join(ROOT, "examples", "**", "*.sh"), recursive=True))
    assert len(scripts) >= 25
    for s in scripts:
        ov = _overrides(s)
        assert ov, s
        text = open(s).read()
        if "entrypoints.main_sft" in text or "main_sft_with_callbacks" in text:
            SFTConfig.from_cli_overrides(ov)
        else:
            SkyRLTrainConfig.from_cli_overrides(ov)


def test_custom_registrations_import():
    import importlib

    from skyrl_b200.algorithms import rl

    importlib.import_module("examples.algorithms.custom_advantage_estimator")
    importlib.import_module("examples.algorithms.custom_policy_loss")
    assert rl.AdvantageEstimatorRegistry.get("centered_reward") is not None
    assert rl.PolicyLossRegistry.get("capped_reinforce") is not None


# ----------------------------------------------------------------------------- executed, not only parsed
import json  # noqa: E402
import subprocess  # noqa: E402

import pytest  # noqa: E402


def _tiny_gsm8k(d):
    import pandas as pd

    rows = []
    for i in range(16):
        rows.append({"prompt": [{"role": "user", "content": f"what is {i} plus {i} ?"}], "env_class": "gsm8k",
                     "reward_spec": {"method": "rule", "ground_truth": str(2 * i)}, "uid": f"q{i}"})
    os.makedirs(d, exist_ok=True)
    pd.DataFrame(rows).to_parquet(os.path.join(d, "train.parquet"))
    pd.DataFrame(rows[:4]).to_parquet(os.path.join(d, "validation.parquet"))
    with open(os.path.join(d, "sft.jsonl"), "w") as f:
        for i in range(16):
            f.write(json.dumps({"messages": [{"role": "user", "content": f"say {i}"},
                                             {"role": "assistant", "content": f"{i} {i + 1} {i + 2}"}]}) + "\n")


_TINY_RL = ["trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4", "trainer.critic_mini_batch_size=4",
            "generator.n_samples_per_prompt=2", "trainer.max_prompt_length=64",
            "generator.sampling_params.max_generate_length=8", "trainer.max_tokens_per_microbatch=4096",
            "trainer.bf16=false", "trainer.gradient_checkpointing=false", "trainer.max_training_steps=1",
            "trainer.epochs=1", "trainer.eval_interval=0", "trainer.eval_before_train=false", "trainer.ckpt_interval=0",
            "trainer.hf_save_interval=0", "generator.inference_engine.enforce_eager=true",
            "generator.inference_engine.max_num_seqs=16", "trainer.resume_mode=none", "trainer.logger=console"]


@pytest.mark.parametrize("script,extra", [
    ("examples/gsm8k/run_gsm8k_grpo.sh", []),
    # all-zero rewards are never informative: the DAPO filter keeps sampling until it gives up after two batches
    ("examples/algorithms/run_dapo.sh", ["trainer.algorithm.dynamic_sampling.max_sample_batches=2"]),
    ("examples/ppo/run_ppo_gsm8k.sh", []),
    ("examples/sft/run_sft.sh", None),
    ("examples/callbacks/run_sft_with_callbacks.sh", None),
    ("examples/multiply/run_multiply.sh", ["environment.env_class=multiply"]),
    ("examples/on_policy_distillation/run_on_policy_distill.sh", []),
    ("examples/turn_level_rewards/run_gsm8k_multi_turn.sh", ["generator.max_input_length=256"]),
    ("examples/gptoss/run_attention_sinks_grpo.sh", ["trainer.policy.model.path=tiny-sinks"]),
])
def test_example_scripts_run_on_cpu(tmp_path, script, extra):
    """The launch scripts themselves are executed (bash, the launcher, the entry point) on a tiny preset and data."""
    path = os.path.join(ROOT, script)
    if not os.path.exists(path):
        alt = sorted(glob.glob(os.path.join(ROOT, os.path.dirname(script), "*.sh")))
        assert alt, script
        path = alt[0]
    data = str(tmp_path / "data")
    _tiny_gsm8k(data)
    if "multiply" in script:  # the example's own dataset writer
        gen = subprocess.run(["python", os.path.join(ROOT, "examples/multiply/multiply_dataset.py"), "--out", data, "--n", "32"],
                             cwd=ROOT, capture_output=True, text=True, timeout=120)
        assert gen.returncode == 0, gen.stderr[-1500:]
    env = dict(os.environ, MODEL="tiny-llama", TEACHER="tiny-llama", DATA=data, NGPU="1", HOME=str(tmp_path), PYTHONPATH=ROOT,
               CUDA_VISIBLE_DEVICES="", SFT_DATA=os.path.join(data, "sft.jsonl"), OMP_NUM_THREADS="2")
    if extra is None:  # SFT
        args = ["batch_size=4", "max_length=64", "max_tokens_per_microbatch=512", "num_steps=2", "bf16=false",
                f"ckpt_path={tmp_path}/ckpt", "ckpt_interval=0"]
    else:
        args = _TINY_RL + [f"trainer.ckpt_path={tmp_path}/ckpt", f"trainer.export_path={tmp_path}/export",
                           f"trainer.log_path={tmp_path}/logs"] + extra
    p = subprocess.run(["bash", path, *args], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    tail = p.stdout[-2500:] + p.stderr[-2500:]
    if script.endswith("run_dapo.sh"):
        assert p.returncode != 0 and "max_sample_batches" in tail, tail
    else:
        assert p.returncode == 0, tail
