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
    # rollouts through the OpenAI-compatible endpoint of the colocated engine
    ("examples/train_integrations/openai_chat/run_chat_grpo.sh", []),
    # a draft head trained beside the policy, used by the engine for speculative decoding
    ("examples/spec_decode/run_mtp_spec_decode.sh", []),
    # REPL environment whose code may query the policy; the generator injects the callbacks
    ("examples/rlm/run_rlm_recursive.sh", ["generator.max_turns=2", "generator.max_input_length=512",
                                           "environment.skyrl_gym.max_env_workers=4"]),
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
    if "rlm" in script:  # rows with a context document for the REPL
        import pandas as pd

        rows = [{"prompt": [{"role": "user", "content": f"which number follows {i} ?"}], "env_class": "rlm",
                 "context": f"the number after {i} is {i + 1}", "reward_spec": {"method": "contains", "ground_truth": str(i + 1)},
                 "uid": f"r{i}"} for i in range(16)]
        pd.DataFrame(rows).to_parquet(os.path.join(data, "train.parquet"))
        pd.DataFrame(rows[:4]).to_parquet(os.path.join(data, "validation.parquet"))
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


def test_full_context_and_collective_check_examples_run(tmp_path):
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2", HOME=str(tmp_path), MODEL="tiny-llama",
               NGPU="1")
    p = subprocess.run(["bash", os.path.join(ROOT, "examples/train_scripts/full_context/run_full_ctx.sh"),
                        "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4", "generator.n_samples_per_prompt=2",
                        "trainer.max_prompt_length=24", "generator.sampling_params.max_generate_length=8",
                        "trainer.max_tokens_per_microbatch=512", "trainer.bf16=false", "num_dummy_steps=2",
                        f"trainer.ckpt_path={tmp_path}/ckpt", f"trainer.export_path={tmp_path}/export"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert "step 2/2: 8 rows x 40 tokens" in p.stdout
    p = subprocess.run(["python", "-m", "torch.distributed.run", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29689", os.path.join(ROOT, "examples/train_scripts/nccl_test.py"), "--mib", "0.5",
                        "--iters", "2"], cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "GLOO_TEST_OK" in p.stdout, p.stdout[-1500:] + p.stderr[-1500:]


def test_tinker_grpo_client_and_session_routing_examples(tmp_path):
    import asyncio

    import torch
    from fastapi.testclient import TestClient

    from examples.tinker.ppo.grpo_client import grpo_datum, run
    from examples.tinker.session_based_routing.route_by_session import converse
    from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_b200.inference.local_client import LocalInferenceClient
    from skyrl_b200.inference.remote_client import RemoteInferenceClient
    from skyrl_b200.inference.server import ServerThread, build_app as build_server
    from skyrl_b200.models.decoder import CausalLM, PRESETS
    from skyrl_b200.parallel.dist import get_env
    from skyrl_b200.tinker.api import build_app
    from skyrl_b200.tinker.backend import SkyRLTrainBackend
    from skyrl_b200.utils.tokenizer import SyntheticTokenizer

    d = grpo_datum([1, 2, 3], [4, 5], [-0.1, -0.2], 0.5)
    li = d["loss_fn_inputs"]
    assert d["model_input"]["chunks"][0]["tokens"] == [1, 2, 3, 4] and li["target_tokens"]["data"] == [2, 3, 4, 5]
    assert li["weights"]["data"] == [0.0, 0.0, 1.0, 1.0] and li["advantages"]["data"] == [0.0, 0.0, 0.5, 0.5]

    tok = SyntheticTokenizer(1024)
    ov = {"trainer.bf16": "false", "generator.inference_engine.max_num_seqs": 16, "trainer.max_prompt_length": 32,
          "generator.sampling_params.max_generate_length": 16, "generator.inference_engine.enforce_eager": "true",
          "generator.inference_engine.engine_init_kwargs": "{num_blocks: 128}", "trainer.gradient_checkpointing": "false"}
    app = build_app(lambda base: SkyRLTrainBackend(base, ov, env=get_env(), tokenizer=tok, checkpoints_base=str(tmp_path)),
                    supported_models=["tiny-llama"], poll_interval=0.01)
    with TestClient(app) as c:
        def call(path, body):
            r = c.post(path, json=body)
            assert r.status_code == 200, (path, r.text)
            return r.json()

        rewards = run(call, "tiny-llama", [[10 + i, 20, 30] for i in range(3)], steps=2, group=4, max_tokens=8, lr=1e-4)
    assert len(rewards) == 2 and all(0.0 <= r <= 1.0 for r in rewards)

    # two servers: every conversation stays on one of them and its turns extend one another
    servers, engines = [], []
    for s in range(2):
        torch.manual_seed(s)
        eng = LLMEngine(CausalLM(PRESETS["tiny-llama"], dtype=torch.float32, device="cpu", seed=s),
                        EngineConfig(block_size=16, max_num_seqs=8, max_model_len=128, num_blocks=64, enforce_eager=True))
        engines.append(eng)
        servers.append(ServerThread(build_server(LocalInferenceClient([eng], tok))).start())
    try:
        async def go():
            async with RemoteInferenceClient([s.url for s in servers]) as rc:
                return await converse(rc, sessions=4, turns=2, max_tokens=4)

        out = asyncio.run(go())
        assert sorted(out) == [f"conv-{i}" for i in range(4)] and all(len(t) == 2 for t in out.values())
        assert sum(e.stats["prefill_calls"] > 0 for e in engines) >= 1
    finally:
        for s in servers:
            s.stop()
