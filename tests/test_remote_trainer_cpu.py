"""GRPO with the RL loop on the client and the model behind the Tinker-compatible REST service (in-process, CPU)."""
import torch

from skyrl_b200.config.config import SkyRLTrainConfig
from skyrl_b200.integrations.remote_trainer import (RemoteBackendTrainer, TrainingServiceClient, batch_to_datums)
from skyrl_b200.parallel import dist as pdist
from skyrl_b200.train.batch import TrainingInputBatch
from skyrl_b200.utils.tokenizer import SyntheticTokenizer


def test_batch_to_datums_strips_padding_and_zeroes_the_prompt():
    seq = torch.tensor([[0, 0, 5, 6, 7, 8, 9, 0], [1, 2, 3, 4, 5, 6, 7, 8]])
    att = torch.tensor([[0, 0, 1, 1, 1, 1, 1, 0], [1, 1, 1, 1, 1, 1, 1, 1]])
    rm = torch.tensor([[1, 1, 0], [1, 1, 1]])
    b = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rm,
                            "loss_mask": torch.tensor([[1.0, 0.0, 0.0], [1.0, 1.0, 1.0]]),
                            "action_log_probs": torch.tensor([[-0.1, -0.2, 0.0], [-0.3, -0.4, -0.5]]),
                            "advantages": torch.tensor([[1.0, 1.0, 0.0], [2.0, 2.0, 2.0]])})
    d = batch_to_datums(b)
    assert d[0]["model_input"]["chunks"][0]["tokens"] == [5, 6, 7, 8]
    assert d[0]["loss_fn_inputs"]["target_tokens"]["data"] == [6, 7, 8, 9]
    assert d[0]["loss_fn_inputs"]["weights"]["data"] == [0.0, 0.0, 1.0, 0.0]
    assert d[0]["loss_fn_inputs"]["logprobs"]["data"] == [0.0, 0.0, torch.tensor(-0.1).item(), torch.tensor(-0.2).item()]
    assert d[1]["loss_fn_inputs"]["advantages"]["data"] == [0.0] * 4 + [2.0] * 3


def test_grpo_steps_through_the_service(tmp_path):
    from fastapi.testclient import TestClient

    from skyrl_b200.parallel.dist import get_env
    from skyrl_b200.tinker.api import build_app
    from skyrl_b200.tinker.backend import SkyRLTrainBackend

    pdist.reset_env_for_tests()
    tok = SyntheticTokenizer(1024)
    ov = {"trainer.bf16": "false", "trainer.policy.optimizer_config.num_warmup_steps": 0,
          "generator.inference_engine.max_num_seqs": 16, "generator.sampling_params.max_generate_length": 16,
          "trainer.max_prompt_length": 64, "generator.inference_engine.enforce_eager": "true",
          "trainer.micro_train_batch_size_per_gpu": 8, "trainer.algorithm.use_kl_loss": "false",
          "generator.inference_engine.engine_init_kwargs": "{num_blocks: 128}"}
    factory = lambda base: SkyRLTrainBackend(base, ov, env=get_env(), tokenizer=tok, checkpoints_base=str(tmp_path / "svc"))
    app = build_app(factory, supported_models=["tiny-llama"], poll_interval=0.01)
    cfg = SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model.path=tiny-llama", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=2",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=12",
        "generator.sampling_params.temperature=1.0", "trainer.max_prompt_length=32", "trainer.algorithm.use_kl_loss=false",
        "trainer.policy.optimizer_config.lr=1e-3", "environment.env_class=synthetic_even", "generator.batched=true",
        "trainer.seed=0", f"trainer.ckpt_path={tmp_path}/ckpt", "trainer.resume_mode=none"])
    g = torch.Generator().manual_seed(0)
    prompts = []
    for i in range(4):
        ids = torch.randint(4, 1024, (16,), generator=g).tolist()
        prompts.append({"prompt": [{"role": "user", "content": ids}], "prompt_token_ids": ids, "uid": f"p{i}"})
    with TestClient(app) as c:
        client = TrainingServiceClient(transport=c, poll_interval=0.01)
        tr = RemoteBackendTrainer(cfg, client, tokenizer=tok)
        tr.build_models()
        assert client.model_id is not None
        first = client.sampling_session_id
        m = tr.train_step(prompts)
        assert m["trainer/global_step"] == 1.0 and 4 * 2 <= m["trainer/num_generated_tokens"] <= 4 * 2 * 12
        # two mini-batches -> two optimizer steps on the service; old log-probs came from the service's forward and
        # agree with what its sampler reported
        assert m["policy/rollout_train_logprobs_abs_diff_mean"] < 1e-3
        assert m["policy/grad_norm"] > 0
        assert client.sampling_session_id is not None and client.sampling_session_id != first
        probe = batch_to_datums(tr._last_batch, with_loss_inputs=False)[:2]
        before = client.forward(probe)["loss_fn_outputs"][0]["logprobs"]["data"]
        m2 = tr.train_step(prompts)
        after = client.forward(probe)["loss_fn_outputs"][0]["logprobs"]["data"]
        assert m2["trainer/global_step"] == 2.0 and before != after  # the second step moved the service's weights
        tr.save_checkpoints()
        saved = client.forward(probe)["loss_fn_outputs"][0]["logprobs"]["data"]
        tr.train_step(prompts)
        assert client.forward(probe)["loss_fn_outputs"][0]["logprobs"]["data"] != saved
        tr.policy.load_checkpoint(str(tmp_path / "ckpt" / "global_step_2" / "policy"))
        restored = client.forward(probe)["loss_fn_outputs"][0]["logprobs"]["data"]
        assert max(abs(a - b) for a, b in zip(restored, saved)) < 1e-5
