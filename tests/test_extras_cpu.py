"""Wire packing, router replay, fake INT4 QAT, MTP soft cross-entropy, multi-tenant adapter store."""
import numpy as np
import pytest
import torch

from skyrl_b200.algorithms import mtp
from skyrl_b200.inference import wire
from skyrl_b200.models import qat, router_replay
from skyrl_b200.models.moe import moe_ffn


def test_wire_round_trip_and_rejections():
    c, n = wire.build_logprobs_content([-0.5, None, float("nan"), float("-inf")])
    assert n == 3 and c[1]["logprob"] == wire.CLAMPED_LOGPROB and c[0]["logprob"] == -0.5
    a = np.random.default_rng(0).integers(0, 128, size=(5, 3, 8))
    p = wire.pack_routed_experts(a)
    assert p["dtype"] == "uint8" and np.array_equal(wire.decode_packed_routed_experts(p), a)
    assert wire.pack_routed_experts(a + 300)["dtype"] == "uint16"
    with pytest.raises(TypeError):
        wire.pack_routed_experts(a.tolist())
    bad = dict(p, shape=[5, 3])
    with pytest.raises(ValueError):
        wire.decode_packed_routed_experts(bad)
    with pytest.raises(ValueError):
        wire.decode_packed_routed_experts(dict(p, dtype="int32"))  # wrong byte count for the claimed dtype


def test_router_replay_forces_recorded_experts():
    torch.manual_seed(0)
    T, H, E, F, k = 12, 16, 6, 8, 2
    h = torch.randn(T, H)
    router = torch.randn(E, H)
    wgu, wd = torch.randn(E, 2 * F, H) * 0.1, torch.randn(E, H, F) * 0.1
    with router_replay.record_routing() as store:
        y0 = moe_ffn(h, router, wgu, wd, k, layer=0)
    idx = router_replay.stack_recorded(store)
    assert idx.shape == (T, 1, k)
    h2 = h + 0.8 * torch.randn(T, H)  # perturbed activations would route differently on their own
    free = moe_ffn(h2, router, wgu, wd, k, layer=0)
    with router_replay.replay_routing(idx):
        forced = moe_ffn(h2, router, wgu, wd, k, layer=0)
    manual = moe_ffn(h2, router, wgu, wd, k, routed_indices=idx[:, 0])
    assert torch.allclose(forced, manual) and not torch.allclose(forced, free)
    with router_replay.replay_routing(idx):
        assert torch.allclose(moe_ffn(h, router, wgu, wd, k, layer=0), y0, atol=1e-6)
    al = router_replay.align_to_packed([idx[:4], idx[4:7]], [5, 3])
    assert al.shape[0] == 8 and torch.equal(al[4], idx[3])


def test_fake_int4_levels_and_straight_through():
    w = torch.randn(8, 64, requires_grad=True)
    q = qat.fake_int4(w, 32)
    lv = (q.detach().reshape(8, 2, 32) / (w.detach().reshape(8, 2, 32).abs().amax(-1, keepdim=True) / 7)).round()
    assert lv.abs().max() <= 7 and torch.unique(lv).numel() <= 15
    q.sum().backward()
    assert torch.equal(w.grad, torch.ones_like(w))
    assert 0 < qat.quantization_error(w.detach()) < 0.2
    with pytest.raises(ValueError):
        qat.fake_int4_quant_dequant(torch.randn(4, 30))


def test_mtp_soft_ce_trains_draft_head_only():
    torch.manual_seed(0)
    T, H, V = 40, 16, 50
    hidden = torch.randn(T, H, requires_grad=True)
    lm = torch.randn(V, H, requires_grad=True)
    cu = torch.tensor([0, 15, 40])
    head = mtp.DraftHead(H)
    same = mtp.soft_cross_entropy(torch.randn(5, V), torch.randn(5, V))
    assert same > 0
    loss0 = mtp.mtp_draft_loss(head, hidden, lm, cu)
    loss0.backward()
    assert hidden.grad is None and lm.grad is None  # trunk and LM head are detached from the draft loss
    assert head.down.weight.grad.abs().sum() > 0
    norm, coef = mtp.clip_grad_norm_separately(head.parameters(), 1e-3)
    assert coef < 1.0 and norm > 0
    opt = torch.optim.Adam(head.parameters(), lr=3e-2)
    for _ in range(60):
        opt.zero_grad()
        l = mtp.mtp_draft_loss(head, hidden, lm, cu)
        l.backward()
        opt.step()
    assert float(l) < float(loss0)


def test_adapter_store_swaps_tenants():
    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.parallel.dist import get_env
    from skyrl_b200.workers.adapter_store import AdapterStore
    from skyrl_b200.workers.worker import PolicyWorker

    cfg = SkyRLTrainConfig.from_cli_overrides(["trainer.policy.model.path=tiny-llama", "trainer.policy.model.lora.rank=4",
                                               "trainer.bf16=false"])
    w = PolicyWorker(cfg.trainer, model_path="tiny-llama", env=get_env(), seed=0)
    store = AdapterStore(w, max_slots=2)
    store.create("a", seed=1)
    w.model.flat_params.add_(1.0)
    w.optimizer.exp_avg.fill_(0.5)
    w.optimizer.step_count = 7
    pa = w.model.flat_params.clone()
    store.create("b", seed=2)
    assert w.optimizer.step_count == 0 and w.optimizer.exp_avg.abs().sum() == 0
    assert not torch.equal(w.model.flat_params, pa)
    pb = w.model.flat_params.clone()
    store.swap_to("a")
    assert torch.equal(w.model.flat_params, pa) and w.optimizer.step_count == 7 and float(w.optimizer.exp_avg[0]) == 0.5
    store.swap_to("b")
    assert torch.equal(w.model.flat_params, pb)
    with pytest.raises(RuntimeError):
        store.create("c")


def test_numa_pinning_reads_sysfs_topology(tmp_path):
    from skyrl_b200.utils import numa

    assert numa.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    root = tmp_path / "sys"
    dev = root / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = root / "devices" / "system" / "node" / "node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("16-19,48\n")
    assert numa.gpu_numa_node("0000:1B:00.0", str(root)) == 1
    applied = {}
    cpus = numa.pin_to_gpu_numa_node(0, str(root), bus_id="0000:1b:00.0", setaffinity=lambda pid, s: applied.update(pid=pid, cpus=s))
    assert cpus == [16, 17, 18, 19, 48] and applied == {"pid": 0, "cpus": {16, 17, 18, 19, 48}}
    # unknown device or node -1: nothing is changed
    (dev / "numa_node").write_text("-1\n")
    assert numa.pin_to_gpu_numa_node(0, str(root), bus_id="0000:1b:00.0", setaffinity=lambda *a: applied.update(bad=1)) == []
    assert numa.pin_to_gpu_numa_node(0, str(root), bus_id="0000:ff:00.0", setaffinity=lambda *a: applied.update(bad=1)) == []
    assert "bad" not in applied


def test_env_var_registry_lists_every_variable_the_code_reads():
    import os
    import re

    from skyrl_b200 import env_vars

    names = {r["name"] for r in env_vars.describe()}
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    found = set()
    for dirpath, _, files in os.walk(os.path.join(root, "skyrl_b200")):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cpp", ".h", ".cuh")) and fn != "env_vars.py":
                text = open(os.path.join(dirpath, fn), errors="ignore").read()
                found |= set(re.findall(r'(?:environ\.get|getenv)\(\s*"((?:SB|SKYRL)_[A-Z0-9_]+)"', text))
    assert found <= names, sorted(found - names)
    assert env_vars.get("SB_PDL") is True and isinstance(env_vars.SKYRL_WORKER_NCCL_TIMEOUT_IN_S, int)


def test_debug_bounds_mode_rejects_bad_indices_before_the_kernel(monkeypatch):
    """SKYRL_B200_DEBUG_BOUNDS=1 stands in for a memory checker: an index outside its table raises at the op boundary."""
    import pytest
    import torch

    from skyrl_b200.ops import _lib, attention, sampling

    table = torch.randn(16, 8)
    kc, vc = torch.zeros(4, 2, 1, 8), torch.zeros(4, 2, 1, 8)
    qkv = torch.randn(3, 3 * 8)
    # off: the CPU reference paths index as usual (a bad id fails inside torch, a negative slot means "skip")
    assert sampling.embed(table, torch.tensor([0, 15])).shape == (2, 8)
    monkeypatch.setenv("SKYRL_B200_DEBUG_BOUNDS", "1")
    assert _lib.debug_bounds()
    with pytest.raises(_lib.IndexOutOfRange, match="token id"):
        sampling.embed(table, torch.tensor([0, 16]))
    with pytest.raises(_lib.IndexOutOfRange, match="cache slot"):
        attention.kv_cache_write(qkv, kc, vc, torch.tensor([0, 8, -1]), 1, 1, 8)
    attention.kv_cache_write(qkv, kc, vc, torch.tensor([0, 7, -1]), 1, 1, 8)  # -1 = skip is legal
    bt = torch.tensor([[0, 3], [1, 9]], dtype=torch.int32)
    with pytest.raises(_lib.IndexOutOfRange, match="block table"):
        attention.attn_decode_paged(qkv[:2], kc, vc, bt, torch.tensor([2, 4], dtype=torch.int32), 1, 1, 8)
    # the bad entry is beyond what the second sequence's context reaches: not read, not an error
    attention.attn_decode_paged(qkv[:2], kc, vc, bt, torch.tensor([2, 2], dtype=torch.int32), 1, 1, 8)


def test_mtp_draft_head_trains_beside_the_policy_without_touching_it(tmp_path):
    """trainer.mtp.enabled: a draft head learns the trunk's next-next-token distribution on detached trunk states with
    its own optimizer; the policy update is bit-identical to a run without it."""
    import torch

    from skyrl_b200.algorithms.mtp import DraftHead, mtp_draft_backward, mtp_draft_loss
    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.parallel import dist as pdist
    from skyrl_b200.train.batch import TrainingInputBatch
    from skyrl_b200.workers.worker import PolicyWorker

    # the chunked backward computes the same loss and gradients as the one-shot loss
    torch.manual_seed(0)
    head = DraftHead(16)
    with torch.no_grad():
        head.down.weight.normal_(0, 0.1)
    h, W = torch.randn(23, 16), torch.randn(50, 16)
    cu = torch.tensor([0, 9, 23])
    mask = torch.rand(23) > 0.3
    ref = mtp_draft_loss(head, h, W, cu, mask)
    ref.backward()
    g_ref = [p.grad.clone() for p in head.parameters()]
    head.zero_grad()
    got = mtp_draft_backward(head, h, W, cu, mask, chunk=5)
    assert abs(float(got) - float(ref)) < 1e-5
    for a, b in zip(g_ref, [p.grad for p in head.parameters()]):
        assert torch.allclose(a, b, atol=1e-5)

    def cfg(mtp):
        return SkyRLTrainConfig.from_cli_overrides([
            "trainer.policy.model.path=tiny-llama", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4",
            "trainer.micro_train_batch_size_per_gpu=2", "generator.n_samples_per_prompt=2", "trainer.bf16=false",
            "trainer.algorithm.use_kl_loss=false", "trainer.policy.optimizer_config.lr=1e-3",
            "trainer.gradient_checkpointing=false", "trainer.max_tokens_per_microbatch=0", "trainer.resume_mode=none",
            f"trainer.mtp.enabled={'true' if mtp else 'false'}", "trainer.mtp.loss_weight=1.0"])

    def batch():
        g = torch.Generator().manual_seed(5)
        B, P, R = 4, 8, 12
        rm = torch.ones(B, R)
        rm[1, -3:] = 0
        att = torch.ones(B, P + R, dtype=torch.long)
        att[1, -3:] = 0
        return TrainingInputBatch({"sequences": torch.randint(4, 1024, (B, P + R), generator=g), "attention_mask": att,
                                   "response_mask": rm, "loss_mask": rm.clone(), "advantages": torch.randn(B, R, generator=g) * rm / rm.sum(),
                                   "action_log_probs": -torch.rand(B, R, generator=g), "rollout_logprobs": None,
                                   "base_action_log_probs": None})

    pdist.reset_env_for_tests()
    plain = PolicyWorker(cfg(False).trainer, model_path="tiny-llama", seed=0)
    plain.forward_backward(batch())
    plain.optim_step()
    pdist.reset_env_for_tests()
    w = PolicyWorker(cfg(True).trainer, model_path="tiny-llama", seed=0)
    before = [p.detach().clone() for p in w.mtp_head.parameters()]
    losses = []
    for _ in range(3):
        st = w.forward_backward(batch())
        w.optim_step()
        losses.append(st["mtp_loss"])
        if len(losses) == 1:
            assert torch.equal(w.model.flat_params, plain.model.flat_params)  # the draft loss never reaches the policy
    assert any(not torch.equal(a, b) for a, b in zip(before, w.mtp_head.parameters()))
    assert w.last_mtp["mtp_grad_norm"] > 0 and all(l == l and l > 0 for l in losses)
    w.save_checkpoint(str(tmp_path / "ck"))
    pdist.reset_env_for_tests()
    w2 = PolicyWorker(cfg(True).trainer, model_path="tiny-llama", seed=0)
    w2.load_checkpoint(str(tmp_path / "ck"))
    for a, b in zip(w.mtp_head.parameters(), w2.mtp_head.parameters()):
        assert torch.equal(a, b)


def test_config_overrides_from_dict_dotlist_round_trip_and_dataloader_rules():
    from skyrl_b200.config.config import ConfigError, SkyRLTrainConfig, _parse_scalar, overrides_dict_to_dotlist

    c = SkyRLTrainConfig.from_cli_overrides({"trainer.seed": 7, "generator.inference_engine.served_model_name": None,
                                             "trainer.run_name": "1e-5", "trainer.policy.optimizer_config.lr": 3e-6})
    assert c.trainer.seed == 7 and c.generator.inference_engine.served_model_name is None
    assert c.trainer.run_name == "1e-5" and c.trainer.policy.optimizer_config.lr == 3e-6
    for v in (None, True, False, 3, 1e-5, 2.5, "1e-5", "null", "true", [1, 2], {"a": [1, None]}, "plain text"):
        text = overrides_dict_to_dotlist({"k": v})[0]
        assert text.startswith("k=") and _parse_scalar(text[2:]) == v and type(_parse_scalar(text[2:])) is type(v)
    assert overrides_dict_to_dotlist({"a": 1, "b": 2}) == ["a=1", "b=2"]
    assert overrides_dict_to_dotlist({"k": object})[0].startswith("k=<class")
    assert _parse_scalar("1e-6") == 1e-6 and _parse_scalar("'1e-6'") == "1e-6"
    d = SkyRLTrainConfig.from_cli_overrides([]).data.dataloader
    assert d.num_workers == 8 and d.persistent_workers is False
    assert SkyRLTrainConfig.from_cli_overrides(["data.dataloader.num_workers=0"]).data.dataloader.num_workers == 0
    assert SkyRLTrainConfig.from_cli_overrides(["data.dataloader.persistent_workers=true"]).data.dataloader.num_workers == 8
    with pytest.raises(ConfigError, match="persistent_workers requires num_workers > 0"):
        SkyRLTrainConfig.from_cli_overrides(["data.dataloader.num_workers=0", "data.dataloader.persistent_workers=true"])
    with pytest.raises(ConfigError, match="num_workers must be None or >= 0"):
        SkyRLTrainConfig.from_cli_overrides(["data.dataloader.num_workers=-1"])
    for bad in (["+trainer.seed=1"], {"+trainer.seed": 1}):
        with pytest.raises(ConfigError, match="not supported"):
            SkyRLTrainConfig.from_cli_overrides(bad)


def test_torch_profiler_config_validation():
    from skyrl_b200.config.config import SkyRLTrainConfig, TorchProfilerConfig
    from skyrl_b200.train.utils import validate_cfg

    TorchProfilerConfig(enable=False, export_type="bogus", activities=["gpu"], ranks=[], active=0, save_path=None).validate()
    ok = lambda **kw: TorchProfilerConfig(enable=True, **{"save_path": "/tmp/prof", **kw})  # noqa: E731
    ok().validate()
    ok(activities=["CPU", "CUDA"]).validate()
    ok(export_type="stacks", with_stack=True).validate()
    for kw, match in (({"ranks": []}, "ranks.*non-empty"), ({"save_path": None}, "save_path.*must be set"),
                      ({"save_path": ""}, "save_path.*must be set"), ({"save_path": "s3://b/run"}, "save_path.*local path"),
                      ({"activities": ["cpu", "gpu"]}, "activities"), ({"activities": []}, "activities.*non-empty"),
                      ({"export_type": "bogus"}, "export_type"), ({"export_type": "stacks", "with_stack": False}, "with_stack"),
                      ({"skip_first": -1}, "skip_first"), ({"active": 0}, "active")):
        with pytest.raises(ValueError, match=match):
            ok(**kw).validate()
    cfg = SkyRLTrainConfig.from_cli_overrides(["trainer.policy.torch_profiler_config.enable=true",
                                               "trainer.policy.torch_profiler_config.save_path=/tmp/prof",
                                               "trainer.policy.torch_profiler_config.export_type=bogus",
                                               "trainer.policy.model.path=tiny-llama"])
    with pytest.raises(ValueError, match="export_type"):
        validate_cfg(cfg)


def test_validate_cfg_rejects_out_of_range_knobs():
    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.train.utils import validate_cfg

    base = ["trainer.policy.model.path=tiny-llama"]
    validate_cfg(SkyRLTrainConfig.from_cli_overrides(base))
    for extra, match in ((["trainer.max_training_steps=0"], "max_training_steps must be > 0"),
                         (["generator.sampling_params.logprobs=2"], "should be 0 or 1"),
                         (["generator.max_input_length=100", "trainer.max_prompt_length=512"], "must be at least"),
                         (["trainer.mtp.enabled=true", "trainer.mtp.num_speculative_tokens=0"], "num_speculative_tokens"),
                         (["trainer.update_epochs_per_batch=0"], "update_epochs_per_batch"),
                         (["generator.n_samples_per_prompt=0"], "n_samples_per_prompt")):
        with pytest.raises(ValueError, match=match):
            validate_cfg(SkyRLTrainConfig.from_cli_overrides(base + extra))
    validate_cfg(SkyRLTrainConfig.from_cli_overrides(base + ["generator.sampling_params.logprobs=null", "trainer.max_training_steps=3"]))


def test_validate_cfg_rejects_engine_layouts_the_engine_does_not_have():
    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.train.utils import validate_cfg

    base = ["trainer.policy.model.path=tiny-llama"]
    for extra, match in ((["generator.inference_engine.pipeline_parallel_size=2"], "pipeline_parallel_size"),
                         (["generator.inference_engine.expert_parallel_size=4"], "expert_parallel_size"),
                         (["generator.inference_engine.data_parallel_size=2"], "num_engines"),
                         (["generator.inference_engine.enable_pd=true"], "disaggregation")):
        with pytest.raises(ValueError, match=match):
            validate_cfg(SkyRLTrainConfig.from_cli_overrides(base + extra))
