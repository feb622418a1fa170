"""Tinker-compatible service on CPU: request store idempotency, look-ahead batching before barriers, the REST round
trip (create model -> forward_backward -> optim_step -> save/load -> sample) against a tiny model."""
import json
import time

import pytest
import torch

from skyrl_b200.tinker import db as tdb
from skyrl_b200.tinker import engine as teng
from skyrl_b200.tinker.backend import SkyRLTrainBackend, datums_to_batch
from skyrl_b200.utils.tokenizer import SyntheticTokenizer


def _datum(tokens, weights=None, **extra):
    L = len(tokens) - 1
    li = {"target_tokens": {"data": tokens[1:], "dtype": "int64", "shape": [L]},
          "weights": {"data": weights or [1.0] * L, "dtype": "float32", "shape": [L]}}
    for k, v in extra.items():
        li[k] = {"data": v, "dtype": "float32", "shape": [len(v)]}
    return {"model_input": {"chunks": [{"type": "encoded_text", "tokens": tokens[:-1]}]}, "loss_fn_inputs": li}


def test_future_idempotency_and_conflict():
    db = tdb.TinkerDB()
    a = db.create_future("forward_backward", "m", {"x": 1}, seq_id=7)
    assert db.create_future("forward_backward", "m", {"x": 1}, seq_id=7) == a
    with pytest.raises(tdb.SequenceReused):
        db.create_future("forward_backward", "m", {"x": 2}, seq_id=7)
    assert db.create_future("forward_backward", "m", {"x": 2}, seq_id=8) != a


def test_datums_rebuild_full_sequence_left_padded():
    b = datums_to_batch([_datum([5, 6, 7, 8]), _datum([9, 10, 11, 12, 13, 14], weights=[0, 0, 1, 1, 1])], pad_token_id=0)
    assert b["sequences"].tolist() == [[0, 0, 5, 6, 7, 8], [9, 10, 11, 12, 13, 14]]
    assert b["attention_mask"].sum(1).tolist() == [4, 6]
    assert b["loss_mask"].tolist() == [[0, 0, 1, 1, 1], [0, 0, 1, 1, 1]]
    assert b["response_mask"].tolist() == [[0, 0, 1, 1, 1], [1, 1, 1, 1, 1]]
    with pytest.raises(ValueError):
        datums_to_batch([{"model_input": {"chunks": [{"tokens": [1, 2]}]},
                          "loss_fn_inputs": {"target_tokens": {"data": [2]}}}], 0)


class _FakeBackend:
    def __init__(self):
        self.calls = []

    def create_model(self, model_id, lora_config=None, model_role="policy"):
        self.calls.append(("create", model_id))

    def forward_backward(self, model_id, datums, loss_fn, cfg=None, forward_only=False):
        self.calls.append(("fb", model_id, len(datums), forward_only))
        return {"loss_fn_output_type": "logprobs", "loss_fn_outputs": [{"i": i} for i in range(len(datums))], "metrics": {}}

    def optim_step(self, model_id, adam_params=None):
        self.calls.append(("optim", model_id))
        return {"metrics": {}}

    def delete_model(self, model_id):
        self.calls.append(("delete", model_id))


def test_engine_batches_passes_up_to_each_models_barrier():
    db = tdb.TinkerDB()
    be = _FakeBackend()
    eng = teng.TinkerEngine(db, lambda base: be)
    for m in ("a", "b"):
        rid = db.create_future(teng.CREATE_MODEL, m, {"base_model": "x"})
        db.create_model(m, "x", None, "policy", "s", rid)
    eng.step()
    body = lambda n: {"forward_backward_input": {"data": [_datum([1, 2, 3])] * n, "loss_fn": "cross_entropy"}}
    r1 = db.create_future(teng.FORWARD_BACKWARD, "a", body(2))
    r2 = db.create_future(teng.FORWARD_BACKWARD, "a", body(3))
    o1 = db.create_future(teng.OPTIM_STEP, "a", {"adam_params": {}})
    r3 = db.create_future(teng.FORWARD_BACKWARD, "a", body(1))  # behind the barrier: must wait for the optim step
    r4 = db.create_future(teng.FORWARD_BACKWARD, "b", body(4))  # other model: unaffected by a's barrier
    got = {r["request_id"] for r in eng.find_batchable_model_passes(teng.FORWARD_BACKWARD)}
    assert got == {r1, r2, r4}
    be.calls.clear()
    eng.step()
    assert ("fb", "a", 5, False) in be.calls and ("fb", "b", 4, False) in be.calls
    assert be.calls.index(("optim", "a")) > be.calls.index(("fb", "a", 5, False))
    assert db.get_future(r3)["status"] == tdb.PENDING or ("fb", "a", 1, False) in be.calls
    eng.step()
    assert db.get_future(r3)["status"] == tdb.COMPLETED
    assert [o["i"] for o in json.loads(db.get_future(r2)["result_data"])["loss_fn_outputs"]] == [2, 3, 4]
    assert db.get_future(o1)["status"] == tdb.COMPLETED


def test_stale_session_unloads_models():
    db = tdb.TinkerDB()
    be = _FakeBackend()
    eng = teng.TinkerEngine(db, lambda base: be, session_timeout_s=0.0)
    db.create_session("s", [], None, "t")
    rid = db.create_future(teng.CREATE_MODEL, "m", {"base_model": "x"})
    db.create_model("m", "x", None, "policy", "s", rid)
    eng.step()
    time.sleep(0.01)
    assert eng.cleanup_stale_sessions() == 1 and ("delete", "m") in be.calls
    assert db.get_model("m")["status"] == "unloaded"


def test_rest_round_trip(tmp_path):
    from fastapi.testclient import TestClient

    from skyrl_b200.parallel.dist import get_env
    from skyrl_b200.tinker.api import build_app

    tok = SyntheticTokenizer(2048)
    ov = {"trainer.bf16": "false", "trainer.policy.optimizer_config.num_warmup_steps": 0,
          "generator.inference_engine.max_num_seqs": 8, "generator.sampling_params.max_generate_length": 16,
          "trainer.max_prompt_length": 64, "generator.inference_engine.enforce_eager": "true",
          "generator.inference_engine.engine_init_kwargs": "{num_blocks: 64}"}
    factory = lambda base: SkyRLTrainBackend(base, ov, env=get_env(), tokenizer=tok, checkpoints_base=str(tmp_path))
    app = build_app(factory, supported_models=["tiny-qwen2-d128"], poll_interval=0.01)
    with TestClient(app) as c:
        assert c.get("/api/v1/healthz").json() == {"status": "ok"}
        sid = c.post("/api/v1/create_session", json={"tags": [], "sdk_version": "t"}).json()["session_id"]
        r = c.post("/api/v1/create_model", json={"session_id": sid, "base_model": "tiny-qwen2-d128", "lora_config": {"rank": 0}})
        mid = r.json()["model_id"]

        def wait(fut):
            r = c.post("/api/v1/retrieve_future", json={"request_id": fut["request_id"]})
            assert r.status_code == 200, r.text
            return r.json()

        wait({"request_id": r.json()["request_id"]})
        assert c.post("/api/v1/get_info", json={"model_id": mid}).json()["status"] == "ready"
        data = [_datum([10 + i, 20, 30, 40, 50, 60]) for i in range(4)]
        losses = []
        for step in range(4):
            fb = c.post("/api/v1/forward_backward", json={"model_id": mid, "seq_id": 2 * step,
                                                          "forward_backward_input": {"data": data, "loss_fn": "cross_entropy"}})
            assert fb.status_code == 200, fb.text
            # a retry with the same seq_id maps to the same future; a different payload is a conflict
            again = c.post("/api/v1/forward_backward", json={"model_id": mid, "seq_id": 2 * step,
                                                             "forward_backward_input": {"data": data, "loss_fn": "cross_entropy"}})
            assert again.json()["request_id"] == fb.json()["request_id"]
            op = c.post("/api/v1/optim_step", json={"model_id": mid, "seq_id": 2 * step + 1,
                                                    "adam_params": {"learning_rate": 5e-3}})
            out = wait(fb.json())
            assert len(out["loss_fn_outputs"]) == 4 and len(out["loss_fn_outputs"][0]["logprobs"]["data"]) == 5
            losses.append(sum(sum(o["elementwise_loss"]["data"]) for o in out["loss_fn_outputs"]))
            assert wait(op.json())["metrics"]["learning_rate"] == pytest.approx(5e-3)
        assert losses[-1] < losses[0]
        bad = c.post("/api/v1/forward_backward", json={"model_id": mid, "seq_id": 0,
                                                       "forward_backward_input": {"data": data[:1], "loss_fn": "cross_entropy"}})
        assert bad.status_code == 409
        sv = wait(c.post("/api/v1/save_weights", json={"model_id": mid, "path": "ck1"}).json())
        assert sv["path"] == f"tinker://{mid}/weights/ck1"
        assert c.post("/api/v1/save_weights", json={"model_id": mid, "path": "ck1"}).status_code == 409
        fw = wait(c.post("/api/v1/forward", json={"model_id": mid, "forward_input": {"data": data, "loss_fn": "cross_entropy"}}).json())
        ref_lp = fw["loss_fn_outputs"][0]["logprobs"]["data"]
        wait(c.post("/api/v1/forward_backward", json={"model_id": mid, "forward_backward_input": {"data": data, "loss_fn": "cross_entropy"}}).json())
        wait(c.post("/api/v1/optim_step", json={"model_id": mid, "adam_params": {"learning_rate": 5e-2}}).json())
        wait(c.post("/api/v1/load_weights", json={"model_id": mid, "path": sv["path"]}).json())
        fw2 = wait(c.post("/api/v1/forward", json={"model_id": mid, "forward_input": {"data": data, "loss_fn": "cross_entropy"}}).json())
        assert fw2["loss_fn_outputs"][0]["logprobs"]["data"] == pytest.approx(ref_lp, abs=1e-4)
        ss = wait(c.post("/api/v1/save_weights_for_sampler", json={"model_id": mid, "sampling_session_seq_id": 0}).json())
        smp = wait(c.post("/api/v1/asample", json={"sampling_session_id": ss["sampling_session_id"], "num_samples": 2,
                                                   "prompt": {"chunks": [{"tokens": [10, 20, 30]}]},
                                                   "sampling_params": {"max_tokens": 5, "temperature": 1.0}}).json())
        assert len(smp["sequences"]) == 2 and all(1 <= len(s["tokens"]) <= 5 for s in smp["sequences"])
        assert len(smp["sequences"][0]["logprobs"]) == len(smp["sequences"][0]["tokens"])
        cks = c.get(f"/api/v1/training_runs/{mid}/checkpoints").json()["checkpoints"]
        assert [k["checkpoint_id"] for k in cks] == ["ck1"]
        arch = c.get(f"/api/v1/training_runs/{mid}/checkpoints/ck1/archive")
        assert arch.status_code == 200 and len(arch.content) > 1000
        assert c.delete(f"/api/v1/training_runs/{mid}/checkpoints/weights/ck1").status_code == 204
        assert c.get(f"/api/v1/training_runs/{mid}/checkpoints").json()["checkpoints"] == []
        runs = c.get("/api/v1/training_runs").json()
        assert runs["cursor"]["total_count"] == 1 and runs["training_runs"][0]["training_run_id"] == mid
        assert c.post("/api/v1/retrieve_future", json={"request_id": "99999"}).status_code == 404


def test_lora_models_share_one_base_and_keep_their_own_state(tmp_path):
    """Two LoRA model ids are tenants of one worker: interleaved forward_backward / optim_step calls give each the
    result it would have had alone, pending gradients survive a swap, and sampling follows the requested id."""
    import torch

    from skyrl_b200.parallel import dist as pdist
    from skyrl_b200.tinker.backend import SkyRLTrainBackend
    from skyrl_b200.utils.tokenizer import SyntheticTokenizer

    pdist.reset_env_for_tests()
    ov = {"trainer.bf16": "false", "generator.sampling_params.max_generate_length": 8, "trainer.max_prompt_length": 16,
          "generator.inference_engine.enforce_eager": "true", "generator.inference_engine.max_num_seqs": 4,
          "trainer.policy.optimizer_config.lr": 1e-2, "trainer.policy.optimizer_config.max_grad_norm": 1e9,
          "trainer.gradient_checkpointing": "false"}

    def backend(sub):
        return SkyRLTrainBackend("tiny-llama", ov, tokenizer=SyntheticTokenizer(1024), checkpoints_base=str(tmp_path / sub))

    data_a = [_datum([5, 6, 7, 8, 9, 10]), _datum([11, 12, 13, 14])]
    data_b = [_datum([21, 22, 23, 24, 25]), _datum([31, 32, 33])]
    lora = lambda seed: {"rank": 4, "alpha": 8, "seed": seed}  # noqa: E731

    # each model alone
    alone = {}
    for name, seed, data in (("a", 1, data_a), ("b", 2, data_b)):
        be = backend("alone_" + name)
        be.create_model(name, lora(seed))
        be.forward_backward(name, data, "cross_entropy")
        be.forward_backward(name, data[:1], "cross_entropy")
        be.optim_step(name, {"learning_rate": 1e-2})
        alone[name] = be.models[name].worker.model.flat_params.clone()

    # both on one backend, calls interleaved so that every swap happens with gradients pending
    be = backend("shared")
    be.create_model("a", lora(1))
    be.create_model("b", lora(2))
    assert be.models["a"].worker is be.models["b"].worker and len(be._lora_hosts) == 1
    be.forward_backward("a", data_a, "cross_entropy")
    be.forward_backward("b", data_b, "cross_entropy")
    be.forward_backward("a", data_a[:1], "cross_entropy")
    be.forward_backward("b", data_b[:1], "cross_entropy")
    ra = be.optim_step("a", {"learning_rate": 1e-2})
    rb = be.optim_step("b", {"learning_rate": 1e-2})
    assert ra["metrics"]["grad_norm"] > 0 and rb["metrics"]["grad_norm"] > 0
    w = be.models["a"].worker
    be._activate(be.models["a"])
    assert torch.allclose(w.model.flat_params, alone["a"], atol=1e-6)
    be._activate(be.models["b"])
    assert torch.allclose(w.model.flat_params, alone["b"], atol=1e-6)
    assert not torch.allclose(alone["a"], alone["b"])

    # sampling runs the merged weights of the requested model id (greedy: different adapters, different log-probs)
    sp = [{"max_tokens": 6, "temperature": 0.0}]
    be.save_sampler_checkpoint("a", None, persist=False)
    sa = be.sample([[5, 6, 7]], sp, [1], model_id="a")[0]["sequences"][0]
    sb = be.sample([[5, 6, 7]], sp, [1], model_id="b")[0]["sequences"][0]
    sa2 = be.sample([[5, 6, 7]], sp, [1], model_id="a")[0]["sequences"][0]
    assert sa["tokens"] == sa2["tokens"] and sa["logprobs"] == pytest.approx(sa2["logprobs"], abs=1e-6)
    assert sa["logprobs"] != pytest.approx(sb["logprobs"], abs=1e-7)

    # deleting one tenant keeps the other and the shared worker; deleting the last one frees the host
    be.delete_model("a")
    assert "b" in be.models and len(be._lora_hosts) == 1
    be.forward_backward("b", data_b, "cross_entropy")
    be.delete_model("b")
    assert not be._lora_hosts and be.engine is None


def test_loss_fn_config_keys_are_validated_and_mapped_onto_the_algorithm_config():
    from fastapi import HTTPException

    from skyrl_b200.tinker.api import _validate_pass_input

    N = SkyRLTrainBackend.normalize_loss_fn_config
    assert N("ppo", {"clip_low_threshold": 0.9, "clip_high_threshold": 1.25}) == pytest.approx({"eps_clip_low": 0.1, "eps_clip_high": 0.25})
    assert N("gspo", {"clip_high_threshold": 1.0004}) == pytest.approx({"eps_clip_high": 0.0004})
    assert N("dppo", {"delta_low": 0.2, "delta_high": 0.3}) == {"dppo": {"delta_low": 0.2, "delta_high": 0.3}}
    got = N("cispo", {"clip_low_threshold": 0.0, "clip_high_threshold": 5.0})
    assert got == {"cispo": {"cispo_eps_clip_low": 1.0, "cispo_eps_clip_high": 4.0}}
    assert N("ppo_critic", {"value_clip": 0.2}) == {"value_clip": 0.2} and N("ppo", None) is None and N("ppo", {}) is None

    datum = _datum([1, 2, 3, 4])
    datum["loss_fn_inputs"].update({"logprobs": {"data": [-1.0] * 3}, "advantages": {"data": [0.5] * 3}})
    ok = lambda fn, cfg: _validate_pass_input({"data": [datum], "loss_fn": fn, "loss_fn_config": cfg})  # noqa: E731
    ok("ppo", {"clip_low_threshold": 0.9, "clip_high_threshold": 1.1})
    ok("ppo", {"value_clip": 0.2})
    ok("ppo_critic", {"value_clip": 0.2})
    ok("dppo", {"delta_low": 0.2, "delta_high": 0.2})
    for fn, cfg, msg in (("dppo", {"clip_low_threshold": 0.9}, "Invalid loss_fn_config keys"),
                         ("ppo", {"clip_ratio": 0.2}, "Invalid loss_fn_config keys"),
                         ("cross_entropy", {"clip_low_threshold": 0.9}, "does not accept loss_fn_config keys"),
                         ("ppo", {"value_clip": "x"}, "must be numbers")):
        with pytest.raises(HTTPException) as e:
            ok(fn, cfg)
        assert e.value.status_code == 422 and msg in e.value.detail


def test_backend_applies_tinker_clip_thresholds(tmp_path):
    """The sampled tokens are far less likely under the model than the given log-probs say (ratio near 0) and their
    advantages are negative: a tight lower threshold clips them (no gradient), a lower threshold of 0 does not."""
    from skyrl_b200.parallel import dist as pdist

    pdist.reset_env_for_tests()
    ov = {"trainer.bf16": "false", "trainer.gradient_checkpointing": "false", "trainer.policy.optimizer_config.max_grad_norm": 1e9}
    be = SkyRLTrainBackend("tiny-llama", ov, tokenizer=SyntheticTokenizer(1024), checkpoints_base=str(tmp_path))
    be.create_model("m", None)
    toks = [5, 6, 7, 8, 9, 10]
    d = _datum(toks)
    n = len(toks) - 1
    d["loss_fn_inputs"].update({"logprobs": {"data": [-0.05] * n, "dtype": "float32", "shape": [n]},      # far from the
                                "advantages": {"data": [-1.0] * n, "dtype": "float32", "shape": [n]}})      # model's own
    be.forward_backward("m", [d], "ppo", {"clip_low_threshold": 0.999, "clip_high_threshold": 1.001})
    tight = float(be.optim_step("m", {"learning_rate": 0.0})["metrics"]["grad_norm"])
    be.forward_backward("m", [d], "ppo", {"clip_low_threshold": 0.0, "clip_high_threshold": 1e9})
    loose = float(be.optim_step("m", {"learning_rate": 0.0})["metrics"]["grad_norm"])
    assert loose > 0 and tight < 1e-3 * loose
    with pytest.raises(ValueError, match="only valid for critic"):
        be.forward_backward("m", [d], "ppo_critic", None)
