"""SFT path on CPU: tokenization masks, packing, sampler state, a short training run that lowers the loss, resume."""
import json
import os

import numpy as np
import pytest
import torch

from skyrl_b200.config.sft_config import SFTConfig
from skyrl_b200.train import sft_data
from skyrl_b200.train.sft_trainer import SFTTrainer
from skyrl_b200.utils.tokenizer import SyntheticTokenizer


@pytest.fixture()
def tok():
    return SyntheticTokenizer(2048)


def _conv(n_turns=2):
    msgs = [{"role": "system", "content": "be brief"}]
    for i in range(n_turns):
        msgs.append({"role": "user", "content": f"question number {i} please"})
        msgs.append({"role": "assistant", "content": f"answer {i} is {i * 7}"})
    return {"messages": msgs}


def test_chat_masks_last_vs_all(tok):
    last = sft_data.tokenize_chat_example(_conv(3), tok, train_on_what="last_assistant_message")
    allm = sft_data.tokenize_chat_example(_conv(3), tok, train_on_what="all_assistant_messages")
    assert last["num_actions"] == len(last["loss_mask"]) and all(last["loss_mask"])
    assert allm["num_actions"] == len(allm["loss_mask"]) and allm["loss_mask"][0] == 1
    assert 0 in allm["loss_mask"]  # user turns between assistant turns are not trained on
    assert sum(allm["loss_mask"]) > sum(last["loss_mask"])
    assert len(allm["input_ids"]) == len(last["input_ids"])
    # truncation that removes every trained token drops the example
    assert sft_data.tokenize_chat_example(_conv(1), tok, max_length=3) is None


def test_tool_call_normalisation():
    msgs = [{"role": "assistant", "content": None,
             "tool_calls": json.dumps([{"type": "function", "function": {"name": "f", "arguments": json.dumps({"x": 1})}}])}]
    out = sft_data.normalize_chat_messages(msgs)
    assert out[0]["content"] == "" and out[0]["tool_calls"][0]["function"]["arguments"] == {"x": 1}


def test_packing_respects_capacity_and_multiple():
    rng = np.random.default_rng(0)
    lens = rng.integers(10, 500, size=200).tolist()
    for fn in (sft_data.ffd_pack, lambda l, c: sft_data.balanced_pack(l, c, 4)):
        bins = fn(lens, 1024)
        assert sorted(i for b in bins for i in b) == list(range(200))
        assert all(sum(lens[i] for i in b) <= 1024 for b in bins)
    assert len(sft_data.balanced_pack(lens, 1024, 4)) % 4 == 0
    with pytest.raises(ValueError):
        sft_data.ffd_pack([2000], 1024)


def test_sampler_state_roundtrip():
    s = sft_data.StatefulSampler(list(range(1, 41)), 8, seed=3)
    it = iter(s)
    first = [next(it), next(it)]
    st = s.state_dict()
    rest = list(it)
    s2 = sft_data.StatefulSampler(list(range(1, 41)), 8, seed=3)
    s2.load_state_dict(st)
    assert list(iter(s2)) == rest and len(first[0]) == 8
    g = sft_data.StatefulSampler([5, 50, 7, 60, 9, 70, 8, 55], 2, seed=0, mode="length_grouped", mega=2)
    order = [i for b in g for i in b]
    assert sorted(order) == list(range(8))


def _examples(tok, n=32):
    ex = []
    for i in range(n):
        ex.append(sft_data.tokenize_chat_example(
            {"messages": [{"role": "user", "content": f"say {i % 4}"}, {"role": "assistant", "content": f"ok {i % 4} " * 3}]},
            tok))
    return ex


@pytest.mark.parametrize("packed", [False, True])
def test_sft_training_reduces_loss_and_resumes(tok, tmp_path, packed):
    cfg = SFTConfig.from_cli_overrides([
        "model.path=tiny-qwen2-d128", "batch_size=8", "micro_train_batch_size_per_gpu=4", "num_steps=6",
        "optimizer_config.lr=2e-3", "optimizer_config.num_warmup_steps=0", f"ckpt_path={tmp_path}/ckpt", "ckpt_interval=3",
        "disable_cache=true", "bf16=false", f"log_path={tmp_path}/logs", "sampler=sequential",
        f"use_sequence_packing={'true' if packed else 'false'}", "max_tokens_per_microbatch=256"])
    ex = _examples(tok)
    tr = SFTTrainer(cfg, tokenizer=tok, train_examples=ex, eval_examples=[("held", ex[:8])]).setup()
    before = tr.run_eval()["eval/held/loss"]
    last = tr.train()
    after = tr.run_eval()["eval/held/loss"]
    assert np.isfinite(last["train/loss"]) and after < before - 0.2
    assert os.path.isdir(os.path.join(str(tmp_path), "ckpt", "global_step_6", "policy"))
    cfg2 = SFTConfig.from_cli_overrides([
        "model.path=tiny-qwen2-d128", "batch_size=8", "micro_train_batch_size_per_gpu=4", "num_steps=7",
        "optimizer_config.lr=2e-3", "optimizer_config.num_warmup_steps=0", f"ckpt_path={tmp_path}/ckpt", "resume_from=latest",
        "disable_cache=true", "bf16=false", f"log_path={tmp_path}/logs", "sampler=sequential"])
    tr2 = SFTTrainer(cfg2, tokenizer=tok, train_examples=ex, eval_examples=[("held", ex[:8])]).setup()
    tr2.train()
    assert tr2.global_step == 7
    assert abs(tr2.run_eval()["eval/held/loss"] - after) < 0.5


def test_dummy_run(tok, tmp_path):
    cfg = SFTConfig.from_cli_overrides(["model.path=tiny-qwen2-d128", "batch_size=2", "max_length=64", "bf16=false",
                                        "dummy_run_full_ctx=true", "dummy_run_max_steps=2", f"log_path={tmp_path}"])
    out = SFTTrainer(cfg, tokenizer=tok).setup().train()
    assert out["train/tokens_per_second"] > 0


def test_sft_loop_fires_reference_style_callbacks(tok, tmp_path):
    """Event names, argument order and per-event fields of the reference's callback interface; control flags set in
    on_step_end are honoured in the same step (an evaluation after step 1, a checkpoint and a stop after step 2)."""
    from skyrl_b200.train.callbacks import EVENTS, TrainingCallback

    class Rec(TrainingCallback):
        seen = []

    rec = Rec()
    for name in EVENTS:
        def handler(trainer, ci, control, name=name):
            rec.seen.append((name, ci.global_step, ci.ckpt_path is not None, ci.metrics is not None, ci.batch is not None))
            if name == "on_step_end" and ci.global_step == 1:
                control.should_evaluate = True
            if name == "on_step_end" and ci.global_step == 2:
                control.should_save = True
                control.should_stop = True
            if name == "on_log":
                ci.logs["custom/x"] = 7.0

        setattr(rec, name, handler)
    cfg = SFTConfig.from_cli_overrides([
        "model.path=tiny-qwen2-d128", "batch_size=8", "micro_train_batch_size_per_gpu=4", "num_steps=6",
        "optimizer_config.lr=1e-3", f"ckpt_path={tmp_path}/ckpt", "ckpt_interval=0", "disable_cache=true", "bf16=false",
        f"log_path={tmp_path}/logs", "sampler=sequential", "eval_interval=0", "eval_before_train=false"])
    ex = _examples(tok)
    tr = SFTTrainer(cfg, tokenizer=tok, train_examples=ex, eval_examples=[("held", ex[:8])]).setup()
    tr.add_callback(rec)
    last = tr.train()
    names = [e[0] for e in rec.seen]
    assert names == ["on_train_start", "on_epoch_start",
                     "on_step_start", "on_step_end", "on_eval_start", "on_eval_end", "on_log",
                     "on_step_start", "on_step_end", "on_log", "on_save",
                     "on_epoch_end", "on_train_end"]
    assert tr.global_step == 2 and last["custom/x"] == 7.0 and "eval/held/loss" not in last
    ev = next(e for e in rec.seen if e[0] == "on_eval_end")
    assert ev[1] == 1 and ev[3]
    assert next(e for e in rec.seen if e[0] == "on_save")[2] and next(e for e in rec.seen if e[0] == "on_step_start")[4]
    assert os.path.isdir(os.path.join(str(tmp_path), "ckpt", "global_step_2", "policy"))
