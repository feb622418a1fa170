"""Utilities for hand-written generators: chat templates, message encoding inside a conversation, loss masks and
log-prob alignment per message, overlong filtering, turn counts, slicing."""
import pytest

from skyrl_b200.train.generators import utils as U
from skyrl_b200.utils.tokenizer import SyntheticTokenizer


class _ChatMLTok:
    """A word-level ChatML-like tokenizer that, like some real templates, injects a default system message when the
    conversation does not start with one, and puts a newline token after the end-of-turn token."""

    IM_START, IM_END, NL = 1000, 1001, 1002
    eos_token_id = 1001

    def __init__(self):
        self.vocab = {}

    def _w(self, text):
        return [self.vocab.setdefault(w, 10 + len(self.vocab)) for w in str(text).split()]

    def apply_chat_template(self, conversation, add_generation_prompt=False, tokenize=True, **kw):
        conv = list(conversation)
        if not conv or conv[0]["role"] != "system":
            conv = [{"role": "system", "content": "you are a default system prompt"}] + conv
        ids = []
        for m in conv:
            ids += [self.IM_START] + self._w(m["role"]) + [self.NL] + self._w(m["content"]) + [self.IM_END, self.NL]
        if add_generation_prompt:
            ids += [self.IM_START] + self._w("assistant") + [self.NL]
        return ids


def test_generation_prompt_and_subset_encoding_do_not_inject_a_default_system_message():
    tok = _ChatMLTok()
    gp = U.get_generation_prompt_ids(tok)
    assert gp == [tok.IM_START] + tok._w("assistant") + [tok.NL]
    ids = U.encode_messages_subset([{"role": "user", "content": "tool says four"}], tok)
    assert ids == [tok.IM_START] + tok._w("user") + [tok.NL] + tok._w("tool says four") + [tok.IM_END, tok.NL]
    assert tok._w("default")[0] not in ids
    with pytest.raises(ValueError):
        U.encode_messages_subset([], tok)
    with pytest.raises(ValueError):
        U.get_generation_prompt_ids(tok, {"enable_thinking": False})


def test_response_ids_mask_and_logprobs_follow_the_messages():
    tok = _ChatMLTok()
    msgs = [{"role": "assistant", "content": "let me look"}, {"role": "user", "content": "result 4"},
            {"role": "assistant", "content": "the answer is 4"}]
    lp1, lp2 = [-0.1, -0.2, -0.3, -0.4], [-1.0, -1.1, -1.2, -1.3]  # second engine stopped before the end-of-turn token
    ids, mask, lps = U.get_response_ids_and_loss_mask_from_messages(msgs, tok, [lp1, lp2])
    assert len(ids) == len(mask) == len(lps)
    gp = U.get_generation_prompt_ids(tok)
    a1 = gp + tok._w("let me look") + [tok.IM_END, tok.NL]
    assert ids[: len(a1)] == a1
    # generation prompt masked, content + end-of-turn trained, trailing newline masked
    assert mask[: len(a1)] == [0] * len(gp) + [1] * 4 + [0]
    assert lps[: len(a1)] == [0.0] * len(gp) + lp1 + [0.0]
    u = [tok.IM_START] + tok._w("user") + [tok.NL] + tok._w("result 4") + [tok.IM_END, tok.NL]
    assert ids[len(a1): len(a1) + len(u)] == u and set(mask[len(a1): len(a1) + len(u)]) == {0}
    tail_mask, tail_lp = mask[len(a1) + len(u):], lps[len(a1) + len(u):]
    assert tail_mask == [0] * len(gp) + [1] * 5 + [0]
    assert tail_lp == [0.0] * len(gp) + lp2 + [0.0] + [0.0]  # 4 given for 5 trained tokens: the end-of-turn entry is 0
    assert U.compute_turn_token_counts([mask]) == [4, 5]
    with pytest.raises(ValueError):
        U.get_response_ids_and_loss_mask_from_messages(msgs, tok, [[-0.1], lp2])
    # the synthetic tokenizer of the test suite works the same way
    st = SyntheticTokenizer(64)
    ids, mask, lps = U.get_response_ids_and_loss_mask_from_messages(
        [{"role": "assistant", "content": "7 8"}, {"role": "user", "content": "9"}], st)
    assert ids == [3, 7, 8, 1, 2, 9, 1] and mask == [0, 1, 1, 1, 0, 0, 0] and lps is None


def test_overlong_filtering_turn_counts_and_slicing():
    masks = [[1, 1, 0, 1], [1, 1, 1], [0, 0]]
    assert U.apply_overlong_filtering(masks, ["stop", "length", "stop"]) == [[1, 1, 0, 1], [0, 0, 0], [0, 0]]
    with pytest.raises(ValueError):
        U.apply_overlong_filtering(masks, ["stop"])
    assert U.compute_turn_token_counts(masks) == [2, 1, 3]
    assert U.compute_turn_token_counts([[], [0, 0]]) == []
    out = {"prompt_token_ids": [[1], [2], [3]], "response_ids": [[4], [5], [6]], "rewards": [0.0, 1.0, 0.5],
           "loss_masks": [[1], [1], [1]], "stop_reasons": ["stop"] * 3, "rollout_metrics": {"x": 1}, "rollout_logprobs": None}
    s = U.slice_generator_output(out, 1, 3)
    assert s["response_ids"] == [[5], [6]] and s["rewards"] == [1.0, 0.5] and s["rollout_metrics"] == {"x": 1}
    assert s["rollout_logprobs"] is None


def test_custom_chat_templates_by_name_and_file(tmp_path):
    assert U.get_custom_chat_template(None) is None
    assert U.get_custom_chat_template({"source": "name", "name_or_path": None}) is None
    t = U.get_custom_chat_template({"source": "name", "name_or_path": "chatml_no_default_system"})
    assert "<|im_start|>" in t and "add_generation_prompt" in t
    with pytest.raises(ValueError):
        U.get_custom_chat_template({"source": "name", "name_or_path": "nope"})
    with pytest.raises(ValueError):
        U.get_custom_chat_template({"name_or_path": "x"})
    f = tmp_path / "my.jinja"
    f.write_text("{{ messages }}")
    assert U.get_custom_chat_template({"source": "file", "name_or_path": str(f)}) == "{{ messages }}"
    bad = tmp_path / "secrets.env"
    bad.write_text("x")
    with pytest.raises(ValueError):
        U.get_custom_chat_template({"source": "file", "name_or_path": str(bad)})
    # the named template renders the way a tokenizer would use it (the generation tags are an extension that
    # transformers registers; plain jinja sees the template without them)
    import re

    import jinja2

    plain = re.sub(r"\{%-? *(end)?generation *-?%\}", "", t)
    txt = jinja2.Template(plain).render(messages=[{"role": "user", "content": "hi"}], add_generation_prompt=True)
    assert txt == "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    assert "generation" in t and {"qwen3_with_thinking", "qwen3_without_thinking"} <= set(U.CUSTOM_CHAT_TEMPLATES)


def _valid_out():
    return {"prompt_token_ids": [[1, 2, 3, 4], [5, 6], [7, 8, 9]], "response_ids": [[10, 11, 12], [13, 14], [15]],
            "rewards": [[0.5, 0.6, 0.7], [0.8, 0.9], [1.0]], "loss_masks": [[1, 1, 0], [1, 1], [0]],
            "stop_reasons": ["stop", "length", "stop"], "rollout_metrics": {}, "rollout_logprobs": None}


def test_validate_generator_output_accepts_well_formed_rows_and_names_the_broken_one():
    V, E = U.validate_generator_output, U.GeneratorOutputError
    out = _valid_out()
    assert V(3, out) == []
    out["rewards"] = [0.5, 0.6, 0.7]
    assert V(3, out) == []
    out["rollout_logprobs"] = [[0.11, 0.12, 0.13], [0.2, 0.3], [0.4]]
    assert V(3, out) == []
    with pytest.raises(E, match="no responses"):
        V(1, dict(_valid_out(), response_ids=[]))
    with pytest.raises(E, match="3 prompts but 2 responses"):
        V(3, {k: (v[:2] if isinstance(v, list) else v) for k, v in _valid_out().items()})
    with pytest.raises(E, match="'stop_reasons' has 2 entries"):
        V(3, dict(_valid_out(), stop_reasons=["stop", "stop"]))
    with pytest.raises(E, match="row 1: loss mask has 3 entries for 2"):
        V(3, dict(_valid_out(), loss_masks=[[1, 1, 0], [1, 1, 1], [0]]))
    with pytest.raises(E, match="row 0: 2 token rewards for 3"):
        V(3, dict(_valid_out(), rewards=[[0.5, 0.6], [0.8, 0.9], [1.0]]))
    with pytest.raises(E, match="row 2: 2 rollout log-probs for 1"):
        V(3, dict(_valid_out(), rollout_logprobs=[[0.1, 0.2, 0.3], [0.2, 0.3], [0.4, 0.5]]))
    with pytest.raises(E, match="mix"):
        V(3, dict(_valid_out(), rewards=[[0.5, 0.6, 0.7], 0.8, [1.0]]))
    with pytest.raises(E, match="must be a number"):
        V(3, dict(_valid_out(), rewards=["a", 0.1, 0.2]))
    with pytest.raises(E, match="token rewards must be numbers"):
        V(3, dict(_valid_out(), rewards=[[0.5, None, 0.7], [0.8, 0.9], [1.0]]))
    assert "masked out" in V(3, dict(_valid_out(), loss_masks=[[0, 0, 0], [0, 0], [0]]))[0]


def test_validate_step_wise_rows():
    from skyrl_b200.train.generators.base import TrajectoryID

    V, E = U.validate_generator_output, U.GeneratorOutputError

    def rows(tids, last):
        n = len(tids)
        return {"prompt_token_ids": [[1]] * n, "response_ids": [[2]] * n, "rewards": [[0.0]] * n, "loss_masks": [[1]] * n,
                "stop_reasons": ["stop"] * n, "rollout_logprobs": None,
                "trajectory_ids": [TrajectoryID(t, 0) for t in tids], "is_last_step": last}

    assert V(2, rows(["a", "a", "b"], [False, True, True]), step_wise=True) == []  # the prompt count is not compared
    assert V(2, rows(["a", "b"], [True, True]), step_wise=True) == []
    with pytest.raises(E, match="needs 'is_last_step'"):
        V(1, dict(rows(["a"], [True]), is_last_step=None), step_wise=True)
    with pytest.raises(E, match="'is_last_step' has 2 entries"):
        V(1, rows(["a", "a", "b"], [True, True]), step_wise=True)
    with pytest.raises(E, match="last row"):
        V(1, rows(["a", "a"], [False, False]), step_wise=True)
    with pytest.raises(E, match="not adjacent"):
        V(1, rows(["a", "b", "a"], [True, True, True]), step_wise=True)
    with pytest.raises(E, match="ends at row 0"):
        V(1, rows(["a", "b"], [False, True]), step_wise=True)
    with pytest.raises(E, match="continues at row 1"):
        V(1, rows(["a", "a"], [True, True]), step_wise=True)


@pytest.mark.parametrize("rewards,avg,pass_n,pos", [
    ([1.0, 2.0], 1.5, 1.0, 1.5),
    ([[1.0, 0.0], [0.0, 1.0]], 1.0, 0.5, 1.0),     # token-level: the last token's reward decides the pass
    ([-1.0, 2.0], 0.5, 0.5, 1.0),                  # positive mass averaged over all trajectories
    ([[1.0, -1.0], [-0.5, 0.5]], 0.0, 0.5, 0.75),
])
def test_reward_metrics_follow_the_reference_definitions(rewards, avg, pass_n, pos):
    m = U.get_metrics_from_generator_output({"rewards": rewards}, ["a", "b"])
    assert (m["avg_score"], m["pass_at_n"], m["mean_positive_reward"]) == pytest.approx((avg, pass_n, pos))
    with pytest.raises(ValueError):
        U.get_metrics_from_generator_output({"rewards": []}, [])


@pytest.mark.parametrize("masks,stops,want", [
    ([[1, 1, 0, 1], [0, 1, 1, 1], [1, 0, 1]], ["stop"] * 3, [[1, 1, 0, 1], [0, 1, 1, 1], [1, 0, 1]]),
    ([[1, 1, 0, 1], [0, 1, 1, 1], [1, 0, 1]], ["length"] * 3, [[0] * 4, [0] * 4, [0] * 3]),
    ([[1, 1], [1, 0, 1], [0, 1, 1, 1]], ["length", "abort", "cancelled"], [[0, 0], [0, 0, 0], [0, 0, 0, 0]]),
    ([], [], []),
])
def test_overlong_filtering_cases_of_the_reference(masks, stops, want):
    before = [list(m) for m in masks]
    assert U.apply_overlong_filtering(masks, stops) == want and masks == before  # the input is not modified


def test_rollout_metrics_assistant_tokens_turns_and_time_splits():
    import numpy as np

    out1 = {"prompt_token_ids": [[1, 2], [3, 4]], "response_ids": [[1, 2], [3, 4]], "rewards": [1.0, 2.0],
            "loss_masks": [[1, 1], [1, 1]], "stop_reasons": ["stop", "stop"], "rollout_logprobs": [[0.1, 0.2], [0.3, 0.4]]}
    out2 = {"prompt_token_ids": [[5, 6, 7], [8]], "response_ids": [[5, 6, 7], [8]], "rewards": [2.0, 3.0],
            "loss_masks": [[1, 1, 1], [1]], "stop_reasons": ["stop", "stop"], "rollout_logprobs": [[0.5, 0.6, 0.7], [0.8]]}
    cat = U.concatenate_generator_outputs([out1, out2])
    assert cat["response_ids"] == [[1, 2], [3, 4], [5, 6, 7], [8]] and cat["rewards"] == [1.0, 2.0, 2.0, 3.0]
    assert cat["rollout_logprobs"] == [[0.1, 0.2], [0.3, 0.4], [0.5, 0.6, 0.7], [0.8]]
    want = {"generate/min_num_tokens": 1, "generate/max_num_tokens": 3, "generate/avg_num_tokens": 2.0,
            "generate/std_num_tokens": np.std([2, 2, 3, 1]), "generate/avg_tokens_non_zero_rewards": 2.0,
            "generate/avg_tokens_zero_rewards": 0, "generate/avg_assistant_tokens": 2.0, "generate/min_assistant_tokens": 1,
            "generate/max_assistant_tokens": 3, "generate/std_assistant_tokens": np.std([2, 2, 3, 1]),
            "generate/tokens_per_turn_mean": 2.0, "generate/tokens_per_turn_std": np.std([2, 2, 3, 1]),
            "generate/tokens_per_turn_max": 3}
    assert cat["rollout_metrics"].keys() == want.keys()
    for k, v in want.items():
        assert cat["rollout_metrics"][k] == pytest.approx(v), k

    m = U.get_rollout_metrics([[1, 2]] * 4, [1.0] * 4, trajectory_completion_times=[10.0, 20.0, 30.0, 40.0],
                              trajectory_time_splits={"llm": [4.0, 8.0, 12.0, 16.0], "env": [5.0, 10.0, 15.0, 20.0]})
    assert m["generate/trajectory_time_llm_mean"] == 10.0 and m["generate/trajectory_time_llm_max"] == 16.0
    assert m["generate/trajectory_time_llm_p90"] == pytest.approx(np.percentile([4.0, 8.0, 12.0, 16.0], 90))
    assert m["generate/trajectory_time_env_mean"] == 12.5 and m["generate/trajectory_time_completion_max"] == 40.0
    assert m["generate/trajectory_time_other_mean"] == pytest.approx(2.5) and m["generate/trajectory_time_other_max"] == pytest.approx(4.0)

    def timed(times, splits):
        n = len(times)
        return {"prompt_token_ids": [[1]] * n, "response_ids": [[1, 2]] * n, "rewards": [1.0] * n, "loss_masks": [[1, 1]] * n,
                "stop_reasons": ["stop"] * n, "rollout_logprobs": None, "trajectory_generation_times": times,
                "trajectory_time_splits": splits}

    both = U.concatenate_generator_outputs([timed([10.0, 20.0], {"llm": [4.0, 8.0], "env": [5.0, 10.0]}),
                                            timed([30.0, 40.0], {"llm": [12.0, 16.0], "env": [15.0, 20.0]})])
    assert both["trajectory_time_splits"] == {"llm": [4.0, 8.0, 12.0, 16.0], "env": [5.0, 10.0, 15.0, 20.0]}
    assert both["rollout_metrics"]["generate/trajectory_time_llm_p90"] == pytest.approx(np.percentile([4.0, 8.0, 12.0, 16.0], 90))
    assert both["rollout_metrics"]["generate/trajectory_time_other_mean"] == pytest.approx(2.5)
    part = U.concatenate_generator_outputs([timed([10.0], {"llm": [4.0], "env": [5.0]}), timed([30.0], None)])
    assert part["trajectory_time_splits"] is None and "generate/trajectory_time_llm_mean" not in part["rollout_metrics"]
    # environment metrics: a registered class aggregates its own episodes (here: a maximum), others are averaged
    import skyrl_b200.gym as gym
    from skyrl_b200.gym.envs.base_text_env import BaseTextEnv

    class MaxTurns(BaseTextEnv):
        @staticmethod
        def aggregate_metrics(metrics):
            return {"turns": max(m["turns"] for m in metrics), "episodes": len(metrics)}

    gym.register("max_turns_env", MaxTurns, override=True)
    m = U.get_rollout_metrics([[1]] * 3, [0.0, 1.0, 0.0], env_metrics=[{"turns": 2}, {"turns": 4}, {"steps": 6}],
                              env_classes=["max_turns_env", "max_turns_env", "not_registered"])
    assert m["environment/turns"] == 4.0 and m["environment/episodes"] == 2.0 and m["environment/steps"] == 6.0
    assert U.get_rollout_metrics([[1]] * 2, [0.0, 1.0], env_metrics=[{"turns": 2}, {"turns": 4}])["environment/turns"] == 3.0
