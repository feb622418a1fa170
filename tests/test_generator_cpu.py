"""The rollout state machine with scripted engines and environments: exact token ids, loss masks, log-probs, rewards
and stop reasons for single-turn, multi-turn (chat-message and single-assistant-message layouts), step-wise,
re-tokenised (custom chat template) and batched rollouts.  Expectations follow the reference's generator tests
(tests/train/generators/test_skyrl_gym_generator.py) in behaviour; the fixtures here are plain fakes, not mocks."""
import asyncio

import pytest

from skyrl_b200 import gym as skyrl_gym
from skyrl_b200.config.config import GeneratorConfig
from skyrl_b200.gym.envs.base_text_env import BaseTextEnv
from skyrl_b200.train.generators.base import TrajectoryID
from skyrl_b200.train.generators.skyrl_gym_generator import SkyRLGymGenerator
from skyrl_b200.utils.tokenizer import SyntheticTokenizer

EOS = SyntheticTokenizer.eos_token_id  # 1; role markers: 2 user, 3 assistant


class ScriptedClient:
    """Returns the next scripted turn for every prompt of a call and records what it was asked."""

    weight_version = 3

    def __init__(self, turns, logprob=-0.5, stop_reasons=None, routes=False):
        self.turns, self.logprob, self.stop_reasons, self.routes = list(turns), logprob, stop_reasons, routes
        self.calls, self.finished = [], []

    async def generate(self, inp):
        self.calls.append({k: inp.get(k) for k in ("prompt_token_ids", "session_ids", "sampling_params", "cache_salt")})
        k = min(len(self.calls) - 1, len(self.turns) - 1)
        ids = list(self.turns[k])
        n = len(inp["prompt_token_ids"])
        tok = SyntheticTokenizer(1024)
        out = {"responses": [tok.decode(ids, skip_special_tokens=False)] * n, "response_ids": [list(ids) for _ in range(n)],
               "stop_reasons": [(self.stop_reasons or ["stop"] * 99)[k]] * n,
               "response_logprobs": [[self.logprob - 0.01 * j for j in range(len(ids))] for _ in range(n)]
               if self.logprob is not None else None}
        if self.routes:
            import numpy as np

            # one row per token fed through the model: context + generated - 1; the value is the row index
            out["rollout_expert_indices"] = [np.arange(len(p) + len(ids) - 1).reshape(-1, 1, 1).repeat(2, 2)
                                             for p in inp["prompt_token_ids"]]
        return out

    async def finish_session(self, sid):
        self.finished.append(sid)


class ScriptedEnv(BaseTextEnv):
    """``script``: one ``(observation text | None, reward, done)`` per step; records the actions it saw."""

    script = []
    seen = []

    def __init__(self, env_config=None, extras=None):
        super().__init__()
        self.extras = extras or {}
        self.k = 0

    def step(self, action):
        type(self).seen.append(action)
        obs, reward, done = type(self).script[min(self.k, len(type(self).script) - 1)][:3]
        extra = type(self).script[min(self.k, len(type(self).script) - 1)][3:] or [{}]
        self.k += 1
        out = {"observations": [{"role": "user", "content": obs}] if obs else [], "reward": reward, "done": done,
               "metadata": {}}
        out.update(extra[0])
        return out

    def get_metrics(self):
        return {"steps": self.k}


skyrl_gym.register("scripted", ScriptedEnv, override=True)


def _cfg(**kw):
    c = GeneratorConfig()
    c.sampling_params.max_generate_length = 50
    c.max_input_length = 512
    c.batched = False
    c.max_turns = 10
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def _gen(client, script, tokenizer=None, **kw):
    ScriptedEnv.script, ScriptedEnv.seen = script, []
    return SkyRLGymGenerator(_cfg(**kw), None, client, tokenizer or SyntheticTokenizer(1024))


PROMPT = [{"role": "user", "content": "100 101"}]
PROMPT_IDS = [2, 100, 101, EOS, 3]  # user marker, content, end of turn, generation prompt


def _loop(g, **kw):
    return asyncio.run(g.agent_loop(PROMPT, "scripted", {}, max_tokens=50, max_input_length=kw.pop("max_input_length", 512),
                                    **kw))


def test_single_turn_keeps_tokens_logprobs_and_passes_session_and_salt():
    client = ScriptedClient([[10, 11, 12, EOS]])
    g = _gen(client, [(None, 1.0, True)], max_turns=1)
    out = _loop(g, trajectory_id=TrajectoryID("p0", 2))
    assert out.prompt_ids == PROMPT_IDS and out.response_ids == [10, 11, 12, EOS]
    assert out.loss_mask == [1, 1, 1, 1] and out.stop_reason == "stop"
    assert out.rollout_logprobs == pytest.approx([-0.5, -0.51, -0.52, -0.53])
    assert out.reward == 1.0 and out.env_metrics == {"steps": 1}
    call = client.calls[0]
    assert call["prompt_token_ids"] == [PROMPT_IDS] and call["session_ids"] == ["p0_2"]
    assert call["cache_salt"] == "policy@3" and call["sampling_params"]["max_generate_length"] == 50
    assert client.finished == ["p0_2"]
    assert ScriptedEnv.seen == ["10 11 12 1"]


def test_multi_turn_chat_layout_masks_observations_and_places_rewards_at_turn_ends():
    client = ScriptedClient([[10, 11, EOS], [20, 21, 22, EOS]])
    g = _gen(client, [("7 8", 0.3, False), (None, 1.7, True)])
    out = _loop(g)
    obs = [2, 7, 8, EOS, 3]  # user message + generation prompt for the next turn
    assert out.response_ids == [10, 11, EOS] + obs + [20, 21, 22, EOS]
    assert out.loss_mask == [1, 1, 1] + [0] * 5 + [1, 1, 1, 1]
    assert out.reward == pytest.approx([0, 0, 0.3] + [0] * 5 + [0, 0, 0, 1.7])
    assert out.rollout_logprobs == pytest.approx([-0.5, -0.51, -0.52] + [0.0] * 5 + [-0.5, -0.51, -0.52, -0.53])
    # the second request carries the first turn and the observation, token for token
    assert client.calls[1]["prompt_token_ids"] == [PROMPT_IDS + [10, 11, EOS] + obs]


def test_multi_turn_single_assistant_message_drops_inner_eos_and_ends_on_one():
    """use_conversation_multi_turn=false: turns and observations continue one assistant message."""
    client = ScriptedClient([[10, 11, 12, EOS], [10, 11, 12]], logprob=None)
    g = _gen(client, [("77", 0.3, False), (None, 1.7, True)], use_conversation_multi_turn=False)
    out = _loop(g)
    # step 1 (3 tokens, its end-of-sequence token dropped) + observation (1) + step 2 (3) + appended end token
    assert out.response_ids == [10, 11, 12, 77, 10, 11, 12, EOS]
    assert out.loss_mask == [1, 1, 1, 0, 1, 1, 1, 1]
    assert out.reward == pytest.approx([0, 0, 0.3, 0, 0, 0, 0, 1.7])  # the last reward sits on the appended token
    assert out.rollout_logprobs is None and out.stop_reason == "stop"
    assert client.calls[1]["prompt_token_ids"] == [PROMPT_IDS + [10, 11, 12, 77]]


def test_single_assistant_message_keeps_the_sampled_final_eos_with_its_logprob():
    client = ScriptedClient([[10, 11, EOS], [20, EOS]])
    g = _gen(client, [("77", 0.0, False), (None, 1.0, True)], use_conversation_multi_turn=False)
    out = _loop(g)
    assert out.response_ids == [10, 11, 77, 20, EOS] and out.loss_mask == [1, 1, 0, 1, 1]
    assert out.rollout_logprobs == pytest.approx([-0.5, -0.51, 0.0, -0.5, -0.51])
    assert out.reward == pytest.approx([0, 0, 0, 0, 1.0])


def test_context_over_the_limit_ends_the_episode_with_length_and_drops_the_dangling_observation():
    client = ScriptedClient([[10, 11, EOS]] * 5)
    g = _gen(client, [("7 8 9", 0.5, False)] * 5)
    out = _loop(g, max_input_length=len(PROMPT_IDS) + 12)
    # two turns fit (5 + 3 + 6 = 14 <= 17, then 14 + 3 + 6 = 23 > 17 stops before a third request)
    assert len(client.calls) == 2 and out.stop_reason == "length"
    obs = [2, 7, 8, 9, EOS, 3]
    assert out.response_ids == [10, 11, EOS] + obs + [10, 11, EOS]  # ends on generated tokens, not on the observation
    assert out.loss_mask == [1, 1, 1] + [0] * 6 + [1, 1, 1]
    assert out.reward == pytest.approx([0, 0, 0.5] + [0] * 6 + [0, 0, 0.5])


def test_zero_reward_on_non_stop():
    client = ScriptedClient([[10, 11, 12]], stop_reasons=["length"])
    g = _gen(client, [(None, 1.0, True)], max_turns=1, zero_reward_on_non_stop=True)
    out = _loop(g)
    assert out.stop_reason == "length" and out.reward == 0.0


def test_postprocessed_action_replaces_the_tokens_and_gives_up_logprobs():
    client = ScriptedClient([[10, 11, 12, 13, EOS]])
    g = _gen(client, [(None, 1.0, True, {"postprocessed_action": "10 11"})], max_turns=1)
    out = _loop(g)
    assert out.response_ids == [10, 11] and out.loss_mask == [1, 1] and out.rollout_logprobs is None


def test_stop_string_turn_gets_an_untrained_eos_in_chat_layout():
    client = ScriptedClient([[10, 11], [20, EOS]])
    g = _gen(client, [("7", 0.0, False), (None, 1.0, True)])
    out = _loop(g, sampling_params={"stop": ["11"], "max_generate_length": 50})
    obs = [2, 7, EOS, 3]
    assert out.response_ids == [10, 11, EOS] + obs + [20, EOS]
    assert out.loss_mask == [1, 1, 0] + [0] * 4 + [1, 1]  # the appended token is context, not a sampled action
    assert out.rollout_logprobs == pytest.approx([-0.5, -0.51, 0.0] + [0.0] * 4 + [-0.5, -0.51])


def test_step_wise_gives_one_row_per_turn_with_the_full_context_as_prompt():
    client = ScriptedClient([[10, 11, EOS], [20, 21, EOS]])
    g = _gen(client, [("7 8", 0.25, False), (None, 1.0, True)], step_wise_trajectories=True)
    steps = _loop(g)
    assert isinstance(steps, list) and len(steps) == 2
    obs = [2, 7, 8, EOS, 3]
    s0, s1 = steps
    assert s0.prompt_ids == PROMPT_IDS and s0.response_ids == [10, 11, EOS] + obs
    assert s0.loss_mask == [1, 1, 1] + [0] * 5 and s0.reward == pytest.approx([0, 0, 0.25] + [0] * 5)
    assert not s0.is_last_step and s0.env_metrics == {}
    assert s1.prompt_ids == PROMPT_IDS + [10, 11, EOS] + obs and s1.response_ids == [20, 21, EOS]
    assert s1.loss_mask == [1, 1, 1] and s1.reward == pytest.approx([0, 0, 1.0]) and s1.is_last_step
    assert s1.env_metrics == {"steps": 2}


def test_generate_flattens_step_wise_rows_and_repeats_trajectory_ids():
    client = ScriptedClient([[10, EOS], [20, EOS]])
    g = _gen(client, [("7", 0.0, False), (None, 1.0, True)], step_wise_trajectories=True)
    tids = [TrajectoryID("a", 0), TrajectoryID("b", 0)]
    out = asyncio.run(g.generate({"prompts": [PROMPT, PROMPT], "env_classes": ["scripted"] * 2, "env_extras": [{}, {}],
                                  "trajectory_ids": tids}))
    assert len(out["response_ids"]) == 4 and out["is_last_step"] == [False, True, False, True]
    assert [t.instance_id for t in out["trajectory_ids"]] == ["a", "a", "b", "b"]
    assert out["rollout_metrics"]["generate/max_num_tokens"] >= 2


def test_overlong_filtering_zeroes_the_mask_of_responses_without_eos():
    client = ScriptedClient([[10, 11, 12]])
    g = _gen(client, [(None, 1.0, True)], max_turns=1, apply_overlong_filtering=True)
    out = asyncio.run(g.generate({"prompts": [PROMPT], "env_classes": ["scripted"], "env_extras": [{}]}))
    assert out["loss_masks"] == [[0, 0, 0]] and out["response_ids"] == [[10, 11, 12]]
    client2 = ScriptedClient([[10, 11, EOS]])
    g2 = _gen(client2, [(None, 1.0, True)], max_turns=1, apply_overlong_filtering=True)
    out2 = asyncio.run(g2.generate({"prompts": [PROMPT], "env_classes": ["scripted"], "env_extras": [{}]}))
    assert out2["loss_masks"] == [[1, 1, 1]]


def test_batched_single_turn_sends_one_request_and_scores_each_row():
    client = ScriptedClient([[10, 11, EOS]])
    g = _gen(client, [(None, 1.0, True)], max_turns=1, batched=True)
    out = asyncio.run(g.generate({"prompts": [PROMPT] * 3, "env_classes": ["scripted"] * 3, "env_extras": [{}] * 3}))
    assert len(client.calls) == 1 and len(client.calls[0]["prompt_token_ids"]) == 3
    assert out["response_ids"] == [[10, 11, EOS]] * 3 and out["rewards"] == [1.0] * 3
    assert out["rollout_logprobs"][0] == pytest.approx([-0.5, -0.51, -0.52]) and out["stop_reasons"] == ["stop"] * 3
    assert out["rollout_expert_indices"] is None


def test_routes_of_the_newest_turn_cover_the_whole_trajectory():
    client = ScriptedClient([[10, 11, EOS], [20, 21, EOS]], routes=True)
    g = _gen(client, [("7", 0.0, False), (None, 1.0, True)])
    out = _loop(g)
    total = len(out.prompt_ids) + len(out.response_ids)
    r = out.rollout_expert_indices
    assert r.shape == (total - 1, 1, 2) and r[:, 0, 0].tolist() == list(range(total - 1))
    # a re-tokenised action keeps only the context's rows: what the model saw afterwards is not what was routed
    client2 = ScriptedClient([[10, 11, 12, EOS]], routes=True)
    g2 = _gen(client2, [(None, 1.0, True, {"postprocessed_action": "10"})], max_turns=1)
    out2 = _loop(g2)
    assert out2.rollout_expert_indices.shape[0] == len(PROMPT_IDS)


def _char_tokenizer():
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    specials = ["<pad>", "<|im_start|>", "<|im_end|>"]
    vocab = {t: i for i, t in enumerate(specials + [chr(c) for c in range(32, 127)] + ["\n"])}
    tk = Tokenizer(models.WordLevel(vocab, unk_token="<pad>"))
    tk.pre_tokenizer = pre_tokenizers.Split("", "isolated")
    tk.decoder = decoders.Fuse()
    tok = PreTrainedTokenizerFast(tokenizer_object=tk, pad_token="<pad>", eos_token="<|im_end|>",
                                  additional_special_tokens=["<|im_start|>"])
    from skyrl_b200.train.generators.utils import CUSTOM_CHAT_TEMPLATES

    tok.chat_template = CUSTOM_CHAT_TEMPLATES["chatml_no_default_system"]
    return tok


class TextClient:
    """Engine fake for the re-tokenising path: answers with text, tokenised by the tokenizer under test."""

    weight_version = 0

    def __init__(self, tok, answers):
        self.tok, self.answers, self.prompts = tok, list(answers), []

    async def generate(self, inp):
        self.prompts.append(self.tok.decode(inp["prompt_token_ids"][0]))
        text = self.answers[len(self.prompts) - 1] + "<|im_end|>"
        ids = self.tok.encode(text, add_special_tokens=False)
        return {"responses": [text], "response_ids": [ids], "stop_reasons": ["stop"], "response_logprobs": None}

    async def finish_session(self, sid):
        pass


def test_custom_chat_template_retokenises_the_history_and_masks_by_generation_blocks():
    from skyrl_b200.config.config import ChatTemplateConfig

    tok = _char_tokenizer()
    client = TextClient(tok, ["<think>a</think>X", "Y"])
    g = _gen(client, [("obs", 0.2, False), ("bye", 0.9, True)], tokenizer=tok,
             chat_template=ChatTemplateConfig(source="name", name_or_path="qwen3_without_thinking"))
    out = asyncio.run(g.agent_loop([{"role": "user", "content": "hi"}], "scripted", {}, 50, 4096))
    # every request is the whole history through the custom template, with the generation prompt
    assert client.prompts[0] == "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    assert client.prompts[1] == ("<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\nX<|im_end|>\n"
                                 "<|im_start|>user\nobs<|im_end|>\n<|im_start|>assistant\n")
    text = tok.decode(out.response_ids)
    # the response drops the last observation and the earlier turn's thinking (that is what this template does)
    assert text == "<|im_start|>assistant\nX<|im_end|>\n<|im_start|>user\nobs<|im_end|>\n<|im_start|>assistant\nY<|im_end|>\n"
    trained = "".join(tok.decode([i]) for i, m in zip(out.response_ids, out.loss_mask) if m)
    assert trained == "X<|im_end|>Y<|im_end|>"
    assert out.reward == pytest.approx(0.9) and out.rollout_logprobs is None and out.stop_reason == "stop"
    assert ScriptedEnv.seen == ["<think>a</think>X<|im_end|>", "Y<|im_end|>"]


def test_chat_layout_with_a_real_fast_tokenizer_appends_observations_token_for_token():
    """The default (token-in, token-out) path against a ``transformers`` tokenizer, whose ``apply_chat_template`` may
    return an encoding object rather than a list."""
    tok = _char_tokenizer()
    client = TextClient(tok, ["A", "B"])
    g = _gen(client, [("obs", 0.0, False), (None, 1.0, True)], tokenizer=tok)
    out = asyncio.run(g.agent_loop([{"role": "user", "content": "hi"}], "scripted", {}, 50, 4096))
    assert tok.decode(out.prompt_ids) == "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    assert tok.decode(out.response_ids) == "A<|im_end|>\n<|im_start|>user\nobs<|im_end|>\n<|im_start|>assistant\nB<|im_end|>"
    trained = "".join(tok.decode([i]) for i, m in zip(out.response_ids, out.loss_mask) if m)
    assert trained == "A<|im_end|>B<|im_end|>"
    # the second request is the first one plus exactly the response tokens so far
    assert client.prompts[1] == tok.decode(out.prompt_ids) + "A<|im_end|>\n<|im_start|>user\nobs<|im_end|>\n<|im_start|>assistant\n"


def _scripted_chat_server(tok, turns, rewrite_after=None):
    """An OpenAI-style endpoint that answers the k-th request with ``turns[k]`` (token ids), templating the prompt the
    way the real server does."""
    from fastapi import FastAPI, Request

    from skyrl_b200.inference.server import ServerThread
    from skyrl_b200.utils.tokenizer import chat_template_ids

    app, seen = FastAPI(), []

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        body = await request.json()
        seen.append(body)
        ids = turns[min(len(seen) - 1, len(turns) - 1)]
        msgs = body["messages"]
        if rewrite_after is not None and len(seen) > rewrite_after:
            msgs = [{"role": "system", "content": "999"}] + msgs
        p = chat_template_ids(tok, msgs, add_generation_prompt=True)
        return {"choices": [{"index": 0, "message": {"role": "assistant", "content": tok.decode(ids)},
                             "finish_reason": "stop" if ids[-1] == EOS else "length", "token_ids": ids,
                             "logprobs": {"content": [{"logprob": -0.25 * (j + 1)} for j in range(len(ids))]}}],
                "prompt_token_ids": p}

    return ServerThread(app).start(), seen


class _Endpoint:
    def __init__(self, url):
        self.url = url

    def get_endpoint_url(self):
        return self.url


def test_chat_protocol_generator_builds_trajectories_from_the_tokens_the_endpoint_reports():
    from examples.train_integrations.openai_chat.chat_generator import ChatCompletionsGenerator

    tok = SyntheticTokenizer(1024)
    ScriptedEnv.script, ScriptedEnv.seen = [("7 8", 0.3, False), (None, 1.0, True)], []
    srv, seen = _scripted_chat_server(tok, [[10, 11, EOS], [20, 21, EOS]])
    try:
        g = ChatCompletionsGenerator(_cfg(), None, _Endpoint(srv.url), tok)
        out = asyncio.run(g.generate({"prompts": [PROMPT], "env_classes": ["scripted"], "env_extras": [{}],
                                      "sampling_params": {"temperature": 0.0, "max_generate_length": 8}}))
    finally:
        srv.stop()
    obs = [2, 7, 8, EOS, 3]
    assert out["prompt_token_ids"] == [PROMPT_IDS]
    assert out["response_ids"] == [[10, 11, EOS] + obs + [20, 21, EOS]]
    assert out["loss_masks"] == [[1, 1, 1] + [0] * 5 + [1, 1, 1]]
    assert out["rewards"][0] == pytest.approx([0, 0, 0.3] + [0] * 5 + [0, 0, 1.0])
    assert out["rollout_logprobs"][0] == pytest.approx([-0.25, -0.5, -0.75] + [0.0] * 5 + [-0.25, -0.5, -0.75])
    assert seen[0]["temperature"] == 0.0 and seen[0]["max_tokens"] == 8 and seen[0]["logprobs"] is True
    assert [m["role"] for m in seen[1]["messages"]] == ["user", "assistant", "user"]

    # a turn cut by the length limit has no end-of-turn token of its own: the one the template adds shows up between the
    # turns and is context, not a sampled action
    ScriptedEnv.script, ScriptedEnv.seen = [("7 8", 0.3, False), (None, 1.0, True)], []
    srv, seen = _scripted_chat_server(tok, [[10, 11], [20, 21, EOS]])
    try:
        g = ChatCompletionsGenerator(_cfg(), None, _Endpoint(srv.url), tok)
        out = asyncio.run(g.generate({"prompts": [PROMPT], "env_classes": ["scripted"], "env_extras": [{}]}))
    finally:
        srv.stop()
    assert out["response_ids"] == [[10, 11, EOS] + obs + [20, 21, EOS]]
    assert out["loss_masks"] == [[1, 1, 0] + [0] * 5 + [1, 1, 1]]
    assert out["rollout_logprobs"][0] == pytest.approx([-0.25, -0.5, 0.0] + [0.0] * 5 + [-0.25, -0.5, -0.75])

    # a scaffold that rewrites history (here: a system message appears from the second request on) breaks the token
    # chain: the trajectory is rebuilt from the messages and gives up its log-probs
    ScriptedEnv.script, ScriptedEnv.seen = [("7 8", 0.3, False), (None, 1.0, True)], []
    srv, seen = _scripted_chat_server(tok, [[10, 11, EOS], [20, 21, EOS]], rewrite_after=1)
    try:
        g = ChatCompletionsGenerator(_cfg(), None, _Endpoint(srv.url), tok)
        out = asyncio.run(g.generate({"prompts": [PROMPT], "env_classes": ["scripted"], "env_extras": [{}]}))
    finally:
        srv.stop()
    assert out["rollout_logprobs"] is None
    assert out["response_ids"] == [[3, 10, 11, EOS, 2, 7, 8, EOS, 3, 20, 21, EOS]]
    assert out["loss_masks"] == [[0, 1, 1, 1, 0, 0, 0, 0, 0, 1, 1, 1]]
    assert out["rewards"] == [pytest.approx(1.3)]  # one scalar for the rebuilt trajectory


def test_step_wise_evaluation_scores_trajectories_by_their_last_step(tmp_path):
    from types import SimpleNamespace

    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.train.evaluate import evaluate

    cfg = SkyRLTrainConfig.from_cli_overrides([
        "generator.step_wise_trajectories=true", "generator.batched=false", "generator.max_turns=3",
        "generator.eval_n_samples_per_prompt=2", "environment.env_class=scripted", "trainer.eval_batch_size=8",
        f"trainer.export_path={tmp_path}", "trainer.dump_eval_results=false", "trainer.print_example_interval=0"])
    client = ScriptedClient([[10, EOS], [20, EOS]])
    ScriptedEnv.script, ScriptedEnv.seen = [("7", 0.0, False), (None, 1.0, True)], []
    g = SkyRLGymGenerator(cfg.generator, None, client, SyntheticTokenizer(1024))
    items = [{"prompt": PROMPT, "uid": f"p{i}", "env_class": "scripted", "env_extras": {"data_source": "toy"}}
             for i in range(3)]
    m = asyncio.run(evaluate(SimpleNamespace(items=items), g, cfg, 0, SyntheticTokenizer(1024)))
    # 3 prompts x 2 samples, two steps each; every trajectory ends with reward 1 on its last step
    assert m["eval/all/avg_score"] == pytest.approx(1.0) and m["eval/all/pass_at_2"] == pytest.approx(1.0)
    assert m["eval/toy/avg_score"] == pytest.approx(1.0)


class _TextTok(SyntheticTokenizer):
    """Synthetic tokenizer that can carry arbitrary text: unknown strings get ids from a growing table."""

    def __init__(self):
        super().__init__(1 << 20)
        self.table, self.back = {}, {}

    def encode(self, text, add_special_tokens=False):
        out = []
        for line in [text]:
            if line not in self.table:
                i = 1000 + len(self.table)
                self.table[line], self.back[i] = i, line
            out.append(self.table[line])
        return out

    def decode(self, ids, skip_special_tokens=True):
        return "".join(self.back.get(int(i), "") for i in ids)


class _PolicyScript:
    """Answers by looking at the last user text of the request: a stand-in for a policy that writes REPL code."""

    weight_version = 0

    def __init__(self, tok, rules):
        self.tok, self.rules, self.requests = tok, rules, []

    async def generate(self, inp):
        outs = []
        for ids in inp["prompt_token_ids"]:
            text = self.tok.decode(ids)
            self.requests.append(text)
            reply = next(r for key, r in self.rules if key in text)
            if callable(reply):
                reply = reply(text)
            outs.append(reply)
        return {"responses": outs, "response_ids": [self.tok.encode(o) + [EOS] for o in outs],
                "stop_reasons": ["stop"] * len(outs), "response_logprobs": None}

    async def finish_session(self, sid):
        pass


def test_rlm_generator_lets_the_repl_query_the_policy_and_spawn_child_episodes():
    from types import SimpleNamespace

    from skyrl_b200.train.generators.rlm_generator import RLMGenerator

    tok = _TextTok()
    # the parent: turn 1 asks a sub-agent and a plain LM call, turn 2 answers with what came back
    parent1 = "```repl\na = rlm_query('CHILD: how many legs has a spider')\nb = llm_query('PLAIN: say hi')\nprint(a, '|', b)\n```"
    rules = [
        ("REPL output 1:\n8 | hi there", "FINAL(8)"),                      # parent, turn 2
        ("CHILD: how many legs has a spider\nassistant-turn-2", "never"),  # (unused)
        ("PLAIN: say hi", "hi there"),                                      # llm_query
        ("`context` is a str of length 33", "FINAL(8)"),                    # the child episode (its context is the prompt)
        ("What do spiders have?", parent1),                                 # parent, turn 1
    ]
    client = _PolicyScript(tok, rules)
    g = RLMGenerator(_cfg(max_turns=4), SimpleNamespace(max_env_workers=4), client, tok, max_depth=1)
    extras = {"reward_spec": {"ground_truth": "8"}, "context": "long document about arachnids"}
    out = asyncio.run(g.agent_loop([{"role": "user", "content": "What do spiders have?"}], "rlm", extras, 64, 4096))
    assert out.reward == pytest.approx([0.0] * (len(out.response_ids) - 1) + [1.0]) and out.stop_reason == "stop"
    assert g.subcall_stats == {"lm_queries": 1, "child_episodes": 1}
    assert out.env_metrics["final_answer"] == "8" and out.env_metrics["depth"] == 0
    # the child saw its own system prompt and context note, not the parent's document
    child_req = next(r for r in client.requests if "`context` is a str of length 33" in r)
    assert "CHILD: how many legs has a spider" in child_req and "arachnids" not in child_req
    # beyond max_depth a recursive call degrades to a plain generation
    g0 = RLMGenerator(_cfg(max_turns=4), SimpleNamespace(max_env_workers=4), _PolicyScript(tok, [
        ("REPL output 1:\nplain answer", "FINAL(done)"), ("CHILD: q", "plain answer"),
        ("Question?", "```repl\nprint(rlm_query('CHILD: q'))\n```")]), tok, max_depth=0)
    out = asyncio.run(g0.agent_loop([{"role": "user", "content": "Question?"}], "rlm",
                                    {"reward_spec": {"ground_truth": "done"}, "context": "c"}, 64, 4096))
    assert out.env_metrics["final_answer"] == "done" and g0.subcall_stats == {"lm_queries": 1, "child_episodes": 0}
