"""ReAct agent runner against a scripted inference client."""
import asyncio

from skyrl_b200.agent import AsyncDispatcher, ReActAgent, Tool
from skyrl_b200.utils.tokenizer import SyntheticTokenizer


class _ScriptedClient:
    def __init__(self, tok, scripts):
        self.tok, self.scripts, self.calls = tok, scripts, {}

    async def generate(self, inp):
        sid = inp["session_ids"][0]
        k = self.calls.get(sid, 0)
        self.calls[sid] = k + 1
        text = self.scripts[min(k, len(self.scripts) - 1)]
        ids = self.tok.encode(text)
        return {"response_ids": [ids], "responses": [text], "response_logprobs": [[-0.1] * len(ids)], "stop_reasons": ["stop"]}


def test_react_loop_masks_observations_and_stops_on_answer():
    tok = SyntheticTokenizer(2048)
    scripts = ['I need to add <tool>{"name": "add", "arguments": {"a": 2, "b": 40}}</tool>', "so <answer>42</answer>"]
    agent = ReActAgent(_ScriptedClient(tok, scripts), tok, [Tool("add", lambda a, b: str(a + b), "adds")], max_turns=4)
    r = asyncio.run(agent.run("what is 2+40?", session_id="s"))
    assert r.answer == "42" and r.stop_reason == "answer" and r.turns == 2
    assert len(r.response_ids) == len(r.loss_mask) == len(r.logprobs)
    assert 0 in r.loss_mask and r.loss_mask[0] == 1 and r.loss_mask[-1] == 1
    assert any(m["role"] == "user" and m["content"] == "42" for m in r.messages)
    bad = ReActAgent(_ScriptedClient(tok, ['<tool>{"name": "nope"}</tool>', "<answer>x</answer>"]), tok, [], max_turns=3)
    r2 = asyncio.run(bad.run("t", session_id="s"))
    assert "Unknown tool" in r2.messages[3]["content"] and r2.answer == "x"
    out = asyncio.run(AsyncDispatcher(agent, 2).run(["a", "b", "c"]))
    assert [o.answer for o in out] == ["42"] * 3


def test_tools_python_search_and_exact_match():
    from skyrl_b200.agent import BM25Index, exact_match, make_tool, normalize_answer

    py = make_tool("python", timeout=5.0)
    assert asyncio.run(py(code="print(6 * 7)")).strip() == "42"
    assert "exit code" in asyncio.run(py(code="raise SystemExit(3)"))
    assert "timed out" in asyncio.run(make_tool("python", timeout=0.5)(code="import time; time.sleep(5)"))
    corpus = ["Paris is the capital of France.", "The Nile is a river in Africa.", "Berlin is the capital of Germany."]
    assert BM25Index(corpus).search("capital of Germany", 1) == [corpus[2]]
    s = make_tool("local_search", passages=corpus, top_k=2)
    assert "Nile" in asyncio.run(s(query="river Africa")) and asyncio.run(s(query="zebra")) == "no results"
    assert normalize_answer("The  Eiffel-Tower!") == "eiffel tower"
    assert exact_match("the eiffel tower", ["Eiffel Tower"]) == 1.0 and exact_match(None, ["x"]) == 0.0
    assert asyncio.run(make_tool("finish")(answer="7")) == "<answer>7</answer>"


def test_runner_dispatchers_and_generator_output():
    from skyrl_b200.agent import AgentGenerator, AgentRunner, BaseTask, register_task

    tok = SyntheticTokenizer(2048)
    scripts = ['look it up <tool>{"name": "local_search", "arguments": {"query": "capital of France"}}</tool>',
               "<answer>Paris</answer>"]
    stages = []

    @register_task("traced_qa")
    class Traced(BaseTask):
        def instruction(self):
            return self.instance["question"]

        async def initialize(self):
            stages.append(("init", self.instance["question"]))

        async def evaluate(self, result):
            stages.append(("eval", self.instance["question"]))
            return 1.0 if result.answer == self.instance["answer"] else 0.0

    rows = [{"question": "capital of France?", "answer": "Paris"}, {"question": "capital of Spain?", "answer": "Madrid"}]
    corpus = ["Paris is the capital of France."]
    for disp in ("async_batch", "async_pipeline"):
        stages.clear()
        runner = AgentRunner({"task": "traced_qa", "dispatcher": disp, "num_trajectories": 3, "max_turns": 4,
                              "max_parallel_agents": 2, "max_eval_parallel_agents": 1,
                              "tools": [{"name": "local_search", "passages": corpus}]}, _ScriptedClient(tok, scripts), tok)
        out = asyncio.run(runner.run(rows))
        assert len(out["results"]) == 6 and out["rewards"] == [1.0, 1.0, 1.0, 0.0, 0.0, 0.0]  # instance-major order
        assert sum(1 for s in stages if s[0] == "init") == 6 and sum(1 for s in stages if s[0] == "eval") == 6
        go = AgentRunner.to_generator_output(out)
        assert len(go["response_ids"]) == 6 and go["stop_reasons"] == ["stop"] * 6
        assert all(len(a) == len(b) == len(c) for a, b, c in zip(go["response_ids"], go["loss_masks"], go["rollout_logprobs"]))
        assert go["rollout_metrics"]["agent/avg_turns"] == 2.0 and go["rollout_metrics"]["agent/avg_reward"] == 0.5
    # a failing stage surfaces after the pipeline has drained instead of hanging it
    import pytest

    @register_task("broken")
    class Broken(Traced):
        async def evaluate(self, result):
            raise RuntimeError("scorer down")

    with pytest.raises(RuntimeError, match="scorer down"):
        asyncio.run(AgentRunner({"task": "broken", "dispatcher": "async_pipeline"}, _ScriptedClient(tok, scripts), tok).run(rows[:1]))
    # as the trainer's generator: one trajectory per (already repeated) prompt row
    gen = AgentGenerator({"task": "general_react", "tools": []}, _ScriptedClient(tok, ["<answer>Paris</answer>"]), tok)
    batch = {"prompts": [[{"role": "user", "content": "capital of France?"}]] * 2,
             "env_extras": [{"question": "capital of France?", "answer": "Paris"}, {"question": "capital of France?", "answer": "Rome"}]}
    g = asyncio.run(gen.generate(batch))
    assert g["rewards"] == [1.0, 0.0] and len(g["prompt_token_ids"]) == 2
